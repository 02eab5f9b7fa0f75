"""Shared helpers of the test-suite: seeded inputs, error metric, library loading."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def uniform(shape, seed):
    """float32 i.i.d. uniform[-1, 1) from numpy's PCG64 generator."""
    g = np.random.Generator(np.random.PCG64(seed))
    return (g.random(shape, dtype=np.float64) * 2.0 - 1.0).astype(np.float32)


def normal(shape, seed, sigma=1.0):
    g = np.random.Generator(np.random.PCG64(seed))
    return (g.standard_normal(shape) * sigma).astype(np.float32)


def rel_fro(x, ref):
    x = np.asarray(x, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    den = np.linalg.norm(ref.ravel())
    return float(np.linalg.norm((x - ref).ravel()) / (den if den > 0 else 1.0))


# Tolerances of the path (relative Frobenius error against the reference's fp32 CPU result).
TOL_FP32 = 1e-5   # 3xTF32 mode, set_tf32(False)
TOL_TF32 = 2e-3   # TF32 mode, set_tf32(True)


def load_golden():
    import json
    data = np.load(os.path.join(GOLDEN, "ref_vectors.npz"))
    with open(os.path.join(GOLDEN, "ref_vectors.json")) as f:
        meta = json.load(f)
    return data, meta
