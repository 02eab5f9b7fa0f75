"""CPU: the C-ABI library loads, exports every declared symbol, and its host-only logic works."""
import ctypes as C
import os
import re

import pytest

from util import ROOT
from aakaar_b200 import cabi


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "akr_b200.h")).read()
    return sorted(set(re.findall(r"AKR_API[^;]*?\b(akr_\w+)\s*\(", text)))


def test_header_declares_entry_points():
    syms = declared_symbols()
    for must in ("akr_matmul_fwd", "akr_matmul_bwd", "akr_matmul_a_bt", "akr_matmul_at_b", "akr_set_tf32",
                 "akr_get_tf32", "akr_synchronize", "akr_alloc", "akr_free", "akr_last_error"):
        assert must in syms
    assert len(syms) >= 35


def test_library_exports_every_declared_symbol():
    lib = cabi.lib()
    for s in declared_symbols():
        assert hasattr(lib, s), f"libakr_b200.so does not export {s}"


def test_no_torch_or_cublas_dependency():
    # The product library must stand alone: no PyTorch, cuBLAS or cuDNN in its dynamic dependencies.
    import subprocess
    so = os.path.join(ROOT, "aakaar_b200", "lib", "libakr_b200.so")
    out = subprocess.run(["readelf", "-d", so], capture_output=True, text=True).stdout
    needed = re.findall(r"NEEDED.*\[(.*?)\]", out)
    for n in needed:
        assert not re.search(r"torch|cublas|cudnn|c10", n), n


def _view(shape, strides=None):
    v = cabi.View()
    v.data = 16  # never dereferenced by the planner
    v.ndim = len(shape)
    v.dtype = 0
    acc, st = 1, []
    for d in reversed(shape):
        st.append(acc)
        acc *= d
    st = list(reversed(st)) if strides is None else strides
    for i, (d, s) in enumerate(zip(shape, st)):
        v.shape[i], v.stride[i] = d, s
    return v


def _plan(sa, sb):
    lib = cabi.lib()
    out = (C.c_int64 * 10)()
    nd = C.c_int32()
    a, b = _view(sa), _view(sb)
    rc = lib.akr_matmul_plan(C.byref(a), C.byref(b), out, C.byref(nd))
    return rc, tuple(out[i] for i in range(nd.value)), lib.akr_last_error().decode()


def test_planner_broadcast_rules_match_reference():
    assert _plan((3, 1, 5, 7), (2, 7, 4))[:2] == (0, (3, 2, 5, 4))
    assert _plan((2, 3, 8), (8, 5))[:2] == (0, (2, 3, 5))
    assert _plan((64, 8, 512, 64), (1, 8, 64, 512))[:2] == (0, (64, 8, 512, 512))
    assert _plan((512, 512), (512, 512))[:2] == (0, (512, 512))


def test_planner_errors_match_reference_texts():
    rc, _, msg = _plan((2, 3), (4, 2))
    assert rc == cabi.ERR_INVALID and msg.startswith("Shape mismatch: inner dimensions must match")
    rc, _, msg = _plan((2, 2, 3), (3, 3, 2))
    assert rc == cabi.ERR_INVALID and msg == "Batch dimensions are not broadcastable for matmul"
    rc, _, msg = _plan((3,), (3, 2))
    assert rc == cabi.ERR_INVALID and msg == "matmul requires tensors with at least 2 dimensions"


def test_tf32_switch_is_global_and_defaults_off():
    lib = cabi.lib()
    prev = lib.akr_get_tf32()
    lib.akr_set_tf32(1)
    assert lib.akr_get_tf32() == 1
    lib.akr_set_tf32(0)
    assert lib.akr_get_tf32() == 0
    lib.akr_set_tf32(prev)
    lib.akr_set_cudnn_tf32(1)
    assert lib.akr_get_cudnn_tf32() == 1
    lib.akr_set_cudnn_tf32(0)


def test_compute_fails_loudly_without_gpu():
    lib = cabi.lib()
    if lib.akr_device_count() > 0:
        pytest.skip("a GPU is present")
    p = C.POINTER(C.c_float)()
    assert lib.akr_alloc(16, C.byref(p)) == cabi.ERR_NOGPU
    assert b"no CPU path" in lib.akr_last_error()
    a, b, c = _view((4, 4)), _view((4, 4)), _view((4, 4))
    assert lib.akr_matmul_fwd(C.byref(a), C.byref(b), None, C.byref(c), 1, None) == cabi.ERR_NOGPU
    assert lib.akr_synchronize() == cabi.ERR_NOGPU
