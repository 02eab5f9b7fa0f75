"""GPU: the drop-in replacement of the reference's src/matmul_kernel.cu, compiled against the reference's own
Tensor / allocator headers (oracle/integration/, prebuilt into oracle/_ref/libakr_dropin.so where the reference
checkout exists), driven through the three entry points the reference's binding layer calls."""
import ctypes as C
import os

import numpy as np
import pytest

from util import ROOT, uniform, rel_fro, TOL_FP32, TOL_TF32

pytestmark = pytest.mark.gpu
LIB = os.path.join(ROOT, "oracle", "_ref", "libakr_dropin.so")


def run(lib, which, tf32, a, b, transpose_a=False):
    ash = (C.c_int * a.ndim)(*a.shape)
    bsh = (C.c_int * b.ndim)(*b.shape)
    cap = 1 << 24
    out = np.empty(cap, np.float32)
    osh, ond = (C.c_int * 8)(), C.c_int(0)
    err = C.create_string_buffer(512)
    rc = lib.stub_run(which, int(tf32), int(transpose_a), a.ctypes.data_as(C.c_void_p), ash, a.ndim,
                      b.ctypes.data_as(C.c_void_p), bsh, b.ndim, out.ctypes.data_as(C.c_void_p), cap, osh, C.byref(ond),
                      err, 512)
    if rc != 0:
        return rc, err.value.decode()
    shape = tuple(osh[i] for i in range(ond.value))
    return 0, out[:int(np.prod(shape))].reshape(shape).copy()


def test_drop_in_entry_points_with_the_reference_tensor_type():
    if not os.path.exists(LIB):
        pytest.skip("oracle/_ref/libakr_dropin.so was not prebuilt (needs the reference checkout at build time)")
    from aakaar_b200 import cabi
    if cabi.lib().akr_device_count() <= 0:
        pytest.skip("no GPU")
    lib = C.CDLL(LIB)
    for tf32, tol in ((False, TOL_FP32), (True, TOL_TF32)):
        a, b = uniform((300, 200), 1), uniform((200, 260), 2)
        rc, c = run(lib, 0, tf32, a, b)
        assert rc == 0 and rel_fro(c, a.astype(np.float64) @ b.astype(np.float64)) < tol
        # N-D with broadcast batch dims, one launch instead of one cublasSgemm per batch index
        a3, b3 = uniform((3, 1, 70, 40), 3), uniform((2, 40, 50), 4)
        rc, c3 = run(lib, 0, tf32, a3, b3)
        assert rc == 0 and c3.shape == (3, 2, 70, 50)
        assert rel_fro(c3, a3.astype(np.float64) @ b3.astype(np.float64)) < tol
        # the two backward products of the 2-D path
        dc = uniform((300, 260), 5)
        rc, da = run(lib, 1, tf32, dc, b)                     # dC . B^T
        assert rc == 0 and rel_fro(da, dc.astype(np.float64) @ b.astype(np.float64).T) < tol
        rc, db = run(lib, 2, tf32, a, dc)                     # A^T . dC
        assert rc == 0 and rel_fro(db, a.astype(np.float64).T @ dc.astype(np.float64)) < tol
        # a transposed VIEW of the reference's Tensor: the stock kernel raises "requires contiguous tensors"
        at = uniform((200, 300), 6)
        rc, ct = run(lib, 0, tf32, at, b, transpose_a=True)
        assert rc == 0 and rel_fro(ct, at.astype(np.float64).T @ b.astype(np.float64)) < tol
    # errors come back as the reference's exception classes (1 = std::invalid_argument) with its texts
    rc, msg = run(lib, 0, False, uniform((4, 5), 7), uniform((6, 4), 8))
    assert rc == 1 and "inner dimensions must match" in msg
    rc, msg = run(lib, 0, False, uniform((2, 4, 5), 7), uniform((3, 5, 4), 8))
    assert rc == 1 and "not broadcastable" in msg
