"""GPU: the allocation-free weight-gradient entry point against the regular one.

akr_matmul_at_b_noalloc serves hosts that may not allocate device memory at call time (their own
pool owns all of HBM, or they cannot afford the synchronisation an allocation implies). It keeps its
scratch in a fixed array inside the library. This file is collected last on purpose: if it fails,
`pytest -x` has already run every other test. It calls through the C ABI only.
"""
import ctypes as C

import numpy as np
import pytest

from util import uniform, normal, rel_fro, TOL_TF32
from aakaar_b200 import cabi
from aakaar_b200.cabi import DeviceArray as DA, MODE_TF32

pytestmark = pytest.mark.gpu


def at_b(fn_name, A, B, with_mode):
    lib = cabi.lib()
    out = DA((A.shape[1], B.shape[1]))
    va, vb, vc = A.view(), B.view(), out.view()
    fn = getattr(lib, fn_name)
    rc = fn(C.byref(va), C.byref(vb), C.byref(vc), MODE_TF32, None) if with_mode else \
        fn(C.byref(va), C.byref(vb), C.byref(vc), None)
    cabi.check(rc)
    return out


def test_noalloc_matches_regular_entry_point_twice_in_a_row():
    # A^T . B with a long contraction and few output tiles: the contraction is split across CTAs,
    # so the fixed scratch (partial tiles + counters) is really used.
    k, m, n = 4096, 64, 512
    a, b = uniform((k, m), 71), normal((k, n), 72)
    A, B = DA.from_numpy(a), DA.from_numpy(b)
    want = at_b("akr_matmul_at_b", A, B, True).to_numpy()
    ref = a.astype(np.float64).T @ b.astype(np.float64)
    assert rel_fro(want, ref) < TOL_TF32
    ws = C.c_size_t()
    cabi.lib().akr_workspace_bytes(C.byref(ws))
    before = ws.value
    for _ in range(2):   # second call reuses the array the first one left behind
        got = at_b("akr_matmul_at_b_noalloc", A, B, False).to_numpy()
        assert rel_fro(got, want) < TOL_TF32
        assert rel_fro(got, ref) < TOL_TF32
    cabi.lib().akr_workspace_bytes(C.byref(ws))
    assert ws.value == before            # the library's allocated workspace did not grow
    # different shape right after, on the same scratch (single output tile column, ragged sizes)
    a2, b2 = uniform((2052, 100), 73), normal((2052, 40), 74)
    A2, B2 = DA.from_numpy(a2), DA.from_numpy(b2)
    got2 = at_b("akr_matmul_at_b_noalloc", A2, B2, False).to_numpy()
    assert rel_fro(got2, at_b("akr_matmul_at_b", A2, B2, True).to_numpy()) < TOL_TF32


def test_noalloc_rejects_what_does_not_fit():
    lib = cabi.lib()
    # The limit is 8 MiB of partial tiles. 1280 x 896 outputs: any split count >= 2 needs at least
    # 2 x 1280 x 896 x 4 B = 8.75 MiB, and this contraction (256 k-blocks, 40 output tiles) is always split.
    k, m, n = 8192, 1280, 896
    A, B, out = DA((k, m)), DA((k, n)), DA((m, n))
    va, vb, vc = A.view(), B.view(), out.view()
    rc = lib.akr_matmul_at_b_noalloc(C.byref(va), C.byref(vb), C.byref(vc), None)
    assert rc == cabi.ERR_INVALID
    msg = lib.akr_last_error()
    assert b"fixed scratch" in msg and b"akr_matmul_at_b" in msg and b"8388608 bytes" in msg
    # an operand that would need a packed copy (row stride not a multiple of 4 elements)
    big = DA((70, 45))
    v = big.as_strided((64, 40), (45, 1))
    vb2 = DA((64, 32))
    out2 = DA((40, 32))
    va, vb, vc = v.view(), vb2.view(), out2.view()
    rc = lib.akr_matmul_at_b_noalloc(C.byref(va), C.byref(vb), C.byref(vc), None)
    assert rc == cabi.ERR_INVALID and b"readable in place" in lib.akr_last_error()
    # shape errors use the same texts as the regular entry point
    va, vb, vc = DA((8, 4)).view(), DA((9, 4)).view(), DA((4, 4)).view()
    assert lib.akr_matmul_at_b_noalloc(C.byref(va), C.byref(vb), C.byref(vc), None) == cabi.ERR_INVALID
    assert b"inner dimensions must match" in lib.akr_last_error()
    # null data pointers and an output row stride shorter than a row are refused before anything is launched
    good = [DA((64, 32)), DA((64, 48)), DA((32, 48))]
    for bad in range(3):
        views = [x.view() for x in good]
        views[bad].data = None
        rc = lib.akr_matmul_at_b_noalloc(C.byref(views[0]), C.byref(views[1]), C.byref(views[2]), None)
        assert rc == cabi.ERR_INVALID and b"null data pointer" in lib.akr_last_error()
    views = [x.view() for x in good]
    views[2].stride[0] = 40
    rc = lib.akr_matmul_at_b_noalloc(C.byref(views[0]), C.byref(views[1]), C.byref(views[2]), None)
    assert rc == cabi.ERR_INVALID and b"row stride" in lib.akr_last_error()


def test_noalloc_just_under_the_limit_matches_regular_entry_point():
    # 512 x 800 outputs over a 4096-deep contraction: 16 output tiles, which the planner splits five ways
    # on a 148-SM GPU -> 5 x 512 x 800 x 4 B = 8 192 000 B of partial tiles, just under the 8 388 608 B limit.
    # (On a GPU where the planner picks a count that does not fit, the call is refused with the limit in
    # its message; the regular entry point is the documented fallback and nothing is compared.)
    k, m, n = 4096, 512, 800
    a, b = uniform((k, m), 75), normal((k, n), 76)
    A, B = DA.from_numpy(a), DA.from_numpy(b)
    lib = cabi.lib()
    out = DA((m, n))
    va, vb, vc = A.view(), B.view(), out.view()
    rc = lib.akr_matmul_at_b_noalloc(C.byref(va), C.byref(vb), C.byref(vc), None)
    if rc == cabi.ERR_INVALID:
        assert b"fixed scratch" in lib.akr_last_error()
        pytest.skip("the planner chose more than two splits for this shape on this GPU")
    cabi.check(rc)
    want = at_b("akr_matmul_at_b", A, B, True).to_numpy()
    assert rel_fro(out.to_numpy(), want) < TOL_TF32


def test_noalloc_abort_is_reported_by_synchronize():
    # Failure path without faulting the GPU: the load warp never signals, every in-kernel wait runs out
    # after 30 ms, the kernel stops cleanly and the next akr_synchronize() reports AKR_ERR_ABORTED once.
    lib = cabi.lib()
    k, m, n = 4096, 64, 512
    a, b = uniform((k, m), 77), normal((k, n), 78)
    A, B = DA.from_numpy(a), DA.from_numpy(b)
    cabi.synchronize()
    try:
        cabi.check(lib.akr_debug_configure(16, 30))
        out = DA((m, n))
        va, vb, vc = A.view(), B.view(), out.view()
        cabi.check(lib.akr_matmul_at_b_noalloc(C.byref(va), C.byref(vb), C.byref(vc), None))
        with pytest.raises(cabi.AkrError) as e:
            cabi.synchronize()
        assert e.value.code == cabi.ERR_ABORTED
        cabi.synchronize()   # reported once, then clear
    finally:
        cabi.check(lib.akr_debug_configure(0, 0))
    # the shared scratch (tile counters left mid-way by the aborted launch) is usable again
    got = at_b("akr_matmul_at_b_noalloc", A, B, False).to_numpy()
    assert rel_fro(got, a.astype(np.float64).T @ b.astype(np.float64)) < TOL_TF32
