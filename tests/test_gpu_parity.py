"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle on the same
seeded inputs, against the committed vectors of the reference's own build, and at full benchmark
sizes through sampled rows and size-independent properties.

Tolerances (relative Frobenius error): 1e-5 in fp32 mode (3xTF32), 2e-3 in TF32 mode.
"""
import numpy as np
import pytest

from util import load_golden, uniform, normal, rel_fro, TOL_FP32, TOL_TF32
from oracle import matmul_oracle as mo
from aakaar_b200 import cabi
from aakaar_b200.cabi import DeviceArray as DA, MODE_FP32, MODE_TF32

pytestmark = pytest.mark.gpu

MODES = [(MODE_FP32, TOL_FP32), (MODE_TF32, TOL_TF32)]
G, META = None, None


def setup_module(module):
    global G, META
    G, META = load_golden()


def dev(x):
    return DA.from_numpy(x)


def fwd_np(a_np, b_np, mode):
    return cabi.matmul_fwd(dev(a_np), dev(b_np), mode=mode).to_numpy()


# ------------------------------------------------------------------ golden vectors of the reference

@pytest.mark.parametrize("mode,tol", MODES)
def test_golden_config1(mode, tol):
    a, b = uniform((512, 512), 101), uniform((512, 512), 102)
    da_, db_ = dev(a), dev(b)
    c = cabi.matmul_fwd(da_, db_, mode=mode)
    ga, gb = cabi.matmul_bwd(da_, db_, dev(np.ones((512, 512), np.float32)), mode=mode)
    rows = META["cases"]["cfg1"]["rows"]
    for name, arr in (("c", c.to_numpy()), ("da", ga.to_numpy()), ("db", gb.to_numpy())):
        assert rel_fro(arr[rows], G[f"cfg1_{name}_rows"]) < tol, name
        assert abs(np.linalg.norm(arr.astype(np.float64)) / G[f"cfg1_{name}_norm"][0] - 1) < tol


@pytest.mark.parametrize("mode,tol", MODES)
def test_golden_small_cases(mode, tol):
    exact = np.array([[22, 28], [49, 64]], dtype=np.float32)
    a = np.array(META["cases"]["doc"]["a"], dtype=np.float32)
    b = np.array(META["cases"]["doc"]["b"], dtype=np.float32)
    np.testing.assert_array_equal(fwd_np(a, b, mode), exact)  # small integers are exact in TF32 too

    for key, (sa, sb, sc, seeds) in {
        "nd": ((3, 1, 5, 7), (2, 7, 4), (3, 2, 5, 4), (11, 12, 13)),
        "bt": ((2, 3, 8), (8, 5), (2, 3, 5), (21, 22, 23)),
        "rag": ((77, 45), (45, 19), (77, 19), (31, 32, 33)),
    }.items():
        a, b, dc = uniform(sa, seeds[0]), uniform(sb, seeds[1]), normal(sc, seeds[2])
        A, B = dev(a), dev(b)
        assert rel_fro(cabi.matmul_fwd(A, B, mode=mode).to_numpy(), G[f"{key}_c"]) < tol
        ga, gb = cabi.matmul_bwd(A, B, dev(dc), mode=mode)
        assert ga.shape == sa and gb.shape == sb
        assert rel_fro(ga.to_numpy(), G[f"{key}_da"]) < tol
        assert rel_fro(gb.to_numpy(), G[f"{key}_db"]) < tol


@pytest.mark.parametrize("mode,tol", MODES)
def test_golden_transposed_view_no_copy(mode, tol):
    # The reference needs A.contiguous(); here the transposed view is read in place.
    base, b = uniform((4, 2, 6, 16), 301), uniform((1, 2, 6, 16), 302)
    Abase, B = dev(base), dev(b)
    A = Abase.transpose(2, 3)
    c = cabi.matmul_fwd(A, B, mode=mode)
    assert c.shape == (4, 2, 16, 16)
    assert rel_fro(c.to_numpy(), G["cfg3s_c"]) < tol
    ga, gb = cabi.matmul_bwd(A, B, dev(np.ones(c.shape, np.float32)), mode=mode)
    assert gb.shape == (1, 2, 6, 16)
    assert rel_fro(np.swapaxes(ga.to_numpy(), -1, -2), G["cfg3s_dbase"]) < tol
    assert rel_fro(gb.to_numpy(), G["cfg3s_db"]) < tol


# ------------------------------------------------------------------ shape grid against the oracle

SHAPES = [
    (1, 1, 1), (1, 7, 3), (5, 1, 9), (16, 16, 16), (33, 65, 17), (128, 128, 32), (128, 256, 64),
    (129, 257, 33), (200, 300, 100), (256, 512, 1000), (511, 130, 7), (64, 2048, 96), (1000, 24, 513),
]


@pytest.mark.parametrize("mode,tol", MODES)
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_shape_grid_forward_backward(M, N, K, mode, tol):
    a, b, dc = uniform((M, K), M * 7 + K), uniform((K, N), N * 3 + K + 1), normal((M, N), M + N)
    A, B = dev(a), dev(b)
    ref = mo.matmul_forward(a, b, np.float64)
    assert rel_fro(cabi.matmul_fwd(A, B, mode=mode).to_numpy(), ref) < tol
    ga, gb = cabi.matmul_bwd(A, B, dev(dc), mode=mode)
    rda, rdb = mo.matmul_backward(a, b, dc, np.float64)
    assert rel_fro(ga.to_numpy(), rda) < tol
    assert rel_fro(gb.to_numpy(), rdb) < tol


BCAST = [
    ((4, 40, 24), (24, 56)),            # rank mismatch: B has no batch dim
    ((24, 56), (5, 56, 40)),            # A has no batch dim
    ((3, 1, 33, 20), (1, 4, 20, 48)),   # both broadcast
    ((2, 3, 4, 16, 8), (4, 8, 24)),     # three batch dims
    ((6, 1, 2, 16, 12), (1, 5, 1, 12, 8)),  # interleaved broadcast dims (host-looped)
    ((1, 1, 9, 5), (1, 5, 3)),          # all-ones batch
    ((1, 16, 27), (5, 27, 100)),        # the conv-as-matmul caller: [1,Cout,C*K] @ [B,C*K,L] (aakaar/__init__.py:305-307)
]


@pytest.mark.parametrize("mode,tol", MODES)
@pytest.mark.parametrize("sa,sb", BCAST)
def test_batch_broadcast(sa, sb, mode, tol):
    a, b = uniform(sa, 5), uniform(sb, 6)
    batch, M, K, N = mo.plan_nd_matmul(sa, sb)
    dc = normal(tuple(batch) + (M, N), 7)
    A, B = dev(a), dev(b)
    assert cabi.plan(A, B) == tuple(batch) + (M, N)
    assert rel_fro(cabi.matmul_fwd(A, B, mode=mode).to_numpy(), mo.matmul_forward(a, b, np.float64)) < tol
    ga, gb = cabi.matmul_bwd(A, B, dev(dc), mode=mode)
    rda, rdb = mo.matmul_backward(a, b, dc, np.float64)
    assert ga.shape == sa and gb.shape == sb
    assert rel_fro(ga.to_numpy(), rda) < tol
    assert rel_fro(gb.to_numpy(), rdb) < tol


# ------------------------------------------------------------------ strided views, no copies

@pytest.mark.parametrize("mode,tol", MODES)
def test_transposed_and_sliced_views(mode, tol):
    base_a, base_b = uniform((3, 72, 136), 81), uniform((3, 200, 72), 82)
    Abase, Bbase = dev(base_a), dev(base_b)
    # A = base_a^T  (M-major view), B = base_b^T (K... N-major becomes K-major view)
    A, B = Abase.transpose(1, 2), Bbase.transpose(1, 2)
    a, b = np.swapaxes(base_a, 1, 2), np.swapaxes(base_b, 1, 2)
    ref = mo.matmul_forward(np.ascontiguousarray(a), np.ascontiguousarray(b), np.float64)
    assert rel_fro(cabi.matmul_fwd(A, B, mode=mode).to_numpy(), ref) < tol
    dc = normal(ref.shape, 83)
    ga, gb = cabi.matmul_bwd(A, B, dev(dc), mode=mode)
    rda, rdb = mo.matmul_backward(np.ascontiguousarray(a), np.ascontiguousarray(b), dc, np.float64)
    assert rel_fro(ga.to_numpy(), rda) < tol and rel_fro(gb.to_numpy(), rdb) < tol

    # slices: aligned offset (TMA in place), odd offset and stepped inner dim (packed)
    big = uniform((160, 200), 84)
    Big = dev(big)
    other = uniform((64, 40), 85)
    Other = dev(other)
    for (r0, r1, c0, c1, cs) in [(32, 96, 64, 128, 1), (3, 67, 5, 69, 1), (0, 64, 1, 129, 2)]:
        sub = big[r0:r1, c0:c1:cs]
        V = Big.as_strided(sub.shape, (200, cs), offset=r0 * 200 + c0)
        ref = mo.matmul_forward(np.ascontiguousarray(sub), other, np.float64)
        assert rel_fro(cabi.matmul_fwd(V, Other, mode=mode).to_numpy(), ref) < tol
        dcs = normal(ref.shape, 86)
        ga, gb = cabi.matmul_bwd(V, Other, dev(dcs), mode=mode)
        rda, rdb = mo.matmul_backward(np.ascontiguousarray(sub), other, dcs, np.float64)
        assert rel_fro(ga.to_numpy(), rda) < tol and rel_fro(gb.to_numpy(), rdb) < tol
    # non-contiguous grad_output (the reference's 2-D backward raises here)
    a, b = uniform((48, 40), 87), uniform((40, 56), 88)
    dct = normal((56, 48), 89)
    DCt = dev(dct).transpose(0, 1)
    ga, gb = cabi.matmul_bwd(dev(a), dev(b), DCt, mode=mode)
    rda, rdb = mo.matmul_backward(a, b, np.ascontiguousarray(dct.T), np.float64)
    assert rel_fro(ga.to_numpy(), rda) < tol and rel_fro(gb.to_numpy(), rdb) < tol


@pytest.mark.parametrize("mode,tol", MODES)
def test_a_bt_at_b_and_bias(mode, tol):
    import ctypes as C
    lib = cabi.lib()
    a, b = uniform((70, 52), 91), uniform((90, 52), 92)
    A, B, Cc = dev(a), dev(b), DA((70, 90))
    va, vb, vc = A.view(), B.view(), Cc.view()
    cabi.check(lib.akr_matmul_a_bt(C.byref(va), C.byref(vb), C.byref(vc), mode, None))
    assert rel_fro(Cc.to_numpy(), a.astype(np.float64) @ b.astype(np.float64).T) < tol
    a2, b2 = uniform((52, 70), 93), uniform((52, 90), 94)
    A2, B2, C2 = dev(a2), dev(b2), DA((70, 90))
    va, vb, vc = A2.view(), B2.view(), C2.view()
    cabi.check(lib.akr_matmul_at_b(C.byref(va), C.byref(vb), C.byref(vc), mode, None))
    assert rel_fro(C2.to_numpy(), a2.astype(np.float64).T @ b2.astype(np.float64)) < tol
    # fused Linear bias
    x, w, bias = normal((130, 64), 95), uniform((64, 200), 96), normal((1, 200), 97)
    y = cabi.matmul_fwd(dev(x), dev(w), bias=dev(bias), mode=mode).to_numpy()
    assert rel_fro(y, x.astype(np.float64) @ w.astype(np.float64) + bias) < tol


def test_error_paths_through_the_abi():
    A, B = dev(np.ones((2, 3), np.float32)), dev(np.ones((4, 2), np.float32))
    with pytest.raises(cabi.AkrError) as e:
        cabi.matmul_fwd(A, B, out=DA((2, 2)))
    assert e.value.code == cabi.ERR_INVALID and e.value.msg.startswith(META["errors"]["k_mismatch"][1])
    with pytest.raises(cabi.AkrError) as e:
        cabi.plan(dev(np.ones((2, 2, 3), np.float32)), dev(np.ones((3, 3, 2), np.float32)))
    assert e.value.msg == META["errors"]["batch_mismatch"][1]
    with pytest.raises(cabi.AkrError):
        cabi.matmul_fwd(dev(np.ones((2, 3), np.float32)), dev(np.ones((3, 2), np.float32)), out=DA((2, 3)))


def test_caching_allocator_semantics():
    import ctypes as C
    lib = cabi.lib()
    h0, m0 = C.c_int64(), C.c_int64()
    lib.akr_allocator_stats(C.byref(h0), C.byref(m0))
    p = C.POINTER(C.c_float)()
    cabi.check(lib.akr_alloc(12345, C.byref(p)))
    first = C.cast(p, C.c_void_p).value
    cabi.check(lib.akr_free(p, 12345))
    q = C.POINTER(C.c_float)()
    cabi.check(lib.akr_alloc(12345, C.byref(q)))   # exact-size reuse
    assert C.cast(q, C.c_void_p).value == first
    r = C.POINTER(C.c_float)()
    cabi.check(lib.akr_alloc(12346, C.byref(r)))   # different size: a miss
    assert C.cast(r, C.c_void_p).value != first
    h1, m1 = C.c_int64(), C.c_int64()
    lib.akr_allocator_stats(C.byref(h1), C.byref(m1))
    assert h1.value >= h0.value + 1 and m1.value >= m0.value + 2 - 1
    cabi.check(lib.akr_free(q, 12345))
    cabi.check(lib.akr_free(r, 12346))


# ------------------------------------------------------------------ benchmark-size checks

def sampled_rows_check(A_np, B_np, C_np, rows, tol):
    ref = A_np[rows].astype(np.float64) @ B_np.astype(np.float64)
    assert rel_fro(C_np[rows], ref) < tol


@pytest.mark.parametrize("mode,tol", MODES)
@pytest.mark.parametrize("n", [2048, 4096])
def test_square_sweep_sampled(n, mode, tol):
    s = 1.0 / np.sqrt(n)
    a, b, dc = normal((n, n), 401, s), normal((n, n), 402, s), normal((n, n), 403)
    A, B, DC = dev(a), dev(b), dev(dc)
    rows = [0, 1, n // 3, n // 2 + 5, n - 1]
    c = cabi.matmul_fwd(A, B, mode=mode).to_numpy()
    sampled_rows_check(a, b, c, rows, tol)
    ga, gb = cabi.matmul_bwd(A, B, DC, mode=mode)
    ga, gb = ga.to_numpy(), gb.to_numpy()
    assert rel_fro(ga[rows], dc[rows].astype(np.float64) @ b.astype(np.float64).T) < tol
    assert rel_fro(gb[rows], a[:, rows].astype(np.float64).T @ dc.astype(np.float64)) < tol
    # on-device cross-check of the whole matrix with the plain-FMA kernel
    c_simt = cabi.matmul_simt(A, B).to_numpy()
    assert rel_fro(c, c_simt) < tol


@pytest.mark.parametrize("mode,tol", MODES)
def test_config3_full_size(mode, tol):
    # A [64,8,512,64] as a transposed view of [64,8,64,512], B [1,8,64,512]; dB sums over the 64.
    base, b = uniform((64, 8, 64, 512), 301), uniform((1, 8, 64, 512), 302)
    Abase, B = dev(base), dev(b)
    A = Abase.transpose(2, 3)
    assert A.strides == (262144, 32768, 1, 512)
    c = cabi.matmul_fwd(A, B, mode=mode)
    assert c.shape == (64, 8, 512, 512)
    cn = c.to_numpy()
    a64 = np.swapaxes(base, -1, -2).astype(np.float64)
    for (i, j) in [(0, 0), (17, 3), (63, 7)]:
        assert rel_fro(cn[i, j], a64[i, j] @ b[0, j].astype(np.float64)) < tol
    dc = np.ones(c.shape, np.float32)
    ga, gb = cabi.matmul_bwd(A, B, dev(dc), mode=mode)
    assert ga.shape == (64, 8, 512, 64) and gb.shape == (1, 8, 64, 512)
    gan, gbn = ga.to_numpy(), gb.to_numpy()
    # dA[i,j] = ones[512,512] @ B[0,j]^T : every row equals the row sums of B over n
    for (i, j) in [(0, 0), (40, 5)]:
        assert rel_fro(gan[i, j], np.ones((512, 512)) @ b[0, j].astype(np.float64).T) < tol
    # dB[0,j] = sum_i A[i,j]^T @ ones : column sums over (i, m), broadcast along n
    for j in (0, 6):
        col = a64[:, j].sum(axis=(0, 1))  # [64] over k
        assert rel_fro(gbn[0, j], np.repeat(col[:, None], 512, axis=1)) < tol


@pytest.mark.parametrize("mode,tol", MODES)
def test_config5a_batched_slice(mode, tol):
    # 1024 of the 8192 independent [256x256]@[256x256] pairs (one GPU's share at 8 GPUs)
    nb = 1024
    a, b = uniform((nb, 256, 256), 501), uniform((nb, 256, 256), 502)
    A, B = dev(a), dev(b)
    c = cabi.matmul_fwd(A, B, mode=mode).to_numpy()
    for i in (0, 511, 1023):
        assert rel_fro(c[i], a[i].astype(np.float64) @ b[i].astype(np.float64)) < tol
    ga, gb = cabi.matmul_bwd(A, B, dev(np.ones((nb, 256, 256), np.float32)), mode=mode)
    ga, gb = ga.to_numpy(), gb.to_numpy()
    ones = np.ones((256, 256))
    for i in (3, 1000):
        assert rel_fro(ga[i], ones @ b[i].astype(np.float64).T) < tol
        assert rel_fro(gb[i], a[i].astype(np.float64).T @ ones) < tol


@pytest.mark.parametrize("mode,tol", MODES)
def test_headline_size_8192_backward_sampled_rows(mode, tol):
    # The size every throughput figure is quoted on (8192^3, seeds of the benchmark): sampled rows of C,
    # dA = dC . B^T and dB = A^T . dC against float64, in both modes.
    n = 8192
    s = np.float32(1.0 / np.sqrt(n))
    a = np.random.Generator(np.random.PCG64(401)).standard_normal((n, n), dtype=np.float32) * s
    b = np.random.Generator(np.random.PCG64(402)).standard_normal((n, n), dtype=np.float32) * s
    dc = np.random.Generator(np.random.PCG64(403)).standard_normal((n, n), dtype=np.float32)
    A, B, DC = dev(a), dev(b), dev(dc)
    rows = [0, 2731, 4100, n - 1]

    def pick(x):
        return np.stack([x.as_strided((n,), (1,), offset=r * n).to_numpy() for r in rows])
    c = cabi.matmul_fwd(A, B, mode=mode)
    b64 = b.astype(np.float64)
    assert rel_fro(pick(c), a[rows].astype(np.float64) @ b64) < tol
    del c
    ga, gb = cabi.matmul_bwd(A, B, DC, mode=mode)
    assert rel_fro(pick(ga), dc[rows].astype(np.float64) @ b64.T) < tol
    del b64
    assert rel_fro(pick(gb), a[:, rows].astype(np.float64).T @ dc.astype(np.float64)) < tol


@pytest.mark.parametrize("mode,tol", MODES)
def test_config5a_full_batch(mode, tol):
    # All 8192 independent [256x256]@[256x256] pairs on one GPU (2 GiB per array): sampled batch entries of
    # C, dA and dB against float64, and a checksum of checksums over the whole result: with dC = ones,
    # sum(dA[i]) = 256 * sum(B[i]) and sum(dB[i]) = 256 * sum(A[i]) for every batch entry i.
    nb = 8192
    ga_ = np.random.Generator(np.random.PCG64(501))
    gb_ = np.random.Generator(np.random.PCG64(502))
    a = ga_.random((nb, 256, 256), dtype=np.float32) * np.float32(2) - np.float32(1)
    b = gb_.random((nb, 256, 256), dtype=np.float32) * np.float32(2) - np.float32(1)
    A, B = dev(a), dev(b)
    c = cabi.matmul_fwd(A, B, mode=mode)
    cn = c.to_numpy()
    for i in (0, 4095, 4096, nb - 1):
        assert rel_fro(cn[i], a[i].astype(np.float64) @ b[i].astype(np.float64)) < tol
    # every batch entry: sum of C[i] = rowsum-of-A . colsum-of-B
    want = np.einsum("bk,bk->b", a.sum(axis=1, dtype=np.float64), b.sum(axis=2, dtype=np.float64))
    got = cn.sum(axis=(1, 2), dtype=np.float64)
    scale = np.sqrt(np.mean(want ** 2))
    assert np.max(np.abs(got - want)) / scale < (50 * tol)
    del cn, c
    DC = DA((nb, 256, 256))
    import ctypes as C
    cabi.check(cabi.lib().akr_fill(C.cast(DC.ptr, C.POINTER(C.c_float)), 1.0, nb * 65536, None))
    ga, gb = cabi.matmul_bwd(A, B, DC, mode=mode)
    gan = ga.to_numpy()
    ones = np.ones((256, 256))
    for i in (3, 5000, nb - 1):
        assert rel_fro(gan[i], ones @ b[i].astype(np.float64).T) < tol
    assert rel_fro(gan.sum(axis=(1, 2), dtype=np.float64), 256.0 * b.sum(axis=(1, 2), dtype=np.float64)) < tol
    del gan, ga
    gbn = gb.to_numpy()
    for i in (3, 5000, nb - 1):
        assert rel_fro(gbn[i], a[i].astype(np.float64).T @ ones) < tol
    assert rel_fro(gbn.sum(axis=(1, 2), dtype=np.float64), 256.0 * a.sum(axis=(1, 2), dtype=np.float64)) < tol


def test_largest_benchmark_square_16384_sampled_rows():
    # the largest size of the benchmark sweep (16384^3, 1 GiB per matrix): sampled rows of C, dA and dB against
    # float64, TF32 mode and the fp32-accurate mode (CTA pairs, low parts derived in the kernel)
    n = 16384
    g = np.random.Generator(np.random.PCG64(404))
    s = np.float32(1.0 / np.sqrt(n))
    a = g.standard_normal((n, n), dtype=np.float32) * s
    b = g.standard_normal((n, n), dtype=np.float32) * s
    A, B = dev(a), dev(b)
    rows = [0, 4097, n - 1]
    for mode, tol in MODES:
        c = cabi.matmul_fwd(A, B, mode=mode)
        got = np.stack([c.as_strided((n,), (1,), offset=r * n).to_numpy() for r in rows])
        sampled_rows_check(a, b, _Rows(got, rows), rows, tol)
        # dA rows and dB rows with dC := C (any dense matrix will do)
        da, db = cabi.matmul_bwd(A, B, c, mode=mode)
        cn = np.stack([c.as_strided((n,), (1,), offset=r * n).to_numpy() for r in rows])
        got_da = np.stack([da.as_strided((n,), (1,), offset=r * n).to_numpy() for r in rows])
        assert rel_fro(got_da, cn.astype(np.float64) @ b.astype(np.float64).T) < tol
        del da
        full_c = c.to_numpy()
        got_db = np.stack([db.as_strided((n,), (1,), offset=r * n).to_numpy() for r in rows])
        assert rel_fro(got_db, a[:, rows].astype(np.float64).T @ full_c.astype(np.float64)) < tol
        del db, c, full_c


class _Rows:
    """Lets sampled_rows_check index a few downloaded rows as if they were the whole matrix."""

    def __init__(self, data, rows):
        self.data, self.rows = data, list(rows)

    def __getitem__(self, rows):
        return self.data[[self.rows.index(r) for r in rows]]


def test_linearity_and_transpose_identity_8192():
    # Size-independent properties at the headline size, TF32 mode:
    #   (A @ B)^T == B^T @ A^T evaluated through transposed VIEWS (exercises the other operand majors)
    n = 8192
    s = 1.0 / np.sqrt(n)
    A, B = dev(normal((n, n), 401, s)), dev(normal((n, n), 402, s))
    c1 = cabi.matmul_fwd(A, B, mode=MODE_TF32)
    c2 = cabi.matmul_fwd(B.transpose(0, 1), A.transpose(0, 1), mode=MODE_TF32)
    x, y = c1.to_numpy(), c2.to_numpy()
    assert rel_fro(y.T, x) < 2 * TOL_TF32
    # fp32 mode agrees with TF32 mode to TF32 accuracy and is itself far tighter on sampled rows
    c3 = cabi.matmul_fwd(A, B, mode=MODE_FP32).to_numpy()
    assert rel_fro(x, c3) < TOL_TF32
    a_np, b_np = A.to_numpy(), B.to_numpy()
    sampled_rows_check(a_np, b_np, c3, [0, 4097, 8191], TOL_FP32)


def test_big_tile_kernel_ragged_all_layouts():
    # Large enough for the 256 x 256-tile TF32 kernel (>= 148 such tiles), ragged in M, N and K,
    # every operand layout through transposed views, plus the fused bias. Sampled rows vs fp64.
    M, N, K = 3000, 3300, 1028
    a, b = normal((M, K), 601, 0.05), normal((K, N), 602, 0.05)
    at, bt = np.ascontiguousarray(a.T), np.ascontiguousarray(b.T)
    bias = normal((1, N), 603)
    A, B, AT, BT = dev(a), dev(b), dev(at), dev(bt)
    rows = [0, 127, 128, 255, 256, 1500, 2943, 2999]
    ref = a[rows].astype(np.float64) @ b.astype(np.float64)
    for Aop, Bop in ((A, B), (A, BT.transpose(0, 1)), (AT.transpose(0, 1), B), (AT.transpose(0, 1), BT.transpose(0, 1))):
        c = cabi.matmul_fwd(Aop, Bop, mode=MODE_TF32).to_numpy()
        assert rel_fro(c[rows], ref) < TOL_TF32
    c = cabi.matmul_fwd(A, B, bias=dev(bias), mode=MODE_TF32).to_numpy()
    assert rel_fro(c[rows], ref + bias) < TOL_TF32
    # batched: 2 x (1536 x 2560 x 1024) -> 2*6*10 = 120 tiles < 148: general kernel; 3 batches -> big kernel
    ab, bb = normal((3, 1536, 1024), 604, 0.05), normal((1, 1024, 2560), 605, 0.05)
    cb = cabi.matmul_fwd(dev(ab), dev(bb), mode=MODE_TF32).to_numpy()
    for i in range(3):
        assert rel_fro(cb[i][[0, 700, 1535]], ab[i][[0, 700, 1535]].astype(np.float64) @ bb[0].astype(np.float64)) < TOL_TF32


def test_sum_to_bias_gradient_shapes():
    # reduce_grad_to_shape for a broadcast add: column-sum fast path (dense, leading dims summed) and generic path
    import ctypes as C
    lib = cabi.lib()
    for gshape, oshape in (((1000, 77), (1, 77)), ((4096, 256), (1, 256)), ((3, 5, 40), (1, 1, 40)), ((3, 5, 40), (40,)),
                           ((64, 16), (1, 16)), ((6, 1, 50), (1, 1, 50)), ((4, 7, 33), (4, 1, 33)), ((9, 9), (1,))):
        g = normal(gshape, 11)
        G_, O_ = dev(g), DA(oshape)
        vg, vo = G_.view(), O_.view()
        cabi.check(lib.akr_sum_to(C.byref(vg), C.byref(vo), None))
        pad = (1,) * (len(gshape) - len(oshape)) + tuple(oshape)
        axes = tuple(i for i, (a, b) in enumerate(zip(gshape, pad)) if a != b)
        ref = g.astype(np.float64).sum(axis=axes, keepdims=True).reshape(oshape)
        assert rel_fro(O_.to_numpy(), ref) < 1e-5, (gshape, oshape)


def test_bounded_wait_abort_is_reported_and_recoverable():
    # Failure path without faulting the GPU: the load warp never signals, so every in-kernel wait runs
    # out (bound lowered to 30 ms), the kernel stops cleanly and the host sees AKR_ERR_ABORTED once.
    lib = cabi.lib()
    a, b = uniform((256, 256), 1), uniform((256, 256), 2)
    A, B = dev(a), dev(b)
    cabi.synchronize()
    try:
        cabi.check(lib.akr_debug_configure(16, 30))
        for mode in (MODE_TF32, MODE_FP32):
            cabi.matmul_fwd(A, B, mode=mode)
            with pytest.raises(cabi.AkrError) as e:
                cabi.synchronize()
            assert e.value.code == cabi.ERR_ABORTED
            cabi.synchronize()   # reported once, then clear
        # the CTA-pair kernel (49 tiles of 256 x 256, 32 k-blocks): both CTAs of every pair give up and
        # meet at the cluster barrier of the teardown
        A2, B2 = dev(uniform((1792, 1024), 3)), dev(uniform((1024, 1792), 4))
        cabi.synchronize()
        cabi.matmul_fwd(A2, B2, mode=MODE_TF32)
        with pytest.raises(cabi.AkrError) as e:
            cabi.synchronize()
        assert e.value.code == cabi.ERR_ABORTED
        cabi.synchronize()
        # the same product on the fp32-accurate CTA-pair kernel (its converter warps wait for tiles that never land)
        cabi.matmul_fwd(A2, B2, mode=MODE_FP32)
        with pytest.raises(cabi.AkrError) as e:
            cabi.synchronize()
        assert e.value.code == cabi.ERR_ABORTED
        cabi.synchronize()
        # 512 x 256 tiles on pairs (128 of them, 32 k-blocks)
        A3, B3 = dev(uniform((4096, 1024), 5)), dev(uniform((1024, 4096), 6))
        cabi.synchronize()
        cabi.matmul_fwd(A3, B3, mode=MODE_TF32)
        with pytest.raises(cabi.AkrError) as e:
            cabi.synchronize()
        assert e.value.code == cabi.ERR_ABORTED
        cabi.synchronize()
    finally:
        cabi.check(lib.akr_debug_configure(0, 0))
    # the context is still usable and results are right again
    c = cabi.matmul_fwd(A, B, mode=MODE_FP32).to_numpy()
    assert rel_fro(c, a.astype(np.float64) @ b.astype(np.float64)) < TOL_FP32


def test_experimental_cta_pair_kernel_parity():
    # The cta_group::2 kernel of the fp32-accurate mode (two CTAs share one 256 x 256 tile), forced onto shapes
    # below its default threshold (short contraction) and on its default territory.
    lib = cabi.lib()
    a, b = uniform((1500, 200), 71), uniform((200, 1700), 72)
    bias = normal((1, 1700), 73)
    ref = a.astype(np.float64) @ b.astype(np.float64)
    try:
        cabi.check(lib.akr_debug_configure(32, 0))
        A, B = dev(a), dev(b)
        assert rel_fro(cabi.matmul_fwd(A, B, mode=MODE_FP32).to_numpy(), ref) < TOL_FP32
        assert rel_fro(cabi.matmul_fwd(A, B, bias=dev(bias), mode=MODE_FP32).to_numpy(), ref + bias) < TOL_FP32
        at, bt = dev(np.ascontiguousarray(a.T)), dev(np.ascontiguousarray(b.T))
        c = cabi.matmul_fwd(at.transpose(0, 1), bt.transpose(0, 1), mode=MODE_FP32).to_numpy()
        assert rel_fro(c, ref) < TOL_FP32
        # a large compute-bound product (the kernel's default territory): 256 pair tiles, 256 k-blocks
        n = 4096
        s_ = 1.0 / np.sqrt(n)
        a2, b2 = normal((n, n), 401, s_), normal((n, n), 402, s_)
        c2 = cabi.matmul_fwd(dev(a2), dev(b2), mode=MODE_FP32).to_numpy()
        sampled_rows_check(a2, b2, c2, [0, 129, 2047, 4095], TOL_FP32)
    finally:
        cabi.check(lib.akr_debug_configure(0, 0))


def test_fp32_pair_kernel_short_contractions_store_through_tma():
    # fp32-accurate products on CTA pairs with a contraction of at most 512 run the layout with two low-part slots
    # and two sets of output staging tiles, and aligned plain outputs leave through TMA boxes of 128 rows x 32
    # columns: ragged edges in M and N (a last pair whose second CTA has no rows, a last box of 4 columns), the four
    # operand layouts, batches, bias; an output whose row length is no multiple of 4 (plain stores instead).
    rng = np.random.default_rng(291)
    def check(bt, M, N, K, ta, tb, with_bias=False):
        a = uniform(bt + ((K, M) if ta else (M, K)), int(rng.integers(1 << 30)))
        b = uniform(bt + ((N, K) if tb else (K, N)), int(rng.integers(1 << 30)))
        A, B = dev(a), dev(b)
        nd = len(bt) + 2
        Av = A.transpose(nd - 2, nd - 1) if ta else A
        Bv = B.transpose(nd - 2, nd - 1) if tb else B
        bias = normal((1, N), 292) if with_bias else None
        c = cabi.matmul_fwd(Av, Bv, bias=dev(bias) if with_bias else None, mode=MODE_FP32).to_numpy()
        an = np.swapaxes(a, -1, -2) if ta else a
        bn = np.swapaxes(b, -1, -2) if tb else b
        ref = np.matmul(an.astype(np.float64), bn.astype(np.float64))
        if with_bias:
            ref = ref + bias
        assert rel_fro(c, ref) < TOL_FP32, (bt, M, N, K, ta, tb)
    for ta in (0, 1):
        for tb in (0, 1):
            check((), 1400, 1796, 288, ta, tb)            # 6 x 8 tiles; 1400 = 5 x 256 + 120: the last pair's second CTA is empty
            check((), 1400, 1796, 64 + 36 * ta + 8 * tb, ta, tb)  # the shortest contractions the pair kernel takes (two or three k-blocks)
    check((), 1536, 1800, 512, 0, 0, with_bias=True)      # 16 k-blocks: the longest contraction of this layout
    check((), 1536, 1800, 544, 0, 0, with_bias=True)      # 17 k-blocks: three low-part slots, one set of staging tiles
    check((48,), 256, 256, 256, 0, 0)                     # one tile per batch entry
    check((3, 4), 300, 520, 256, 0, 1)
    check((), 1400, 1798, 288, 0, 0)                      # rows of 1798 floats are not 16-byte aligned: plain stores


def test_tf32_cta_pair_kernel_parity():
    # TF32 products on CTA pairs (cta_group::2, one 256 x 256 tile per pair): ragged edges, all four
    # operand layouts, bias, C +=, broadcast batches and a summed batch dim (weight gradient), with the
    # kernel preferred wherever it applies (flag 2048) and under its default routing.
    lib = cabi.lib()
    try:
        for flags in (2048, 0):
            cabi.check(lib.akr_debug_configure(flags, 0))
            M, N, K = (1500, 1700, 200) if flags else (2100, 1800, 1100)
            a, b = uniform((M, K), 81), uniform((K, N), 82)
            bias = normal((1, N), 83)
            ref = a.astype(np.float64) @ b.astype(np.float64)
            A, B = dev(a), dev(b)
            at, bt = dev(np.ascontiguousarray(a.T)), dev(np.ascontiguousarray(b.T))
            for Av in (A, at.transpose(0, 1)):
                for Bv in (B, bt.transpose(0, 1)):
                    assert rel_fro(cabi.matmul_fwd(Av, Bv, mode=MODE_TF32).to_numpy(), ref) < TOL_TF32
            assert rel_fro(cabi.matmul_fwd(A, B, bias=dev(bias), mode=MODE_TF32).to_numpy(), ref + bias) < TOL_TF32
            # ragged sizes that defeat the vector / TMA store path (N % 4 != 0)
            a3, b3 = uniform((1300, 264), 84), uniform((264, 1299), 85)
            c3 = cabi.matmul_fwd(dev(a3), dev(b3), mode=MODE_TF32).to_numpy()
            assert rel_fro(c3, a3.astype(np.float64) @ b3.astype(np.float64)) < TOL_TF32
        cabi.check(lib.akr_debug_configure(2048, 0))
        # batched with broadcast: [3,1,520,96] @ [2,96,530] -> 6 x (3 x 3) tiles; backward sums dB over the batch
        a4, b4 = uniform((3, 1, 520, 96), 86), uniform((2, 96, 530), 87)
        dc4 = uniform((3, 2, 520, 530), 88)
        A4, B4, G4 = dev(a4), dev(b4), dev(dc4)
        assert rel_fro(cabi.matmul_fwd(A4, B4, mode=MODE_TF32).to_numpy(), mo.matmul_forward(a4, b4, np.float64)) < TOL_TF32
        da, db = cabi.matmul_bwd(A4, B4, G4, mode=MODE_TF32)
        rda, rdb = mo.matmul_backward(a4, b4, dc4, np.float64)
        assert rel_fro(da.to_numpy(), rda) < TOL_TF32 and rel_fro(db.to_numpy(), rdb) < TOL_TF32
    finally:
        cabi.check(lib.akr_debug_configure(0, 0))


def test_tf32_tall_pair_tile_kernel_parity():
    # Large TF32 products run 512 x 256 tiles on CTA pairs (each CTA 256 rows of A and 128 columns of B per k-block,
    # two accumulators per CTA). Shapes big enough for that routing: ragged edges in M, N and K, the four operand
    # layouts, a last tile whose second CTA has no rows at all, batches, bias, and the backward products; sampled
    # rows against float64.
    rng = np.random.default_rng(91)
    def check(bt, M, N, K, ta, tb, with_bias=False):
        a = uniform(bt + ((K, M) if ta else (M, K)), int(rng.integers(1 << 30)))
        b = uniform(bt + ((N, K) if tb else (K, N)), int(rng.integers(1 << 30)))
        A, B = dev(a), dev(b)
        nd = len(bt) + 2
        Av = A.transpose(nd - 2, nd - 1) if ta else A
        Bv = B.transpose(nd - 2, nd - 1) if tb else B
        bias = normal((1, N), 92) if with_bias else None
        c = cabi.matmul_fwd(Av, Bv, bias=dev(bias) if with_bias else None, mode=MODE_TF32).to_numpy()
        rows = np.unique(np.concatenate([np.arange(4), np.array([127, 128, 255, 256, 257, 383, 384, 511, 512, 513]),
                                         rng.integers(0, M, 12), np.arange(M - 3, M)]))
        an = np.swapaxes(a, -1, -2) if ta else a
        bn = np.swapaxes(b, -1, -2) if tb else b
        ref = np.matmul(an[..., rows, :].astype(np.float64), bn.astype(np.float64))
        if with_bias:
            ref = ref + bias
        assert rel_fro(c[..., rows, :], ref) < TOL_TF32, (bt, M, N, K, ta, tb)
    for ta in (0, 1):
        for tb in (0, 1):
            check((), 4100, 4100, 1030, ta, tb)
    check((), 4352, 4096, 1024, 0, 0, with_bias=True)   # 8.5 tiles of 512 rows: the last pair's second CTA is empty
    check((3,), 2048, 2048, 1056, 0, 0)
    # backward at a size that routes dA (K-major x K-major) and dB (M-major x N-major) there too
    M, K, N = 4096, 4224, 4100
    a, b, dc = uniform((M, K), 93), uniform((K, N), 94), uniform((M, N), 95)
    da, db = cabi.matmul_bwd(dev(a), dev(b), dev(dc), mode=MODE_TF32)
    rows = np.array([0, 1, 255, 256, 511, 512, 2047, 4095])
    assert rel_fro(da.to_numpy()[rows], dc[rows].astype(np.float64) @ b.astype(np.float64).T) < TOL_TF32
    krows = np.array([0, 1, 255, 256, 511, 512, 2047, 4223])
    assert rel_fro(db.to_numpy()[krows], a[:, krows].astype(np.float64).T @ dc.astype(np.float64)) < TOL_TF32


def test_tf32_128_column_tiles_with_64_deep_stages():
    # TF32 products whose output is 65..128 columns wide and whose contraction is at least 512 run 128 x 128 tiles
    # with 64-deep stages made of two 32-deep sub-tiles. Contraction tails that end in the first sub-tile (K % 64 in
    # 1..32: the second one is all zero fill), in the second one, and none; the four operand layouts; a batch; bias.
    rng = np.random.default_rng(191)
    def check(bt, M, N, K, ta, tb, with_bias=False):
        a = uniform(bt + ((K, M) if ta else (M, K)), int(rng.integers(1 << 30)))
        b = uniform(bt + ((N, K) if tb else (K, N)), int(rng.integers(1 << 30)))
        A, B = dev(a), dev(b)
        nd = len(bt) + 2
        Av = A.transpose(nd - 2, nd - 1) if ta else A
        Bv = B.transpose(nd - 2, nd - 1) if tb else B
        bias = normal((1, N), 192) if with_bias else None
        c = cabi.matmul_fwd(Av, Bv, bias=dev(bias) if with_bias else None, mode=MODE_TF32).to_numpy()
        an = np.swapaxes(a, -1, -2) if ta else a
        bn = np.swapaxes(b, -1, -2) if tb else b
        ref = np.matmul(an.astype(np.float64), bn.astype(np.float64))
        if with_bias:
            ref = ref + bias
        assert rel_fro(c, ref) < TOL_TF32, (bt, M, N, K, ta, tb)
    for ta in (0, 1):
        for tb in (0, 1):
            for K in (512, 516, 544, 548, 1000):          # K must be a multiple of 4 only for M-major operands
                check((), 300, 128 if tb == 0 else 100, K, ta, tb)
    check((), 1000, 100, 513, 0, 1)                       # a one-element tail (K-major operands have no stride rule)
    check((5,), 260, 96, 800, 0, 0, with_bias=True)
    check((), 40000, 128, 576, 0, 0)                      # more tiles than CTAs: the ring and TMEM halves wrap


def test_clock_probe_reports_the_sm_clock_of_a_launch():
    # akr_debug_configure(32768): every CTA records cycles and nanoseconds; the ratio is the SM clock the kernel ran
    # at (B200: at most 1965 MHz), the cycle count is at least what the MMAs alone need; the product stays correct.
    lib = cabi.lib()
    a, b = uniform((2048, 2048), 71), uniform((2048, 2048), 72)
    A, B = dev(a), dev(b)
    try:
        cabi.check(lib.akr_debug_configure(32768, 0))
        c = cabi.matmul_fwd(A, B, mode=MODE_TF32)
        cabi.synchronize()
        r = cabi.gemm_clock_read(148)
    finally:
        cabi.check(lib.akr_debug_configure(0, 0))
    assert 300.0 < r["sm_mhz_min"] <= r["sm_mhz"] < 2100.0, r
    assert r["cycles"] >= 64 * 512 and r["us"] > 0, r      # one 128 x 256 tile per CTA: 64 k-blocks of 4 MMAs
    rows = np.array([0, 5, 777, 2047])
    assert rel_fro(c.to_numpy()[rows], a[rows].astype(np.float64) @ b.astype(np.float64)) < TOL_TF32


@pytest.mark.parametrize("mode,tol", [(MODE_TF32, TOL_TF32), (MODE_FP32, TOL_FP32)])
def test_split_contractions_on_cta_pairs(mode, tol):
    # Weight-gradient shapes (few output tiles, long contraction): the contraction is split over CTA pairs, every pair
    # writes a partial tile and the reduction kernel adds them. Ragged edges, the four layouts, a batch, a bias row
    # (applied by the reduction), and C += (the reduction reads the old C).
    rng = np.random.default_rng(97)
    for (bt, M, N, K, ta, tb) in (((), 512, 512, 4096, 1, 0), ((), 1000, 700, 5000, 0, 0), ((), 768, 768, 3072, 0, 1),
                                  ((2,), 300, 520, 2500, 1, 1), ((), 1536, 1536, 4096, 0, 0)):
        a = uniform(bt + ((K, M) if ta else (M, K)), int(rng.integers(1 << 30)))
        b = uniform(bt + ((N, K) if tb else (K, N)), int(rng.integers(1 << 30)))
        A, B = dev(a), dev(b)
        nd = len(bt) + 2
        Av = A.transpose(nd - 2, nd - 1) if ta else A
        Bv = B.transpose(nd - 2, nd - 1) if tb else B
        ref = np.matmul((np.swapaxes(a, -1, -2) if ta else a).astype(np.float64), (np.swapaxes(b, -1, -2) if tb else b).astype(np.float64))
        assert rel_fro(cabi.matmul_fwd(Av, Bv, mode=mode).to_numpy(), ref) < tol, (bt, M, N, K, ta, tb)
        bias = normal((1, N), 98)
        assert rel_fro(cabi.matmul_fwd(Av, Bv, bias=dev(bias), mode=mode).to_numpy(), ref + bias) < tol, (bt, M, N, K)
    # the same through the backward entry point: dB = A^T dC with a long batch of rows
    a, b, dc = uniform((6000, 520), 99), uniform((520, 700), 100), uniform((6000, 700), 101)
    da, db = cabi.matmul_bwd(dev(a), dev(b), dev(dc), mode=mode)
    assert rel_fro(db.to_numpy(), a.astype(np.float64).T @ dc.astype(np.float64)) < tol
    assert rel_fro(da.to_numpy(), dc.astype(np.float64) @ b.astype(np.float64).T) < tol


def _random_case(rng):
    """A random product: batch broadcasting, operand layouts (transposed / sliced views), ragged sizes."""
    nb = int(rng.integers(0, 4))
    batch = [int(rng.integers(1, 5)) for _ in range(nb)]
    M, N, K = (int(rng.integers(1, 300)) for _ in range(3))
    def operand(rows, cols, seed):
        bshape = [d if rng.random() < 0.7 else 1 for d in batch]
        drop = int(rng.integers(0, len(bshape) + 1)) if rng.random() < 0.3 else 0   # fewer batch dims than the other
        bshape = bshape[drop:]
        transposed = rng.random() < 0.5
        pad_r, pad_c = int(rng.integers(0, 3)), int(rng.integers(0, 3)) * 4 if rng.random() < 0.5 else int(rng.integers(0, 5))
        store = (rows, cols) if not transposed else (cols, rows)
        full = tuple(bshape) + (store[0] + pad_r, store[1] + pad_c)
        base = uniform(full, seed)
        r0, c0 = int(rng.integers(0, pad_r + 1)), int(rng.integers(0, pad_c + 1))
        view_np = base[..., r0:r0 + store[0], c0:c0 + store[1]]
        Dbase = dev(base)
        strides = list(Dbase.strides)
        off = r0 * strides[-2] + c0 * strides[-1]
        shape = list(bshape) + list(store)
        V = Dbase.as_strided(shape, strides, offset=off)
        if transposed:
            V = V.transpose(len(shape) - 2, len(shape) - 1)
            view_np = np.swapaxes(view_np, -1, -2)
        return V, np.ascontiguousarray(view_np), Dbase
    A, a_np, keep_a = operand(M, K, int(rng.integers(1 << 30)))
    B, b_np, keep_b = operand(K, N, int(rng.integers(1 << 30)))
    return A, a_np, B, b_np, (keep_a, keep_b)


@pytest.mark.parametrize("mode,tol", MODES)
def test_random_shapes_layouts_and_broadcasts(mode, tol):
    rng = np.random.Generator(np.random.PCG64(20260 + mode))
    for case in range(40):
        A, a_np, B, b_np, keep = _random_case(rng)
        ref = mo.matmul_forward(a_np, b_np, np.float64)
        c = cabi.matmul_fwd(A, B, mode=mode)
        assert c.shape == ref.shape, (case, A.shape, B.shape)
        scale = max(1e-30, float(np.linalg.norm(ref)))
        assert np.linalg.norm(c.to_numpy().astype(np.float64) - ref) / scale < tol, (case, A.shape, A.strides, B.shape, B.strides)
        dc = normal(ref.shape, 77 + case)
        ga, gb = cabi.matmul_bwd(A, B, dev(dc), mode=mode)
        rda, rdb = mo.matmul_backward(a_np, b_np, dc, np.float64)
        assert ga.shape == tuple(a_np.shape) and gb.shape == tuple(b_np.shape)
        for got, want, what in ((ga, rda, "dA"), (gb, rdb, "dB")):
            n = max(1e-30, float(np.linalg.norm(want)))
            assert np.linalg.norm(got.to_numpy().astype(np.float64) - want) / n < tol, (case, what, A.shape, A.strides, B.shape, B.strides)


@pytest.mark.gpu
@pytest.mark.parametrize("dt", [np.float64, np.int32, np.int64])
def test_typed_forward_through_abi(dt):
    # forward-only dtypes of the reference (src/matmul_kernel.cu:151-341): bit-exact for integers
    # (64-bit accumulation, wrap to the operand width), 1e-14 for float64; strided views read in place
    g = np.random.Generator(np.random.PCG64(5))
    if dt == np.float64:
        a, b = g.standard_normal((2, 3, 33, 70)), g.standard_normal((3, 41, 70))
    else:
        hi = 2 ** 30 if dt == np.int32 else 2 ** 45          # int32 products overflow and must wrap
        a = g.integers(-hi, hi, (2, 3, 33, 70)).astype(dt)
        b = g.integers(-hi, hi, (3, 41, 70)).astype(dt)
    bt = np.swapaxes(b, -1, -2)                               # (3, 70, 41) strided view
    got = cabi.matmul_typed(a, bt)
    want = mo.matmul_forward_typed(a, bt)
    assert got.dtype == dt and got.shape == (2, 3, 33, 41)
    if dt == np.float64:
        assert rel_fro(got, want) < 1e-14
    else:
        np.testing.assert_array_equal(got, want)
    with pytest.raises(RuntimeError, match="share one dtype"):
        cabi.matmul_typed(a, bt.astype(np.float32))


# ------------------------------------------------------------------ fused epilogues

@pytest.mark.parametrize("mode,tol", MODES)
def test_backward_through_tanh_in_the_epilogue(mode, tol):
    # dZ = (dC B^T) * (1 - A^2) with A = tanh(Z): 2-D, ragged, a transposed A view, a broadcast-batch A
    # (reduced first, multiplied once), and a shape that takes the split-contraction path
    cases = [((200, 96), (96, 72), False), ((130, 257), (257, 33), False), ((96, 200), (96, 72), True),
             ((1, 40, 24), (5, 24, 56), False), ((3, 2, 48, 40), (2, 40, 64), False), ((64, 2048), (2048, 16), False)]
    for sa, sb, transposed in cases:
        z = normal(sa, 7)
        a = np.tanh(z).astype(np.float32)
        A = dev(a)
        if transposed:
            A = A.transpose(0, 1)
            a = np.ascontiguousarray(a.T)
        b = uniform(sb, 8)
        batch, M, K, N = mo.plan_nd_matmul(a.shape, sb)
        dc = normal(tuple(batch) + (M, N), 9)
        dz, db = cabi.matmul_bwd_tanh(A, dev(b), dev(dc), mode=mode)
        rdz, rdb = mo.matmul_backward_tanh(a, b, dc, np.float64)
        assert dz.shape == a.shape and db.shape == sb
        assert rel_fro(dz.to_numpy(), rdz) < tol, (sa, sb)
        assert rel_fro(db.to_numpy(), rdb) < tol, (sa, sb)
    # only dZ
    dz, db = cabi.matmul_bwd_tanh(dev(a), dev(b), dev(dc), mode=mode, need_db=False)
    assert db is None and rel_fro(dz.to_numpy(), rdz) < tol


@pytest.mark.parametrize("mode,tol", MODES)
def test_alpha_beta_epilogue(mode, tol):
    # C = alpha * (A @ B) + beta * D: small, ragged, batched with a broadcast addend view, CTA-pair sized
    for sa, sb in [((64, 64), (64, 64)), ((129, 70), (70, 257)), ((2, 3, 40, 24), (3, 24, 56)), ((1500, 1100), (1100, 1700))]:
        a, b = uniform(sa, 21), uniform(sb, 22)
        batch, M, K, N = mo.plan_nd_matmul(sa, sb)
        d = normal(tuple(batch) + (M, N), 23)
        got = cabi.matmul_axpby(dev(a), dev(b), 2.0315, -4.775, dev(d), mode=mode).to_numpy()
        assert rel_fro(got, mo.matmul_axpby(a, b, 2.0315, -4.775, d, np.float64)) < tol, (sa, sb)
        got = cabi.matmul_axpby(dev(a), dev(b), 0.5, 0.0, None, mode=mode).to_numpy()
        assert rel_fro(got, mo.matmul_axpby(a, b, 0.5, 0.0, None, np.float64)) < tol
    # addend given as a transposed view (column stride != 1)
    a, b, dt = uniform((96, 40), 24), uniform((40, 72), 25), normal((72, 96), 26)
    got = cabi.matmul_axpby(dev(a), dev(b), 1.0, 3.4445, dev(dt).transpose(0, 1), mode=mode).to_numpy()
    assert rel_fro(got, mo.matmul_axpby(a, b, 1.0, 3.4445, np.ascontiguousarray(dt.T), np.float64)) < tol
    with pytest.raises(cabi.AkrError):
        cabi.matmul_axpby(dev(a), dev(b), 1.0, 1.0, dev(dt), mode=mode)   # wrong addend shape


@pytest.mark.parametrize("mode,tol", MODES)
def test_newton_schulz_chain_with_fused_epilogues(mode, tol):
    # Muon's orthogonalisation (aakaar/optim.py:533-542), three launches per iteration: X^T X through a
    # transposed view, b A + c A A and a X + X B through the alpha / beta epilogue
    g = normal((192, 320), 31)
    X = dev((g / (np.sqrt((g.astype(np.float64) ** 2).sum()) + 1e-7)).astype(np.float32))
    a_, b_, c_ = 3.4445, -4.7750, 2.0315
    for _ in range(5):
        A = cabi.matmul_fwd(X.transpose(0, 1), X, mode=mode)
        B = cabi.matmul_axpby(A, A, c_, b_, A, mode=mode)
        X = cabi.matmul_axpby(X, B, 1.0, a_, X, mode=mode)
    ref = mo.newton_schulz(g, 5, np.float64)
    assert rel_fro(X.to_numpy(), ref) < 20 * tol    # five chained iterations amplify the rounding of each product
    s = np.linalg.svd(X.to_numpy().astype(np.float64), compute_uv=False)
    assert 0.5 < s.min() and s.max() < 1.5          # singular values pushed towards 1


@pytest.mark.parametrize("mode,tol", MODES)
def test_random_mid_size_shapes_sampled(mode, tol):
    # Sizes that reach the CTA-pair, 256 x 256 and split-contraction kernels (ragged edges, K not a multiple of
    # the k-block, batches, transposed operands, bias / addend epilogues); sampled rows against float64.
    rng = np.random.Generator(np.random.PCG64(777 + mode))
    for case in range(10):
        M, N = int(rng.integers(129, 2600)), int(rng.integers(129, 2600))
        K = int(rng.integers(64, 6000)) if case % 3 else int(rng.integers(6000, 40000))
        if case % 3 == 0:
            M, N = int(rng.integers(64, 600)), int(rng.integers(64, 600))     # long contraction, small output
        nb = int(rng.integers(1, 3)) if M * N * K < 2e9 else 1
        ta, tb = bool(rng.integers(0, 2)), bool(rng.integers(0, 2))
        a = uniform((nb, K, M) if ta else (nb, M, K), 1000 + case)
        b = uniform((N, K) if tb else (K, N), 2000 + case)
        A, B = dev(a), dev(b)
        Av = A.transpose(1, 2) if ta else A
        Bv = B.transpose(0, 1) if tb else B
        an = np.swapaxes(a, 1, 2) if ta else a
        bn = b.T if tb else b
        rows = sorted(set(int(r) for r in rng.integers(0, M, 5)) | {0, M - 1})
        ref = an[:, rows].astype(np.float64) @ bn.astype(np.float64)
        what = (case, M, N, K, nb, ta, tb)
        c = cabi.matmul_fwd(Av, Bv, mode=mode).to_numpy()
        assert rel_fro(c[:, rows], ref) < tol, what
        d = normal((nb, M, N), 3000 + case)
        c2 = cabi.matmul_axpby(Av, Bv, 0.75, -1.5, dev(d), mode=mode).to_numpy()
        assert rel_fro(c2[:, rows], 0.75 * ref - 1.5 * d[:, rows]) < tol, what
        bias = normal((1, N), 4000 + case)
        c3 = cabi.matmul_fwd(Av, Bv, bias=dev(bias), mode=mode).to_numpy()
        assert rel_fro(c3[:, rows], ref + bias) < tol, what


@pytest.mark.parametrize("mode,tol", MODES)
def test_bias_gradient_handed_along_by_the_producing_kernel(mode, tol):
    # db of y = x W + b is the column sum of dy (broadcast-add backward of the reference). The kernel that WRITES
    # dy returns it: the backward product of the next layer (optionally through tanh'), or the MSE forward pass.
    rng = np.random.Generator(np.random.PCG64(77))
    for (M, K, N, batch) in ((1000, 520, 300, ()), (4096, 1024, 512, ()), (130, 96, 260, (3,)), (2500, 2600, 2700, ())):
        a = np.tanh(rng.standard_normal(batch + (M, K)).astype(np.float32))
        b = rng.standard_normal((K, N)).astype(np.float32) * np.float32(1 / np.sqrt(K))
        dc = rng.standard_normal(batch + (M, N)).astype(np.float32)
        A, B, G = dev(a), dev(b), dev(dc)
        for through_tanh in (False, True):
            da, db, cs = cabi.matmul_bwd_colsum(A, B, G, a_is_tanh=through_tanh, mode=mode)
            want_da, want_db = (cabi.matmul_bwd_tanh if through_tanh else cabi.matmul_bwd)(A, B, G, mode=mode)
            assert np.array_equal(da.to_numpy(), want_da.to_numpy())      # same product, same epilogue
            assert np.array_equal(db.to_numpy(), want_db.to_numpy())
            ref = da.to_numpy().astype(np.float64).reshape(-1, K).sum(axis=0)
            assert rel_fro(cs.to_numpy(), ref) < 1e-5, (M, K, N, batch, through_tanh)
            again = cabi.matmul_bwd_colsum(A, B, G, a_is_tanh=through_tanh, mode=mode)[2]
            assert np.array_equal(cs.to_numpy(), again.to_numpy())        # no atomics: repeatable bit for bit
    # MSE forward: loss, gradient and the gradient's column sums in one pass (and the odd-width fallback)
    import ctypes as C
    lib = cabi.lib()
    for rows, cols in ((4096, 1024), (37, 132), (50, 30)):
        p, t = rng.standard_normal((rows, cols)).astype(np.float32), rng.standard_normal((rows, cols)).astype(np.float32)
        P, T, D, L, S = dev(p), dev(t), DA((rows, cols)), DA((1,)), DA((cols,))
        cabi.check(lib.akr_mse_fwd_grad_colsum(cabi.fptr(P), cabi.fptr(T), cabi.fptr(L), cabi.fptr(D), cabi.fptr(S),
                                               rows, cols, None))
        d64 = p.astype(np.float64) - t.astype(np.float64)
        assert abs(L.to_numpy()[0] - (d64 ** 2).mean()) < 1e-5 * (d64 ** 2).mean()
        assert rel_fro(D.to_numpy(), 2 * d64 / d64.size) < 1e-6
        assert rel_fro(S.to_numpy(), (2 * d64 / d64.size).sum(axis=0)) < 1e-5
