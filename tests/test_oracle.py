"""CPU: the numpy restatement (oracle/) against the reference's own outputs and doc examples."""
import numpy as np
import pytest

from util import load_golden, uniform, normal, rel_fro
from oracle import matmul_oracle as mo

G, META = load_golden()
TOL = 2e-6  # two fp32 sgemm implementations differ only by summation order


def test_doc_example_known_answer():
    # docs/concepts/math-operations/matmul.md:36-57 - values follow from the inputs printed there
    a = np.array(META["cases"]["doc"]["a"], dtype=np.float32)
    b = np.array(META["cases"]["doc"]["b"], dtype=np.float32)
    c = mo.matmul_forward(a, b)
    np.testing.assert_array_equal(c, np.array([[22, 28], [49, 64]], dtype=np.float32))
    da, db = mo.matmul_backward(a, b, np.ones((2, 2), np.float32))
    np.testing.assert_array_equal(da, np.array([[3, 7, 11], [3, 7, 11]], dtype=np.float32))
    np.testing.assert_array_equal(db, np.array([[5, 5], [7, 7], [9, 9]], dtype=np.float32))
    # and the reference produced exactly these
    np.testing.assert_array_equal(G["doc_c"], c)
    np.testing.assert_array_equal(G["doc_da"], da)
    np.testing.assert_array_equal(G["doc_db"], db)


def test_config1_against_reference_rows():
    a, b = uniform((512, 512), 101), uniform((512, 512), 102)
    c = mo.matmul_forward(a, b)
    da, db = mo.matmul_backward(a, b, np.ones((512, 512), np.float32))
    rows = META["cases"]["cfg1"]["rows"]
    for name, arr in (("c", c), ("da", da), ("db", db)):
        assert rel_fro(arr[rows], G[f"cfg1_{name}_rows"]) < TOL
        assert abs(np.linalg.norm(arr.astype(np.float64)) / G[f"cfg1_{name}_norm"][0] - 1) < 1e-6


@pytest.mark.parametrize("acc", [np.float32, np.float64])
def test_nd_broadcast_cases(acc):
    a, b, dc = uniform((3, 1, 5, 7), 11), uniform((2, 7, 4), 12), normal((3, 2, 5, 4), 13)
    assert rel_fro(mo.matmul_forward(a, b, acc), G["nd_c"]) < TOL
    da, db = mo.matmul_backward(a, b, dc, acc)
    assert da.shape == a.shape and db.shape == b.shape
    assert rel_fro(da, G["nd_da"]) < TOL and rel_fro(db, G["nd_db"]) < TOL

    a, b, dc = uniform((2, 3, 8), 21), uniform((8, 5), 22), normal((2, 3, 5), 23)
    assert rel_fro(mo.matmul_forward(a, b, acc), G["bt_c"]) < TOL
    da, db = mo.matmul_backward(a, b, dc, acc)
    assert db.shape == (8, 5)
    assert rel_fro(da, G["bt_da"]) < TOL and rel_fro(db, G["bt_db"]) < TOL


def test_transposed_view_case_matches_reference():
    base, b = uniform((4, 2, 6, 16), 301), uniform((1, 2, 6, 16), 302)
    a = np.ascontiguousarray(np.swapaxes(base, -1, -2))
    c = mo.matmul_forward(a, b)
    assert rel_fro(c, G["cfg3s_c"]) < TOL
    da, db = mo.matmul_backward(a, b, np.ones(c.shape, np.float32))
    assert db.shape == (1, 2, 6, 16)
    assert rel_fro(np.swapaxes(da, -1, -2), G["cfg3s_dbase"]) < TOL
    assert rel_fro(db, G["cfg3s_db"]) < TOL


def test_ragged_and_shared_operand():
    a, b, dc = uniform((77, 45), 31), uniform((45, 19), 32), normal((77, 19), 33)
    assert rel_fro(mo.matmul_forward(a, b), G["rag_c"]) < TOL
    da, db = mo.matmul_backward(a, b, dc)
    assert rel_fro(da, G["rag_da"]) < TOL and rel_fro(db, G["rag_db"]) < TOL
    s = uniform((6, 6), 41)
    da, db = mo.matmul_backward(s, s, np.ones((6, 6), np.float32))
    assert rel_fro(mo.matmul_forward(s, s), G["ss_c"]) < TOL
    assert rel_fro(da + db, G["ss_ds"]) < TOL


def test_mlp_step_matches_reference():
    x, tgt = normal((64, 32), 201), normal((64, 16), 202)
    rng = np.random.RandomState(203)
    w1 = rng.uniform(-1 / np.sqrt(32), 1 / np.sqrt(32), (32, 48)).astype(np.float32)
    w2 = rng.uniform(-1 / np.sqrt(48), 1 / np.sqrt(48), (48, 16)).astype(np.float32)
    b1, b2 = np.zeros((1, 48), np.float32), np.zeros((1, 16), np.float32)
    loss, new, grads = mo.mlp_step(x, tgt, w1, b1, w2, b2, 0.01)
    assert abs(float(loss) / float(G["mlp_loss"].ravel()[0]) - 1) < 1e-5
    assert rel_fro(grads["y"], G["mlp_y"]) < TOL
    for n in ("w1", "b1", "w2", "b2"):
        assert rel_fro(grads[n], G[f"mlp_d{n}"]) < 5e-6, n
    for n, p in zip(("w1", "b1", "w2", "b2"), new):
        assert rel_fro(p, G[f"mlp_new_{n}"]) < 1e-6, n


def test_error_behaviour_follows_reference():
    errs = META["errors"]
    with pytest.raises(ValueError) as e:
        mo.matmul_forward(np.ones((2, 3), np.float32), np.ones((4, 2), np.float32))
    assert str(e.value).startswith(errs["k_mismatch"][1])
    with pytest.raises(ValueError) as e:
        mo.matmul_forward(np.ones((2, 2, 3), np.float32), np.ones((3, 3, 2), np.float32))
    assert str(e.value) == errs["batch_mismatch"][1]
    with pytest.raises(ValueError) as e:
        mo.matmul_forward(np.ones((2, 3), np.float32).T, np.ones((2, 2), np.float32))
    assert str(e.value) == errs["non_contiguous"][1]
    with pytest.raises(ValueError):
        mo.plan_nd_matmul((3,), (3, 2))


def test_batch_offset_broadcast_rules():
    batch, M, K, N = mo.plan_nd_matmul((3, 1, 5, 7), (2, 7, 4))
    assert (batch, M, K, N) == ((3, 2), 5, 7, 4)
    # flat index 3 = (1, 1): A varies on dim0 only, B on dim1 only
    assert mo.batch_offset(3, batch, (3, 1, 5, 7), 35) == 35
    assert mo.batch_offset(3, batch, (2, 7, 4), 28) == 28
    assert mo.batch_offset(4, batch, (3, 1, 5, 7), 35) == 70
    assert mo.batch_offset(4, batch, (2, 7, 4), 28) == 0


def test_typed_forward_matches_reference():
    g = np.random.Generator(np.random.PCG64(77))
    a64, b64 = g.standard_normal((3, 1, 9, 14)), g.standard_normal((2, 14, 11))
    assert rel_fro(mo.matmul_forward_typed(a64, b64), G["f64_c"]) < 1e-14
    ai32 = g.integers(-2 ** 20, 2 ** 20, (17, 23)).astype(np.int32)
    bi32 = g.integers(-2 ** 20, 2 ** 20, (23, 13)).astype(np.int32)
    np.testing.assert_array_equal(mo.matmul_forward_typed(ai32, bi32), G["i32_c"])   # wraps like the reference
    ai64 = g.integers(-2 ** 40, 2 ** 40, (2, 5, 7)).astype(np.int64)
    bi64 = g.integers(-2 ** 20, 2 ** 20, (7, 4)).astype(np.int64)
    np.testing.assert_array_equal(mo.matmul_forward_typed(ai64, bi64), G["i64_c"])


def test_tanh_backward_and_newton_schulz_match_reference():
    z, b, dc = normal((13, 9), 41), uniform((9, 7), 42), normal((13, 7), 43)
    dz, db = mo.matmul_backward_tanh(np.tanh(z).astype(np.float32), b, dc)
    assert rel_fro(dz, G["tanhmm_dz"]) < 2e-6 and rel_fro(db, G["tanhmm_db"]) < 2e-6
    assert rel_fro(mo.newton_schulz(normal((24, 40), 44), 5), G["muon_ns5"]) < 1e-5
    a, b2, d = uniform((5, 4), 1), uniform((4, 6), 2), normal((5, 6), 3)
    np.testing.assert_allclose(mo.matmul_axpby(a, b2, 2.0, -3.0, d), 2.0 * (a @ b2) - 3.0 * d, rtol=1e-5, atol=1e-6)


def test_muon_steps_match_reference():
    p, buf = uniform((24, 40), 45), None
    for seed in (46, 47):
        p, buf = mo.muon_step(p, normal((24, 40), seed), buf, lr=0.02, momentum=0.95, ns_steps=5, weight_decay=0.01)
    assert rel_fro(p, G["muon_p2"]) < 1e-5


def test_conv_fallback_matches_reference():
    # 1-D = one image row: stride 2, padding 2, dilation 2
    x, w = normal((3, 4, 19), 51), uniform((5, 4, 3), 52)
    y, dx, dw = mo.conv2d_forward_backward(x[:, :, None, :], w[:, :, None, :], normal((3, 5, 10), 53)[:, :, None, :],
                                           (1, 2), (0, 2), (1, 2))
    assert rel_fro(y[:, :, 0, :], G["conv1d_y"]) < 2e-6
    assert rel_fro(dx[:, :, 0, :], G["conv1d_dx"]) < 2e-6 and rel_fro(dw[:, :, 0, :], G["conv1d_dw"]) < 2e-6
    x2, w2 = normal((2, 3, 9, 11), 54), uniform((4, 3, 3, 2), 55)
    y2, dx2, dw2 = mo.conv2d_forward_backward(x2, w2, normal(G["conv2d_y"].shape, 56), (2, 1), (1, 0), (1, 2))
    assert rel_fro(y2, G["conv2d_y"]) < 2e-6
    assert rel_fro(dx2, G["conv2d_dx"]) < 2e-6 and rel_fro(dw2, G["conv2d_dw"]) < 2e-6


def test_conv3d_and_transposed_convolutions_match_reference():
    # vectors of the reference's own im2col_3d / col2im_* + matmul compositions (tests/golden/make_golden.py 8g)
    G, _ = load_golden()
    x, w = normal((2, 3, 5, 6, 7), 61), uniform((4, 3, 2, 3, 2), 62)
    y, dx, dw = mo.conv_nd_forward_backward(x, w, normal(G["conv3d_y"].shape, 63), (2, 1, 1), (1, 0, 1), (1, 1, 2))
    assert rel_fro(y, G["conv3d_y"]) < 2e-6
    assert rel_fro(dx, G["conv3d_dx"]) < 2e-6 and rel_fro(dw, G["conv3d_dw"]) < 2e-6
    for name, xs, ws, st, pd, dl, seed in (("convT1d", (3, 4, 9), (4, 5, 3), (2,), (1,), (2,), 64),
                                           ("convT2d", (2, 3, 5, 6), (3, 4, 3, 3), (2, 1), (1, 0), (1, 2), 67),
                                           ("convT3d", (2, 3, 3, 4, 5), (3, 2, 2, 2, 2), (1, 2, 1), (0, 1, 0), (1, 1, 2), 70)):
        x, w = normal(xs, seed + 1), uniform(ws, seed + 2)
        y, dx, dw = mo.conv_transpose_nd_forward_backward(x, w, normal(G[name + "_y"].shape, seed), st, pd, dl)
        assert y.shape == G[name + "_y"].shape
        assert rel_fro(y, G[name + "_y"]) < 2e-6, name
        assert rel_fro(dx, G[name + "_dx"]) < 2e-6 and rel_fro(dw, G[name + "_dw"]) < 2e-6, name
    # the 2-D case through the N-D oracle agrees with the 2-D one
    x2, w2 = normal((2, 3, 9, 11), 54), uniform((4, 3, 3, 2), 55)
    y2, dx2, dw2 = mo.conv_nd_forward_backward(x2, w2, normal(G["conv2d_y"].shape, 56), (2, 1), (1, 0), (1, 2))
    assert rel_fro(y2, G["conv2d_y"]) < 2e-6 and rel_fro(dx2, G["conv2d_dx"]) < 2e-6 and rel_fro(dw2, G["conv2d_dw"]) < 2e-6
