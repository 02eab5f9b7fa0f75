"""GPU: the Python package (reference-facing API) end to end - autograd, Linear training step."""
import numpy as np
import pytest

from util import load_golden, uniform, normal, rel_fro, TOL_FP32, TOL_TF32
from oracle import matmul_oracle as mo

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ak():
    import aakaar_b200
    return aakaar_b200


@pytest.mark.parametrize("tf32,tol", [(False, TOL_FP32), (True, TOL_TF32)])
def test_config1_autograd(ak, tf32, tol):
    G, META = load_golden()
    ak.set_tf32(tf32)
    try:
        a = ak.from_numpy(uniform((512, 512), 101), "cuda", requires_grad=True)
        b = ak.from_numpy(uniform((512, 512), 102), "cuda", requires_grad=True)
        c = ak.matmul(a, b)
        assert c.requires_grad and c.shape == [512, 512] and c.device == "cuda"
        c.backward(ak.from_numpy(np.ones((512, 512), np.float32), "cuda"))
        rows = META["cases"]["cfg1"]["rows"]
        assert rel_fro(c.to_numpy()[rows], G["cfg1_c_rows"]) < tol
        assert rel_fro(a.grad.to_numpy()[rows], G["cfg1_da_rows"]) < tol
        assert rel_fro(b.grad.to_numpy()[rows], G["cfg1_db_rows"]) < tol
    finally:
        ak.set_tf32(False)


def test_doc_example_and_shared_operand(ak):
    G, META = load_golden()
    a = ak.from_numpy(np.array(META["cases"]["doc"]["a"], np.float32), "cuda", requires_grad=True)
    b = ak.from_numpy(np.array(META["cases"]["doc"]["b"], np.float32), "cuda", requires_grad=True)
    r = ak.matmul(a, b)
    assert r.shape == [2, 2]
    r.sum().backward()
    np.testing.assert_allclose(r.to_numpy(), G["doc_c"], rtol=1e-6)
    np.testing.assert_allclose(a.grad.to_numpy(), G["doc_da"], rtol=1e-6)
    np.testing.assert_allclose(b.grad.to_numpy(), G["doc_db"], rtol=1e-6)
    s = ak.from_numpy(uniform((6, 6), 41), "cuda", requires_grad=True)
    c = s @ s
    c.backward(ak.from_numpy(np.ones((6, 6), np.float32), "cuda"))
    assert rel_fro(c.to_numpy(), G["ss_c"]) < TOL_FP32
    assert rel_fro(s.grad.to_numpy(), G["ss_ds"]) < TOL_FP32


def test_strided_view_autograd_and_only_needed_grads(ak):
    G, _ = load_golden()
    base = ak.from_numpy(uniform((4, 2, 6, 16), 301), "cuda", requires_grad=True)
    b = ak.from_numpy(uniform((1, 2, 6, 16), 302), "cuda", requires_grad=True)
    a = base.transpose(-1, -2)
    assert not a.is_contiguous()
    c = ak.matmul(a, b)               # the reference raises ValueError here
    c.backward(ak.from_numpy(np.ones(c.shape, np.float32), "cuda"))
    assert rel_fro(c.to_numpy(), G["cfg3s_c"]) < TOL_FP32
    assert base.grad.shape == [4, 2, 6, 16] and b.grad.shape == [1, 2, 6, 16]
    assert rel_fro(base.grad.to_numpy(), G["cfg3s_dbase"]) < TOL_FP32
    assert rel_fro(b.grad.to_numpy(), G["cfg3s_db"]) < TOL_FP32
    x = ak.from_numpy(uniform((8, 4), 1), "cuda")
    w = ak.from_numpy(uniform((4, 3), 2), "cuda", requires_grad=True)
    y = x @ w
    assert y.requires_grad
    y.backward(ak.from_numpy(np.ones((8, 3), np.float32), "cuda"))
    assert x.grad is None and w.grad is not None


def test_backward_rules(ak):
    a = ak.from_numpy(uniform((4, 4), 1), "cuda", requires_grad=True)
    b = ak.from_numpy(uniform((4, 4), 2), "cuda")
    c = a @ b
    with pytest.raises(RuntimeError, match="explicit gradient"):
        c.backward()
    g = ak.from_numpy(np.ones((4, 4), np.float32), "cuda")
    c.backward(g)
    with pytest.raises(RuntimeError, match="second time"):
        c.backward(g)
    c2 = a @ b
    c2.backward(g, retain_graph=True)
    c2.backward(g)
    with ak.no_grad():
        assert not (a @ b).requires_grad
    with pytest.raises(ValueError, match="inner dimensions must match"):
        ak.matmul(a, ak.from_numpy(np.ones((3, 2), np.float32), "cuda"))
    with pytest.raises(ValueError, match="at least 2 dimensions"):
        ak.matmul(a, ak.from_numpy(np.ones((4,), np.float32), "cuda"))


@pytest.mark.parametrize("tf32,tol", [(False, 2e-5), (True, 4e-3)])
def test_mlp_training_step_small(ak, tf32, tol):
    G, _ = load_golden()
    ak.set_tf32(tf32)
    try:
        np.random.seed(203)
        l1, l2 = ak.nn.Linear(32, 48), ak.nn.Linear(48, 16)
        x = ak.from_numpy(normal((64, 32), 201), "cuda")
        t = ak.from_numpy(normal((64, 16), 202), "cuda")
        opt = ak.optim.SGD(l1.parameters() + l2.parameters(), lr=0.01)
        y = l2(l1(x).tanh())
        loss = ak.mse_loss(y, t)
        loss.backward()
        assert abs(loss.item() / float(G["mlp_loss"].ravel()[0]) - 1) < tol
        assert rel_fro(y.to_numpy(), G["mlp_y"]) < tol
        for n, p in (("w1", l1.weight), ("b1", l1.bias), ("w2", l2.weight), ("b2", l2.bias)):
            assert p.grad.shape == p.shape
            assert rel_fro(p.grad.to_numpy(), G[f"mlp_d{n}"]) < tol, n
        opt.step()
        for n, p in (("w1", l1.weight), ("b1", l1.bias), ("w2", l2.weight), ("b2", l2.bias)):
            assert rel_fro(p.to_numpy(), G[f"mlp_new_{n}"]) < tol, n
        opt.zero_grad()
        assert l1.weight.grad is None
    finally:
        ak.set_tf32(False)


@pytest.mark.parametrize("tf32,tol", [(False, 2e-5), (True, 4e-3)])
def test_mlp_config2_full_size(ak, tf32, tol):
    # input [4096,1024], Linear 1024->4096, tanh, Linear 4096->1024, MSE, SGD lr 0.01; vs the oracle
    ak.set_tf32(tf32)
    try:
        np.random.seed(203)
        l1, l2 = ak.nn.Linear(1024, 4096), ak.nn.Linear(4096, 1024)
        w1, w2 = l1.weight.to_numpy(), l2.weight.to_numpy()
        xn, tn = normal((4096, 1024), 201), normal((4096, 1024), 202)
        x, t = ak.from_numpy(xn, "cuda"), ak.from_numpy(tn, "cuda")
        opt = ak.optim.SGD(l1.parameters() + l2.parameters(), lr=0.01)
        loss = ak.mse_loss(l2(l1(x).tanh()), t)
        loss.backward()
        opt.step()
        ak.synchronize()
        rloss, new, grads = mo.mlp_step(xn, tn, w1, np.zeros((1, 4096), np.float32), w2,
                                        np.zeros((1, 1024), np.float32), 0.01)
        assert abs(loss.item() / float(rloss) - 1) < tol
        assert rel_fro(l1.weight.grad.to_numpy(), grads["w1"]) < tol
        assert rel_fro(l2.weight.grad.to_numpy(), grads["w2"]) < tol
        assert rel_fro(l1.bias.grad.to_numpy(), grads["b1"]) < tol
        assert rel_fro(l2.bias.grad.to_numpy(), grads["b2"]) < tol
        assert rel_fro(l1.weight.to_numpy(), new[0]) < tol
    finally:
        ak.set_tf32(False)


def test_newton_schulz_chain_through_views(ak):
    # The Muon optimiser's orthogonalisation step (aakaar/optim.py:533-542) is a chain of products on
    # transposed operands; here the transposes stay views (the reference materialises them).
    x_np = uniform((64, 160), 9) * np.float32(0.05)
    a_, b_, c_ = 3.4445, -4.7750, 2.0315
    X = ak.from_numpy(x_np, "cuda")
    ref = x_np.astype(np.float64)
    with ak.no_grad():
        for _ in range(3):
            A = X @ X.T                      # [64,64], second operand is a strided view
            B = A * b_ + (A @ A) * c_
            X = X * a_ + B @ X
            Ar = ref @ ref.T
            ref = a_ * ref + (b_ * Ar + c_ * (Ar @ Ar)) @ ref
    assert rel_fro(X.to_numpy(), ref) < 1e-5


def test_typed_forward_only_matmul(ak):
    # float64 / int32 / int64: forward product with broadcasting, no autograd (as in the reference)
    G, META = load_golden()
    g = np.random.Generator(np.random.PCG64(77))
    a64, b64 = g.standard_normal((3, 1, 9, 14)), g.standard_normal((2, 14, 11))
    c = ak.matmul(ak.from_numpy(a64, "cuda"), ak.from_numpy(b64, "cuda"))
    assert c.dtype == "float64" and c.shape == [3, 2, 9, 11] and not c.requires_grad
    assert rel_fro(c.to_numpy(), G["f64_c"]) < 1e-14
    ai32 = g.integers(-2 ** 20, 2 ** 20, (17, 23)).astype(np.int32)
    bi32 = g.integers(-2 ** 20, 2 ** 20, (23, 13)).astype(np.int32)
    np.testing.assert_array_equal(ak.matmul(ak.from_numpy(ai32, "cuda"), ak.from_numpy(bi32, "cuda")).to_numpy(), G["i32_c"])
    ai64 = g.integers(-2 ** 40, 2 ** 40, (2, 5, 7)).astype(np.int64)
    bi64 = g.integers(-2 ** 20, 2 ** 20, (7, 4)).astype(np.int64)
    np.testing.assert_array_equal(ak.matmul(ak.from_numpy(ai64, "cuda"), ak.from_numpy(bi64, "cuda")).to_numpy(), G["i64_c"])
    with pytest.raises(RuntimeError, match="share one dtype"):
        ak.matmul(ak.from_numpy(a64, "cuda"), ak.from_numpy(b64.astype(np.float32), "cuda"))
    with pytest.raises(RuntimeError, match="only float32"):
        ak.from_numpy(a64, "cuda").tanh()


def test_tanh_backward_folded_into_next_matmul(ak):
    # Linear -> tanh -> Linear -> MSE: with the fusion the tanh node's backward runs inside the epilogue
    # of the second layer's dA product and both bias gradients are handed along by the kernels that write
    # the gradients they are column sums of (the MSE forward pass, the dA epilogue): fewer launches in the
    # backward pass (TF32 mode: 4 instead of 8), gradients unchanged
    from aakaar_b200 import _C
    x, tgt = normal((96, 40), 1), normal((96, 24), 2)
    w1, b1 = uniform((40, 72), 3) * 0.2, uniform((1, 72), 4) * 0.1
    w2, b2 = uniform((72, 24), 5) * 0.2, uniform((1, 24), 6) * 0.1
    _, _, ref = mo.mlp_step(x, tgt, w1, b1, w2, b2, 0.0, np.float64)
    for tf32, tol in ((False, TOL_FP32), (True, TOL_TF32)):
        results = {}
        ak.set_tf32(tf32)
        try:
            for fused in (False, True):
                _C._set_backward_fusion(fused)
                X, Tg = ak.from_numpy(x), ak.from_numpy(tgt)
                P = [ak.from_numpy(v, requires_grad=True) for v in (w1, b1, w2, b2)]
                h = _C.linear(X, P[0], P[1]).tanh()
                loss = ak.mse_loss(_C.linear(h, P[2], P[3]), Tg)
                ak.synchronize()
                _C._launch_count(True)
                loss.backward()
                ak.synchronize()
                results[fused] = ([p.grad.to_numpy() for p in P], _C._launch_count(True))
        finally:
            _C._set_backward_fusion(True)
            ak.set_tf32(False)
        (g0, n0), (g1, n1) = results[False], results[True]
        assert n1 < n0 and (not tf32 or n1 <= n0 - 3), (tf32, n0, n1)
        for got0, got1, key in zip(g0, g1, ("w1", "b1", "w2", "b2")):
            assert rel_fro(got1, ref[key]) < tol, key
            assert rel_fro(got1, got0) < tol, key
    # a tanh output with a second consumer is not fused (its gradient has two contributions)
    Z = ak.from_numpy(normal((16, 8), 7), requires_grad=True)
    W = ak.from_numpy(uniform((8, 8), 8), requires_grad=True)
    h = Z.tanh()
    out = (_C.cuda_matmul(h, W) + h).sum()
    out.backward()
    zn, wn = normal((16, 8), 7).astype(np.float64), uniform((8, 8), 8).astype(np.float64)
    hn = np.tanh(zn)
    dz = (np.ones((16, 8)) @ wn.T + 1.0) * (1 - hn * hn)
    assert rel_fro(Z.grad.to_numpy(), dz) < TOL_FP32


def test_muon_optimizer_matches_reference(ak):
    G, META = load_golden()
    P = ak.from_numpy(uniform((24, 40), 45), requires_grad=True)
    vec = ak.from_numpy(uniform((40,), 49), requires_grad=True)          # 1-D parameter: plain momentum update
    opt = ak.optim.Muon([P, vec], lr=0.02, momentum=0.95, ns_steps=5, weight_decay=0.01)
    v_ref, v_buf = uniform((40,), 49), None
    for seed in (46, 47):
        P.grad = ak.from_numpy(normal((24, 40), seed))
        vec.grad = ak.from_numpy(normal((40,), seed + 10))
        opt.step()
        v_ref, v_buf = mo.muon_step(v_ref, normal((40,), seed + 10), v_buf, weight_decay=0.01)
    assert rel_fro(P.to_numpy(), G["muon_p2"]) < TOL_FP32
    assert rel_fro(vec.to_numpy(), v_ref) < TOL_FP32
    opt.zero_grad()
    assert P.grad is None


@pytest.mark.parametrize("tf32,tol", [(False, TOL_FP32), (True, TOL_TF32)])
def test_conv_fallback_callers(ak, tf32, tol):
    # conv1d / conv2d as unfold + ONE broadcast-batched matmul, forward and backward, against the vectors of
    # the reference's own im2col + matmul composition
    G, META = load_golden()
    ak.set_tf32(tf32)
    try:
        X1 = ak.from_numpy(normal((3, 4, 19), 51), requires_grad=True)
        W1 = ak.from_numpy(uniform((5, 4, 3), 52), requires_grad=True)
        Y1 = ak.conv1d(X1, W1, stride=2, padding=2, dilation=2)
        assert Y1.shape == list(G["conv1d_y"].shape)
        Y1.backward(ak.from_numpy(normal(tuple(Y1.shape), 53)))
        assert rel_fro(Y1.to_numpy(), G["conv1d_y"]) < tol
        assert rel_fro(X1.grad.to_numpy(), G["conv1d_dx"]) < tol and rel_fro(W1.grad.to_numpy(), G["conv1d_dw"]) < tol
        X2 = ak.from_numpy(normal((2, 3, 9, 11), 54), requires_grad=True)
        W2 = ak.from_numpy(uniform((4, 3, 3, 2), 55), requires_grad=True)
        Y2 = ak.conv2d(X2, W2, stride=(2, 1), padding=(1, 0), dilation=(1, 2))
        assert Y2.shape == list(G["conv2d_y"].shape)
        Y2.backward(ak.from_numpy(normal(tuple(Y2.shape), 56)))
        assert rel_fro(Y2.to_numpy(), G["conv2d_y"]) < tol
        assert rel_fro(X2.grad.to_numpy(), G["conv2d_dx"]) < tol and rel_fro(W2.grad.to_numpy(), G["conv2d_dw"]) < tol
        # a larger case against the oracle: 3x3, 64 -> 128 channels, 32 x 32 images, batch 8
        x, w = normal((8, 64, 32, 32), 57), uniform((128, 64, 3, 3), 58) * 0.05
        dy = normal((8, 128, 32, 32), 59)
        X, W = ak.from_numpy(x, requires_grad=True), ak.from_numpy(w, requires_grad=True)
        Y = ak.conv2d(X, W, padding=(1, 1))
        Y.backward(ak.from_numpy(dy))
        ry, rdx, rdw = mo.conv2d_forward_backward(x, w, dy, (1, 1), (1, 1), (1, 1), np.float64)
        assert rel_fro(Y.to_numpy(), ry) < tol
        assert rel_fro(X.grad.to_numpy(), rdx) < tol and rel_fro(W.grad.to_numpy(), rdw) < tol
    finally:
        ak.set_tf32(False)


@pytest.mark.parametrize("tf32,tol", [(False, TOL_FP32), (True, TOL_TF32)])
def test_conv3d_and_transposed_convolutions(ak, tf32, tol):
    # conv3d (unfold + one broadcast-batched matmul) and conv_transpose{1,2,3}d (matmul with the weights read as a
    # transposed view + fold), forward and backward, against the vectors of the reference's own compositions;
    # then a non-cubic transposed kernel (beyond what the reference's fold accepts) against the oracle
    G, _ = load_golden()
    ak.set_tf32(tf32)
    try:
        X = ak.from_numpy(normal((2, 3, 5, 6, 7), 61), requires_grad=True)
        W = ak.from_numpy(uniform((4, 3, 2, 3, 2), 62), requires_grad=True)
        Y = ak.conv3d(X, W, stride=(2, 1, 1), padding=(1, 0, 1), dilation=(1, 1, 2))
        assert Y.shape == list(G["conv3d_y"].shape)
        Y.backward(ak.from_numpy(normal(tuple(Y.shape), 63)))
        assert rel_fro(Y.to_numpy(), G["conv3d_y"]) < tol
        assert rel_fro(X.grad.to_numpy(), G["conv3d_dx"]) < tol and rel_fro(W.grad.to_numpy(), G["conv3d_dw"]) < tol
        for name, fn, xs, ws, st, pd, dl, seed in (
                ("convT1d", ak.conv_transpose1d, (3, 4, 9), (4, 5, 3), 2, 1, 2, 64),
                ("convT2d", ak.conv_transpose2d, (2, 3, 5, 6), (3, 4, 3, 3), (2, 1), (1, 0), (1, 2), 67),
                ("convT3d", ak.conv_transpose3d, (2, 3, 3, 4, 5), (3, 2, 2, 2, 2), (1, 2, 1), (0, 1, 0), (1, 1, 2), 70)):
            X = ak.from_numpy(normal(xs, seed + 1), requires_grad=True)
            W = ak.from_numpy(uniform(ws, seed + 2), requires_grad=True)
            Y = fn(X, W, stride=st, padding=pd, dilation=dl)
            assert Y.shape == list(G[name + "_y"].shape), name
            Y.backward(ak.from_numpy(normal(tuple(Y.shape), seed)))
            assert rel_fro(Y.to_numpy(), G[name + "_y"]) < tol, name
            assert rel_fro(X.grad.to_numpy(), G[name + "_dx"]) < tol, name
            assert rel_fro(W.grad.to_numpy(), G[name + "_dw"]) < tol, name
        x, w = normal((4, 16, 12, 10), 81), uniform((16, 24, 3, 2), 82) * 0.2
        X, W = ak.from_numpy(x, requires_grad=True), ak.from_numpy(w, requires_grad=True)
        Y = ak.conv_transpose2d(X, W, stride=(2, 3), padding=(1, 0))
        dy = normal(tuple(Y.shape), 83)
        Y.backward(ak.from_numpy(dy))
        ry, rdx, rdw = mo.conv_transpose_nd_forward_backward(x, w, dy, (2, 3), (1, 0), (1, 1), np.float64)
        assert rel_fro(Y.to_numpy(), ry) < tol
        assert rel_fro(X.grad.to_numpy(), rdx) < tol and rel_fro(W.grad.to_numpy(), rdw) < tol
        with pytest.raises(NotImplementedError):
            ak.conv_transpose1d(X, W, output_padding=1)
    finally:
        ak.set_tf32(False)
    # modules: parameters drawn as the reference draws them, bias added, its gradient the sum over batch and positions
    np.random.seed(11)
    m = ak.nn.ConvTranspose2d(3, 5, 3, stride=2, padding=1)
    np.random.seed(11)
    lim = 1.0 / np.sqrt(3 * 9)
    w = np.random.uniform(-lim, lim, (3, 5, 3, 3)).astype(np.float32)
    b = np.random.uniform(-lim, lim, (1, 5, 1, 1)).astype(np.float32)
    np.testing.assert_array_equal(m.weight.to_numpy(), w)
    np.testing.assert_array_equal(m.bias.to_numpy(), b)
    x = normal((2, 3, 6, 7), 84)
    X = ak.from_numpy(x, requires_grad=True)
    y = m(X)
    dy = normal(tuple(y.shape), 85)
    y.backward(ak.from_numpy(dy))
    ry, rdx, rdw = mo.conv_transpose_nd_forward_backward(x, w, dy, (2, 2), (1, 1), (1, 1), np.float64)
    assert rel_fro(y.to_numpy(), ry + b) < TOL_FP32
    assert rel_fro(X.grad.to_numpy(), rdx) < TOL_FP32 and rel_fro(m.weight.grad.to_numpy(), rdw) < TOL_FP32
    assert rel_fro(m.bias.grad.to_numpy(), dy.sum(axis=(0, 2, 3), keepdims=True)) < TOL_FP32
    c3 = ak.nn.Conv3d(2, 3, (2, 1, 2), padding=(1, 0, 0))
    x3 = normal((2, 2, 4, 3, 5), 86)
    y3 = c3(ak.from_numpy(x3))
    ry3, _, _ = mo.conv_nd_forward_backward(x3, c3.weight.to_numpy(), np.zeros(tuple(y3.shape), np.float32), (1, 1, 1),
                                            (1, 0, 0), (1, 1, 1), np.float64)
    assert rel_fro(y3.to_numpy(), ry3 + c3.bias.to_numpy()) < TOL_FP32


def test_conv_modules_with_bias(ak):
    np.random.seed(7)
    conv = ak.nn.Conv2d(3, 5, (3, 2), stride=(2, 1), padding=(1, 0), dilation=(1, 2))
    np.random.seed(7)
    w = np.random.uniform(-1 / np.sqrt(18), 1 / np.sqrt(18), (5, 3, 3, 2)).astype(np.float32)
    b = np.random.uniform(-1 / np.sqrt(18), 1 / np.sqrt(18), (1, 5, 1, 1)).astype(np.float32)
    np.testing.assert_array_equal(conv.weight.to_numpy(), w)
    np.testing.assert_array_equal(conv.bias.to_numpy(), b)
    x = normal((2, 3, 9, 11), 61)
    X = ak.from_numpy(x, requires_grad=True)
    y = conv(X)
    dy = normal(tuple(y.shape), 62)
    y.backward(ak.from_numpy(dy))
    ry, rdx, rdw = mo.conv2d_forward_backward(x, w, dy, (2, 1), (1, 0), (1, 2), np.float64)
    assert rel_fro(y.to_numpy(), ry + b) < TOL_FP32
    assert rel_fro(X.grad.to_numpy(), rdx) < TOL_FP32 and rel_fro(conv.weight.grad.to_numpy(), rdw) < TOL_FP32
    assert rel_fro(conv.bias.grad.to_numpy(), dy.sum(axis=(0, 2, 3), keepdims=True)) < TOL_FP32
    c1 = ak.nn.Conv1d(4, 6, 3, padding=1, bias=False)
    assert c1(ak.from_numpy(normal((2, 4, 16), 63))).shape == [2, 6, 16] and len(c1.parameters()) == 1
    with pytest.raises(ValueError, match="input channels"):
        c1(ak.from_numpy(normal((2, 5, 16), 64)))


def test_readme_training_example(ak):
    # README.md:101-137 of the reference, verbatim apart from the import: K = 1 and N = 1 products, the
    # example's own mse through tensor * tensor, 300 SGD steps; losses against the reference's own run
    G, META = load_golden()
    from aakaar_b200.nn import Linear
    from aakaar_b200.optim import SGD
    np.random.seed(0)
    N = 64
    x_np = np.linspace(-3, 3, N).reshape(N, 1).astype(np.float32)
    y_np = np.sin(x_np).astype(np.float32)
    x, y = ak.from_numpy(x_np), ak.from_numpy(y_np)
    fc1, fc2 = Linear(1, 16), Linear(16, 1)

    def forward(x):
        return fc2(fc1(x).tanh())

    def mse_loss(pred, target):
        diff = pred - target
        return (diff * diff).sum() / pred.size

    opt = SGD(fc1.parameters() + fc2.parameters(), lr=0.05)
    losses = []
    for epoch in range(300):
        opt.zero_grad()
        loss = mse_loss(forward(x), y)
        loss.backward()
        opt.step()
        losses.append(loss.item())
    got = np.array([losses[0], losses[1], losses[2], losses[99], losses[299]])
    np.testing.assert_allclose(got[:3], G["readme_losses"][:3], rtol=1e-5)
    np.testing.assert_allclose(got[3:], G["readme_losses"][3:], rtol=2e-3)   # 100 - 300 chained fp32 steps
    assert got[-1] < 0.05 * got[0]


def test_autograd_through_getitem_views(ak):
    # Tensor.__getitem__ records a node (src/bindings.cpp:2670-2727): the incoming gradient lands in a zero
    # tensor of the base's shape at the positions the view covers. Slices feed the strided matmul path.
    a = uniform((6, 10, 12), 91)
    b = uniform((12, 7), 92)
    A = ak.from_numpy(a, requires_grad=True)
    B = ak.from_numpy(b, requires_grad=True)
    sub = A[1:5, 2:10:2]                      # [4, 4, 12] with a stepped middle dim
    assert sub.requires_grad and sub.shape == [4, 4, 12]
    out = ak.matmul(sub, B)
    dy = normal((4, 4, 7), 93)
    out.backward(ak.from_numpy(dy))
    a64, b64 = a.astype(np.float64), b.astype(np.float64)
    ref_da = np.zeros_like(a64)
    ref_da[1:5, 2:10:2] = dy.astype(np.float64) @ b64.T
    ref_db = np.einsum("ijk,ijn->kn", a64[1:5, 2:10:2], dy.astype(np.float64))
    assert rel_fro(A.grad.to_numpy(), ref_da) < TOL_FP32
    assert rel_fro(B.grad.to_numpy(), ref_db) < TOL_FP32
    # an integer index drops a dim; two views of one base accumulate into its gradient
    W = ak.from_numpy(uniform((5, 8, 8), 94), requires_grad=True)
    x = ak.from_numpy(uniform((3, 8), 95))
    y = ak.matmul(x, W[2]) + ak.matmul(x, W[-1])
    y.sum().backward()
    ref = np.zeros((5, 8, 8))
    ref[2] = ref[4] = uniform((3, 8), 95).astype(np.float64).T @ np.ones((3, 8))
    assert rel_fro(W.grad.to_numpy(), ref) < TOL_FP32
    with pytest.raises(IndexError):
        W[7]


def test_optimizers_step_view_parameters(ak):
    # a parameter that is a transposed view takes the same update as its dense twin (the reference's unfused
    # fallback, aakaar/optim.py:24-48), written back through the view's strides
    base = uniform((6, 4), 96)
    g = normal((4, 6), 97)
    P = ak.from_numpy(base).transpose(0, 1)        # [4, 6], non-contiguous
    P.requires_grad = True
    P.grad = ak.from_numpy(g)
    opt = ak.optim.SGD([P], lr=0.1, momentum=0.9, weight_decay=0.01)
    opt.step()
    opt.step()
    p = base.T.astype(np.float64).copy()
    g64 = g.astype(np.float64)
    v = None
    for _ in range(2):
        gg = g64 + 0.01 * p
        v = gg if v is None else 0.9 * v + gg
        p = p - 0.1 * v
    assert not P.is_contiguous()
    assert rel_fro(P.contiguous().to_numpy(), p) < TOL_FP32


@pytest.mark.parametrize("momentum,nesterov,dampening,wd", [(0.0, False, 0.0, 0.0), (0.0, False, 0.0, 0.05),
                                                             (0.9, False, 0.1, 0.01), (0.8, True, 0.0, 0.0)])
def test_sgd_steps_a_parameter_list_in_one_launch(ak, momentum, nesterov, dampening, wd):
    # SGD.step (aakaar/optim.py:24-48 -> src/optim_kernels.cu:21-55) over several tensors of odd sizes: one
    # launch for the whole list, same arithmetic as one launch per tensor
    from aakaar_b200 import _C
    shapes = [(300, 40), (1, 40), (5000,), (3,), (64, 64)]
    ps = [uniform(s, 100 + i) for i, s in enumerate(shapes)]
    gs = [[normal(s, 200 + 10 * step + i) for i, s in enumerate(shapes)] for step in range(3)]
    P = [ak.from_numpy(p, requires_grad=True) for p in ps]
    opt = ak.optim.SGD(P, lr=0.05, momentum=momentum, weight_decay=wd, dampening=dampening, nesterov=nesterov)
    ref = [p.astype(np.float64) for p in ps]
    vel = [None] * len(ps)
    for step in range(3):
        for t, g in zip(P, gs[step]):
            t.grad = ak.from_numpy(g)
        ak.synchronize()
        _C._launch_count(True)
        opt.step()
        ak.synchronize()
        assert _C._launch_count(True) == 1
        for i, g in enumerate(gs[step]):
            gg = g.astype(np.float64) + wd * ref[i]
            if momentum != 0:
                vel[i] = gg if vel[i] is None else momentum * vel[i] + (1 - dampening) * gg
                upd = gg + momentum * vel[i] if nesterov else vel[i]
            else:
                upd = gg
            ref[i] = ref[i] - 0.05 * upd
    for t, r in zip(P, ref):
        assert rel_fro(t.to_numpy(), r) < TOL_FP32
