"""Generates tests/golden/ref_vectors.npz by running the REFERENCE's own CPU build.

Run in the authoring container only (needs oracle/_ref built by oracle/build_ref.sh from the
reference checkout):  python tests/golden/make_golden.py

Every case records seeded inputs recipes (regenerated in the tests from the same seeds) and the
reference's outputs. Large outputs are stored as sampled rows plus norms so the file stays small.
Inputs come from numpy PCG64 generators, float32, exactly as tests/util.py regenerates them.
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle", "_ref"))
sys.path.insert(0, os.path.join(ROOT, "tests"))
import _C as ref  # noqa: E402  (the reference's pybind11 module, CPU build)

from util import uniform, normal  # noqa: E402


def T(x, grad=False):
    return ref.from_numpy(np.ascontiguousarray(x, dtype=np.float32), "cpu", grad)


def fwd_bwd(a_np, b_np, dc_np=None, contiguous_a=None):
    """Reference forward + backward. `contiguous_a`: a callable building A from its base tensor."""
    a = T(a_np, True)
    b = T(b_np, True)
    c = ref.cpu_matmul(a, b)
    if dc_np is None:
        dc_np = np.ones(c.shape, dtype=np.float32)
    c.backward(T(dc_np))
    return c.to_numpy(), a.grad.to_numpy(), b.grad.to_numpy()


out = {}
meta = {"generator": "reference CPU build (oracle/_ref), OpenBLAS 0.3.15", "cases": {}}

# 1. documentation example, docs/concepts/math-operations/matmul.md:36-57
a = np.array([[1, 2, 3], [4, 5, 6]], dtype=np.float32)
b = np.array([[1, 2], [3, 4], [5, 6]], dtype=np.float32)
A, B = T(a, True), T(b, True)
C = ref.cpu_matmul(A, B)
loss = C.sum()
loss.backward()
out["doc_c"], out["doc_da"], out["doc_db"] = C.to_numpy(), A.grad.to_numpy(), B.grad.to_numpy()
meta["cases"]["doc"] = {"a": a.tolist(), "b": b.tolist()}

# 2. config 1: 512^3, uniform[-1,1) seeds 101/102, dC = ones; sampled rows + norms
a, b = uniform((512, 512), 101), uniform((512, 512), 102)
c, da, db = fwd_bwd(a, b)
rows = [0, 7, 255, 511]
for name, arr in (("c", c), ("da", da), ("db", db)):
    out[f"cfg1_{name}_rows"] = arr[rows]
    out[f"cfg1_{name}_norm"] = np.array([np.linalg.norm(arr.astype(np.float64))])
    out[f"cfg1_{name}_sum"] = np.array([arr.astype(np.float64).sum()])
meta["cases"]["cfg1"] = {"rows": rows, "seed_a": 101, "seed_b": 102}

# 3. N-D broadcast, both sides broadcast somewhere: A[3,1,5,7] @ B[2,7,4]
a, b = uniform((3, 1, 5, 7), 11), uniform((2, 7, 4), 12)
dc = normal((3, 2, 5, 4), 13)
out["nd_c"], out["nd_da"], out["nd_db"] = fwd_bwd(a, b, dc)

# 4. [B,T,in] @ [in,out]: leading dims of dW summed away
a, b = uniform((2, 3, 8), 21), uniform((8, 5), 22)
dc = normal((2, 3, 5), 23)
out["bt_c"], out["bt_da"], out["bt_db"] = fwd_bwd(a, b, dc)

# 5. config 3 analogue: A = base[4,2,6,16].transpose(-1,-2) (reference needs .contiguous()), B [1,2,6,16]
base, b = uniform((4, 2, 6, 16), 301), uniform((1, 2, 6, 16), 302)
base_t = T(base, True)
a_view = base_t.transpose(2, 3).contiguous()
bt = T(b, True)
c = ref.cpu_matmul(a_view, bt)
c.backward(T(np.ones(c.shape, dtype=np.float32)))
out["cfg3s_c"], out["cfg3s_dbase"], out["cfg3s_db"] = c.to_numpy(), base_t.grad.to_numpy(), bt.grad.to_numpy()

# 6. ragged 2-D sizes (no multiple of any tile), dC random
a, b = uniform((77, 45), 31), uniform((45, 19), 32)
dc = normal((77, 19), 33)
out["rag_c"], out["rag_da"], out["rag_db"] = fwd_bwd(a, b, dc)

# 7. shared operand: s @ s accumulates both contributions into s.grad
s_np = uniform((6, 6), 41)
s = T(s_np, True)
c = ref.cpu_matmul(s, s)
c.backward(T(np.ones((6, 6), dtype=np.float32)))
out["ss_c"], out["ss_ds"] = c.to_numpy(), s.grad.to_numpy()

# 8. MLP training step (config 2 analogue, small): Linear 32->48, tanh, Linear 48->16, MSE, SGD lr 0.01
x, tgt = normal((64, 32), 201), normal((64, 16), 202)
rng = np.random.RandomState(203)
w1 = rng.uniform(-1 / np.sqrt(32), 1 / np.sqrt(32), (32, 48)).astype(np.float32)
w2 = rng.uniform(-1 / np.sqrt(48), 1 / np.sqrt(48), (48, 16)).astype(np.float32)
W1, B1 = T(w1, True), T(np.zeros((1, 48), np.float32), True)
W2, B2 = T(w2, True), T(np.zeros((1, 16), np.float32), True)
X, TG = T(x), T(tgt)
h = (ref.cpu_matmul(X, W1) + B1).tanh()
y = ref.cpu_matmul(h, W2) + B2
diff = y - TG
loss = (diff * diff).sum() / y.size
loss.backward()
out["mlp_loss"] = loss.to_numpy()
out["mlp_y"] = y.to_numpy()
for n, p in (("w1", W1), ("b1", B1), ("w2", W2), ("b2", B2)):
    out[f"mlp_d{n}"] = p.grad.to_numpy()
for p in (W1, B1, W2, B2):
    vel = ref.from_numpy(np.zeros(p.shape, np.float32), "cpu", False)
    ref._sgd_step_fused(p, p.grad, vel, 0.01, 0.0, 0.0, 0.0, 0, 0, 0)
for n, p in (("w1", W1), ("b1", B1), ("w2", W2), ("b2", B2)):
    out[f"mlp_new_{n}"] = p.to_numpy()

# 8b. forward-only typed matmul of the reference: float64, int32 (64-bit accumulation, wraps), int64 with broadcast
g = np.random.Generator(np.random.PCG64(77))
a64, b64 = g.standard_normal((3, 1, 9, 14)), g.standard_normal((2, 14, 11))
out["f64_c"] = ref.cpu_matmul(ref.from_numpy(a64, "cpu", False), ref.from_numpy(b64, "cpu", False)).to_numpy()
ai32 = g.integers(-2 ** 20, 2 ** 20, (17, 23)).astype(np.int32)
bi32 = g.integers(-2 ** 20, 2 ** 20, (23, 13)).astype(np.int32)
out["i32_c"] = ref.cpu_matmul(ref.from_numpy(ai32, "cpu", False), ref.from_numpy(bi32, "cpu", False)).to_numpy()
ai64 = g.integers(-2 ** 40, 2 ** 40, (2, 5, 7)).astype(np.int64)
bi64 = g.integers(-2 ** 20, 2 ** 20, (7, 4)).astype(np.int64)
out["i64_c"] = ref.cpu_matmul(ref.from_numpy(ai64, "cpu", False), ref.from_numpy(bi64, "cpu", False)).to_numpy()

# 8c. backward through tanh then matmul (the two autograd nodes the fused epilogue replaces), and the
#     Newton-Schulz chain of Muon composed from the reference's own tensor ops (aakaar/optim.py:533-542)
z, b, dc = normal((13, 9), 41), uniform((9, 7), 42), normal((13, 7), 43)
Z, B = T(z, True), T(b, True)
Cm = ref.cpu_matmul(Z.tanh(), B)
Cm.backward(T(dc))
out["tanhmm_dz"], out["tanhmm_db"] = Z.grad.to_numpy(), B.grad.to_numpy()
g0 = normal((24, 40), 44)
G0 = T(g0)
X = G0 / ((G0 * G0).sum().sqrt() + 1e-7)
for _ in range(5):
    A_ = X.transpose(0, 1).contiguous() @ X
    B_ = -4.7750 * A_ + 2.0315 * (A_ @ A_)
    X = 3.4445 * X + X @ B_
out["muon_ns5"] = X.to_numpy()

# 8d. two Muon steps on one [24, 40] weight, composed from the reference's tensor ops exactly as
#     aakaar/optim.py:544-564 composes them (lr 0.02, momentum 0.95, 5 Newton-Schulz steps, weight decay 0.01)
P = T(uniform((24, 40), 45))
buf = None
for step_seed in (46, 47):
    grad = T(normal((24, 40), step_seed)) + P * 0.01
    buf = grad if buf is None else buf * 0.95 + grad * (1 - 0.95)
    X = buf / ((buf * buf).sum().sqrt() + 1e-7)
    for _ in range(5):
        A_ = X.transpose(0, 1).contiguous() @ X
        B_ = -4.7750 * A_ + 2.0315 * (A_ @ A_)
        X = 3.4445 * X + X @ B_
    P = P - X * 0.02
out["muon_p2"] = P.to_numpy()

# 8e. the convolution fallback that calls the matmul path (aakaar/__init__.py:289-307, 330-352), composed from
#     the reference's own im2col + reshape + matmul ops, forward and backward
xc, wc = normal((3, 4, 19), 51), uniform((5, 4, 3), 52)
X1, W1 = T(xc, True), T(wc, True)
L_out = (19 + 2 * 2 - 2 * (3 - 1) - 1) // 2 + 1
Y1 = ref.cpu_matmul(W1.reshape([1, 5, 12]), ref.im2col_1d(X1, 3, 2, 2, 2, L_out))
dy1 = normal(tuple(Y1.shape), 53)
Y1.backward(T(dy1))
out["conv1d_y"], out["conv1d_dx"], out["conv1d_dw"] = Y1.to_numpy(), X1.grad.to_numpy(), W1.grad.to_numpy()
xc2, wc2 = normal((2, 3, 9, 11), 54), uniform((4, 3, 3, 2), 55)
X2, W2 = T(xc2, True), T(wc2, True)
OH2, OW2 = (9 + 2 * 1 - 1 * (3 - 1) - 1) // 2 + 1, (11 + 2 * 0 - 2 * (2 - 1) - 1) // 1 + 1
Y2 = ref.cpu_matmul(W2.reshape([1, 4, 18]), ref.im2col_2d(X2, 3, 2, 2, 1, 1, 0, 1, 2, OH2, OW2)).reshape([2, 4, OH2, OW2])
dy2 = normal(tuple(Y2.shape), 56)
Y2.backward(T(dy2))
out["conv2d_y"], out["conv2d_dx"], out["conv2d_dw"] = Y2.to_numpy(), X2.grad.to_numpy(), W2.grad.to_numpy()

# 8g. conv3d and the transposed convolutions (aakaar/__init__.py:365-388, 398-519), composed from the reference's own
#     im2col_3d / col2im_* + reshape / transpose + matmul ops exactly as its Python fallback composes them
xc3, wc3 = normal((2, 3, 5, 6, 7), 61), uniform((4, 3, 2, 3, 2), 62)
X3, W3 = T(xc3, True), T(wc3, True)
OD3, OH3, OW3 = (5 + 2 * 1 - 1 * (2 - 1) - 1) // 2 + 1, (6 + 2 * 0 - 1 * (3 - 1) - 1) // 1 + 1, (7 + 2 * 1 - 2 * (2 - 1) - 1) // 1 + 1
col3 = ref.im2col_3d(X3, 2, 3, 2, 2, 1, 1, 1, 0, 1, 1, 1, 2, OD3, OH3, OW3)
Y3 = ref.cpu_matmul(W3.reshape([4, 36]).reshape([1, 4, 36]), col3).reshape([2, 4, OD3, OH3, OW3])
dy3 = normal(tuple(Y3.shape), 63)
Y3.backward(T(dy3))
out["conv3d_y"], out["conv3d_dx"], out["conv3d_dw"] = Y3.to_numpy(), X3.grad.to_numpy(), W3.grad.to_numpy()

def ref_conv_transpose(x_np, w_np, dims, stride, padding, dilation, seed):
    """conv_transpose{1,2,3}d of the reference's fallback path; kernels are cubic (its col2im infers the size)."""
    X, W = T(x_np, True), T(w_np, True)
    cin, cout = w_np.shape[0], w_np.shape[1]
    k = w_np.shape[2:]
    spatial = x_np.shape[2:]
    outsz = [(spatial[i] - 1) * stride[i] - 2 * padding[i] + dilation[i] * (k[i] - 1) + 1 for i in range(dims)]
    kk = int(np.prod(k))
    w_t = W.reshape([cin, cout * kk]).transpose(0, 1).reshape([1, cout * kk, cin])
    col = ref.cpu_matmul(w_t, X.reshape([x_np.shape[0], cin, int(np.prod(spatial))]))
    if dims == 1:
        Y = ref.col2im_1d(col, cout, outsz[0], stride[0], padding[0], dilation[0], spatial[0])
    elif dims == 2:
        Y = ref.col2im_2d(col, cout, outsz[0], outsz[1], stride[0], stride[1], padding[0], padding[1], dilation[0], dilation[1],
                          spatial[0], spatial[1])
    else:
        Y = ref.col2im_3d(col, cout, outsz[0], outsz[1], outsz[2], *stride, *padding, *dilation, *spatial)
    dy = normal(tuple(Y.shape), seed)
    Y.backward(T(dy))
    return Y.to_numpy(), X.grad.to_numpy(), W.grad.to_numpy()

for name, xs_, ws_, dims, st_, pd_, dl_, seed in (
        ("convT1d", (3, 4, 9), (4, 5, 3), 1, (2,), (1,), (2,), 64),
        ("convT2d", (2, 3, 5, 6), (3, 4, 3, 3), 2, (2, 1), (1, 0), (1, 2), 67),
        ("convT3d", (2, 3, 3, 4, 5), (3, 2, 2, 2, 2), 3, (1, 2, 1), (0, 1, 0), (1, 1, 2), 70)):
    y_, dx_, dw_ = ref_conv_transpose(normal(xs_, seed + 1), uniform(ws_, seed + 2), dims, st_, pd_, dl_, seed)
    out[name + "_y"], out[name + "_dx"], out[name + "_dw"] = y_, dx_, dw_

# 8f. the README's training example (README.md:101-137): Linear(1,16) -> tanh -> Linear(16,1) on sin(x), its own
#     mse (diff * diff).sum() / n, plain SGD lr 0.05, 300 epochs; weights drawn as aakaar/nn.py:5-13 draws them
np.random.seed(0)
xs = np.linspace(-3, 3, 64).reshape(64, 1).astype(np.float32)
Xs, Ys = T(xs), T(np.sin(xs).astype(np.float32))
params = []
for fin, fout in ((1, 16), (16, 1)):
    lim = 1.0 / np.sqrt(fin)
    params.append(T(np.random.uniform(-lim, lim, (fin, fout)).astype(np.float32), True))
    params.append(T(np.zeros((1, fout), dtype=np.float32), True))
losses = []
for epoch in range(300):
    for p_ in params:
        p_.zero_grad()
    h_ = (ref.cpu_matmul(Xs, params[0]) + params[1]).tanh()
    diff = (ref.cpu_matmul(h_, params[2]) + params[3]) - Ys
    loss_ = (diff * diff).sum() / 64
    loss_.backward()
    losses.append(float(loss_.item()))
    ref._set_grad_enabled(False)
    for p_ in params:
        p_.copy_(p_ - p_.grad * 0.05)
    ref._set_grad_enabled(True)
out["readme_losses"] = np.array([losses[0], losses[1], losses[2], losses[99], losses[299]], dtype=np.float64)

# 9. error behaviour of the reference (messages the C ABI reproduces)
errs = {}
def err_of(fn):
    try:
        fn()
    except Exception as e:  # noqa: BLE001
        return [type(e).__name__, str(e)]
    return None
errs["k_mismatch"] = err_of(lambda: ref.cpu_matmul(T(np.ones((2, 3))), T(np.ones((4, 2)))))
errs["batch_mismatch"] = err_of(lambda: ref.cpu_matmul(T(np.ones((2, 2, 3))), T(np.ones((3, 3, 2)))))
errs["non_contiguous"] = err_of(lambda: ref.cpu_matmul(T(np.ones((2, 3))).transpose(0, 1), T(np.ones((2, 2)))))
errs["f64_autograd"] = err_of(lambda: ref.cpu_matmul(ref.from_numpy(np.ones((2, 2)), "cpu", True), ref.from_numpy(np.ones((2, 2)), "cpu", False)))
errs["non_scalar_backward"] = err_of(lambda: ref.cpu_matmul(T(np.ones((2, 3)), True), T(np.ones((3, 2)))).backward())
meta["errors"] = errs

np.savez_compressed(os.path.join(HERE, "ref_vectors.npz"), **out)
with open(os.path.join(HERE, "ref_vectors.json"), "w") as f:
    json.dump(meta, f, indent=1)
print("wrote", len(out), "arrays;", os.path.getsize(os.path.join(HERE, "ref_vectors.npz")), "bytes")
print(json.dumps(errs, indent=1))
