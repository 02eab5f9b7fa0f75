"""CPU restatement of the reference's fp32 matmul path (forward + autograd backward).

TEST INFRASTRUCTURE ONLY. Nothing in the product package imports this module; it is the checker
used by tests/, by ``__graft_entry__.smoke()`` and by the ``cpu_baseline`` / ``--impl reference``
legs of bench.py. The product path is CUDA-only and fails loudly without its extension.

Every function follows one piece of the reference (paths relative to the reference checkout):

* ``plan_nd_matmul`` / ``batch_offset``  - src/matmul_kernel.cu:55-109 (CUDA planner, the one with the
  explicit rank check) and the equivalent lambdas in src/cpu_kernel.cpp:102-138.
* ``matmul_forward``                     - src/cpu_kernel.cpp:98-153 (one row-major sgemm per
  broadcast batch index, contiguous operands only).
* ``matmul_a_bt`` / ``matmul_at_b``      - src/cpu_kernel.cpp:1674-1691 (2-D backward products).
* ``matmul_backward``                    - the backward lambda of dispatch_matmul,
  src/bindings.cpp:1726-1759 (2-D fast path, otherwise transposed copies + forward + reduction).
* ``reduce_grad_to_shape``               - src/bindings.cpp:1467-1503.
* ``linear_forward``                     - aakaar/nn.py:5-18 (y = x @ W + b, W stored (in, out)).
* ``matmul_backward_tanh``               - matmul node backward followed by the tanh node backward,
  src/bindings.cpp:1726-1759 then :777-806 (``g * (1 - t^2)``, src/cpu_kernel.cpp:500-514).
* ``matmul_axpby`` / ``newton_schulz``   - the Newton-Schulz chain of the Muon optimizer,
  aakaar/optim.py:533-542 (matmul + scalar multiply + add, composed as the reference composes them).
* ``im2col_2d`` / ``col2im_2d`` / ``conv2d_forward_backward`` - the convolution fallback that calls
  the matmul path: src/conv2d_kernel.cpp:7-70 (and src/conv_kernel.cpp:15-60 for 1-D = one row),
  aakaar/__init__.py:289-307, 330-352.
* ``tanh`` / ``mse_loss`` / ``sgd_step`` - src/cpu_kernel.cpp:484-514, aakaar/__init__.py:222-224,
  src/optim_kernels_cpu.cpp:7-28 (support ops of the Linear training step).

The arithmetic of the reference lives in OpenBLAS ``cblas_sgemm`` (third party, version not pinned
by the reference; the build in oracle/_ref links OpenBLAS 0.3.15). Here the same products are
numpy float32 ``@`` (also an sgemm) or float64 for a stricter check; both differ from the
reference only in summation order, so parity is stated as relative Frobenius error, not bitwise.

Pinning: tests/test_oracle.py checks this module against (a) the documentation examples the
reference ships (docs/concepts/math-operations/matmul.md:36-57, docs/getting-started/
quick-start.md:57-73) and (b) vectors produced by the reference's own CPU build
(oracle/build_ref.sh -> oracle/_ref), committed under tests/golden/.
"""
from __future__ import annotations

import numpy as np

__all__ = [
    "plan_nd_matmul",
    "batch_offset",
    "matmul_forward",
    "matmul_forward_typed",
    "matmul_a_bt",
    "matmul_at_b",
    "matmul_backward",
    "matmul_backward_tanh",
    "matmul_axpby",
    "newton_schulz",
    "muon_step",
    "im2col_2d",
    "col2im_2d",
    "conv2d_forward_backward",
    "reduce_grad_to_shape",
    "linear_forward",
    "tanh",
    "tanh_backward",
    "mse_loss",
    "sgd_step",
    "mlp_step",
    "rel_frobenius",
]


def rel_frobenius(x, ref) -> float:
    """||x - ref||_F / ||ref||_F in float64."""
    x = np.asarray(x, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    den = np.linalg.norm(ref.ravel())
    num = np.linalg.norm((x - ref).ravel())
    return float(num / den) if den > 0 else float(num)


def plan_nd_matmul(shape_a, shape_b):
    """Right-aligned broadcast of the batch dims; returns (batch_shape, M, K, N).

    Raises ValueError with the reference's messages (src/matmul_kernel.cu:56-70).
    """
    shape_a = tuple(int(d) for d in shape_a)
    shape_b = tuple(int(d) for d in shape_b)
    if len(shape_a) < 2 or len(shape_b) < 2:
        raise ValueError("matmul requires tensors with at least 2 dimensions")
    M, K = shape_a[-2], shape_a[-1]
    K2, N = shape_b[-2], shape_b[-1]
    if K != K2:
        raise ValueError("Shape mismatch: inner dimensions must match for matmul")
    ba, bb = shape_a[:-2], shape_b[:-2]
    ndb = max(len(ba), len(bb))
    out = [0] * ndb
    for i in range(ndb):
        da = ba[len(ba) - 1 - i] if i < len(ba) else 1
        db = bb[len(bb) - 1 - i] if i < len(bb) else 1
        if da != db and da != 1 and db != 1:
            raise ValueError("Batch dimensions are not broadcastable for matmul")
        out[ndb - 1 - i] = max(da, db)
    return tuple(out), M, K, N


def batch_offset(flat_idx, out_batch, in_shape, mat_size):
    """Element offset of batch `flat_idx` inside a contiguous operand; size-1 dims map to 0."""
    in_batch = tuple(in_shape[:-2])
    ndb, nd_in = len(out_batch), len(in_batch)
    idx = [0] * ndb
    rem = flat_idx
    for i in range(ndb - 1, -1, -1):
        idx[i] = rem % out_batch[i]
        rem //= out_batch[i]
    off, stride = 0, mat_size
    for i in range(ndb - 1, -1, -1):
        in_i = i - (ndb - nd_in)
        in_dim = in_batch[in_i] if in_i >= 0 else 1
        use = 0 if in_dim == 1 else idx[i]
        if in_i >= 0:
            off += use * stride
            stride *= in_dim
    return off


def _require_contiguous(x, what):
    if not x.flags["C_CONTIGUOUS"]:
        raise ValueError(what)


def matmul_forward(a, b, acc=np.float32):
    """C[bi] = A[offA(bi)] @ B[offB(bi)] for every broadcast batch index bi."""
    a = np.asarray(a)
    b = np.asarray(b)
    _require_contiguous(a, "matmul requires contiguous tensors. Call .contiguous() first.")
    _require_contiguous(b, "matmul requires contiguous tensors. Call .contiguous() first.")
    batch, M, K, N = plan_nd_matmul(a.shape, b.shape)
    total = int(np.prod(batch)) if batch else 1
    out = np.empty(tuple(batch) + (M, N), dtype=np.float32)
    af, bf, of = a.reshape(-1), b.reshape(-1), out.reshape(-1)
    for bi in range(total):
        oa = batch_offset(bi, batch, a.shape, M * K)
        ob = batch_offset(bi, batch, b.shape, K * N)
        am = af[oa:oa + M * K].reshape(M, K).astype(acc, copy=False)
        bm = bf[ob:ob + K * N].reshape(K, N).astype(acc, copy=False)
        of[bi * M * N:(bi + 1) * M * N] = (am @ bm).astype(np.float32).reshape(-1)
    return out


def matmul_forward_typed(a, b):
    """Forward-only product for float64 / int32 / int64 operands (no autograd in the reference):
    src/cpu_kernel.cpp:1052-1185. Integers accumulate in 64 bits and wrap to the operand dtype."""
    a, b = np.asarray(a), np.asarray(b)
    if a.dtype != b.dtype:
        raise RuntimeError("matmul: operands must share one dtype")
    plan_nd_matmul(a.shape, b.shape)
    if a.dtype == np.float64:
        return np.matmul(a, b)
    if a.dtype in (np.int32, np.int64):
        with np.errstate(over="ignore"):
            return np.matmul(a.astype(np.int64), b.astype(np.int64)).astype(a.dtype)
    raise RuntimeError("matmul_forward_typed: unsupported dtype")


def matmul_a_bt(a, b, acc=np.float32):
    """C(m,n) = A(m,k) @ B(n,k)^T, B in its original (n,k) layout."""
    _require_contiguous(a, "matmul_a_bt requires contiguous tensors.")
    _require_contiguous(b, "matmul_a_bt requires contiguous tensors.")
    return (a.astype(acc, copy=False) @ b.astype(acc, copy=False).T).astype(np.float32)


def matmul_at_b(a, b, acc=np.float32):
    """C(m,n) = A(k,m)^T @ B(k,n), A in its original (k,m) layout."""
    _require_contiguous(a, "matmul_at_b requires contiguous tensors.")
    _require_contiguous(b, "matmul_at_b requires contiguous tensors.")
    return (a.astype(acc, copy=False).T @ b.astype(acc, copy=False)).astype(np.float32)


def reduce_grad_to_shape(grad, target_shape, skip_trailing=0, acc=np.float32):
    """Sum a broadcast gradient back to `target_shape`.

    Leading extra dims are summed away (axis 0, repeatedly, keepdim=False); then every aligned dim
    where the target is 1 and the gradient is not is summed with keepdim=True. The last
    `skip_trailing` dims are never touched.
    """
    g = np.asarray(grad)
    target_shape = tuple(target_shape)
    if g.ndim < len(target_shape):
        raise RuntimeError("reduce_grad_to_shape: gradient has fewer dims than its target shape")
    for _ in range(g.ndim - len(target_shape)):
        g = g.astype(acc, copy=False).sum(axis=0).astype(np.float32)
    for i in range(len(target_shape) - skip_trailing):
        if i >= g.ndim:
            break
        if target_shape[i] == 1 and g.shape[i] != 1:
            g = g.astype(acc, copy=False).sum(axis=i, keepdims=True).astype(np.float32)
    if skip_trailing == 0 and g.shape != target_shape:
        raise RuntimeError("reduce_grad_to_shape: reduced gradient shape does not match target shape")
    return g


def matmul_backward(a, b, grad_out, acc=np.float32):
    """(dA, dB) for C = A @ B given dC. Both are always computed, as the reference does."""
    a, b, grad_out = np.asarray(a), np.asarray(b), np.asarray(grad_out)
    if a.ndim == 2 and b.ndim == 2 and grad_out.ndim == 2:
        return matmul_a_bt(grad_out, b, acc), matmul_at_b(a, grad_out, acc)
    bT = np.ascontiguousarray(np.swapaxes(b, -1, -2))
    aT = np.ascontiguousarray(np.swapaxes(a, -1, -2))
    da_full = matmul_forward(grad_out, bT, acc)
    db_full = matmul_forward(aT, grad_out, acc)
    return (reduce_grad_to_shape(da_full, a.shape, 2, acc),
            reduce_grad_to_shape(db_full, b.shape, 2, acc))


def matmul_backward_tanh(a_tanh, b, grad_out, acc=np.float32):
    """(dZ, dB) for C = tanh(Z) @ B, given A = tanh(Z): the matmul backward, then dZ = dA * (1 - A^2)."""
    da, db = matmul_backward(a_tanh, b, grad_out, acc)
    a = np.asarray(a_tanh).astype(acc, copy=False)
    return (da.astype(acc, copy=False) * (1.0 - a * a)).astype(np.float32), db


def matmul_axpby(a, b, alpha, beta, d, acc=np.float32):
    """alpha * (a @ b) + beta * d, the shape of one Newton-Schulz line (``b * A + c * (A @ A)``)."""
    prod = matmul_forward(np.ascontiguousarray(a), np.ascontiguousarray(b), acc).astype(acc, copy=False)
    out = acc(alpha) * prod
    if d is not None and beta != 0:
        out = out + acc(beta) * np.asarray(d).astype(acc, copy=False)
    return out.astype(np.float32)


def newton_schulz(G, steps, acc=np.float32):
    """Muon._newton_schulz_orthogonalize: X = G / (|G|_F + 1e-7); then `steps` times
    A = X^T X, B = b A + c A A, X = a X + X B."""
    G = np.asarray(G).astype(acc, copy=False)
    X = G / (np.sqrt((G * G).sum(dtype=acc)) + acc(1e-7))
    a, b, c = 3.4445, -4.7750, 2.0315
    for _ in range(steps):
        A = X.T @ X
        B = acc(b) * A + acc(c) * (A @ A)
        X = acc(a) * X + X @ B
    return X.astype(np.float32)


def muon_step(param, grad, buf, lr=0.02, momentum=0.95, ns_steps=5, weight_decay=0.0, acc=np.float32):
    """One Muon.step for one parameter (aakaar/optim.py:544-564). Returns (new_param, new_buf)."""
    p, g = np.asarray(param).astype(acc, copy=False), np.asarray(grad).astype(acc, copy=False)
    if weight_decay != 0:
        g = g + p * acc(weight_decay)
    buf = g if buf is None else np.asarray(buf).astype(acc, copy=False) * acc(momentum) + g * acc(1 - momentum)
    update = newton_schulz(buf, ns_steps, acc).astype(acc) if p.ndim == 2 else buf
    return (p - update * acc(lr)).astype(np.float32), buf.astype(np.float32)


def im2col_2d(x, KH, KW, SH, SW, PH, PW, DH, DW, OH, OW):
    """(B, C, H, W) -> (B, C*KH*KW, OH*OW); row (c, kh, kw), zero outside the input."""
    x = np.asarray(x)
    B, C, H, W = x.shape
    col = np.zeros((B, C, KH, KW, OH, OW), dtype=x.dtype)
    for kh in range(KH):
        for kw in range(KW):
            for oh in range(OH):
                h = oh * SH - PH + kh * DH
                if h < 0 or h >= H:
                    continue
                for ow in range(OW):
                    w = ow * SW - PW + kw * DW
                    if 0 <= w < W:
                        col[:, :, kh, kw, oh, ow] = x[:, :, h, w]
    return col.reshape(B, C * KH * KW, OH * OW)


def col2im_2d(gcol, C, H, W, KH, KW, SH, SW, PH, PW, DH, DW, OH, OW):
    """Adjoint of im2col_2d: every input element sums the window entries that read it."""
    gcol = np.asarray(gcol)
    B = gcol.shape[0]
    g = gcol.reshape(B, C, KH, KW, OH, OW)
    gx = np.zeros((B, C, H, W), dtype=np.float64)
    for kh in range(KH):
        for kw in range(KW):
            for oh in range(OH):
                h = oh * SH - PH + kh * DH
                if h < 0 or h >= H:
                    continue
                for ow in range(OW):
                    w = ow * SW - PW + kw * DW
                    if 0 <= w < W:
                        gx[:, :, h, w] += g[:, :, kh, kw, oh, ow]
    return gx.astype(np.float32)


def conv2d_forward_backward(x, weight, grad_out, stride=(1, 1), padding=(0, 0), dilation=(1, 1), acc=np.float32):
    """y = conv2d(x, weight) as unfold + matmul, and (dx, dweight) for a given dy."""
    (SH, SW), (PH, PW), (DH, DW) = stride, padding, dilation
    C_out, C_in, KH, KW = weight.shape
    B, _, H, W = x.shape
    OH = (H + 2 * PH - DH * (KH - 1) - 1) // SH + 1
    OW = (W + 2 * PW - DW * (KW - 1) - 1) // SW + 1
    col = im2col_2d(x, KH, KW, SH, SW, PH, PW, DH, DW, OH, OW)
    w_flat = np.ascontiguousarray(weight).reshape(1, C_out, C_in * KH * KW)
    y = matmul_forward(w_flat, col, acc).reshape(B, C_out, OH, OW)
    dw_flat, dcol = matmul_backward(w_flat, col, np.ascontiguousarray(grad_out).reshape(B, C_out, OH * OW), acc)
    dx = col2im_2d(dcol, C_in, H, W, KH, KW, SH, SW, PH, PW, DH, DW, OH, OW)
    return y, dx, dw_flat.reshape(weight.shape)


def im2col_3d(x, K, S, P, D, O):
    """(B, C, D, H, W) -> (B, C*KD*KH*KW, OD*OH*OW) (run_cpu_im2col_3d, src/conv3d_kernel.cpp): row
    (c, kd, kh, kw), column (od, oh, ow), zero outside the input. K, S, P, D, O: 3-tuples."""
    x = np.asarray(x)
    B, C = x.shape[:2]
    dims = x.shape[2:]
    col = np.zeros((B, C) + tuple(K) + tuple(O), dtype=x.dtype)
    for kd in range(K[0]):
        for kh in range(K[1]):
            for kw in range(K[2]):
                for od in range(O[0]):
                    d = od * S[0] - P[0] + kd * D[0]
                    if d < 0 or d >= dims[0]:
                        continue
                    for oh in range(O[1]):
                        h = oh * S[1] - P[1] + kh * D[1]
                        if h < 0 or h >= dims[1]:
                            continue
                        for ow in range(O[2]):
                            w = ow * S[2] - P[2] + kw * D[2]
                            if 0 <= w < dims[2]:
                                col[:, :, kd, kh, kw, od, oh, ow] = x[:, :, d, h, w]
    return col.reshape(B, C * int(np.prod(K)), int(np.prod(O)))


def col2im_3d(gcol, C, dims, K, S, P, D, O):
    """Adjoint of im2col_3d (run_cpu_col2im_3d): (B, C*KD*KH*KW, OD*OH*OW) summed into (B, C, *dims)."""
    gcol = np.asarray(gcol)
    B = gcol.shape[0]
    g = gcol.reshape((B, C) + tuple(K) + tuple(O))
    gx = np.zeros((B, C) + tuple(dims), dtype=np.float64)
    for kd in range(K[0]):
        for kh in range(K[1]):
            for kw in range(K[2]):
                for od in range(O[0]):
                    d = od * S[0] - P[0] + kd * D[0]
                    if d < 0 or d >= dims[0]:
                        continue
                    for oh in range(O[1]):
                        h = oh * S[1] - P[1] + kh * D[1]
                        if h < 0 or h >= dims[1]:
                            continue
                        for ow in range(O[2]):
                            w = ow * S[2] - P[2] + kw * D[2]
                            if 0 <= w < dims[2]:
                                gx[:, :, d, h, w] += g[:, :, kd, kh, kw, od, oh, ow]
    return gx.astype(np.float32)


def _pad3(v, fill):
    v = tuple(v)
    return (fill,) * (3 - len(v)) + v


def conv_nd_forward_backward(x, weight, grad_out, stride, padding, dilation, acc=np.float32):
    """conv1d / conv2d / conv3d of the reference's fallback (aakaar/__init__.py:289-388) as unfold + matmul,
    and (dx, dweight) for a given dy. Rank is taken from the weight; lower ranks run as depth-1 volumes."""
    nd = weight.ndim - 2
    K, S, P, D = _pad3(weight.shape[2:], 1), _pad3(stride, 1), _pad3(padding, 0), _pad3(dilation, 1)
    dims = _pad3(x.shape[2:], 1)
    O = tuple((dims[i] + 2 * P[i] - D[i] * (K[i] - 1) - 1) // S[i] + 1 for i in range(3))
    B, C_in, C_out = x.shape[0], x.shape[1], weight.shape[0]
    col = im2col_3d(np.asarray(x).reshape((B, C_in) + dims), K, S, P, D, O)
    w_flat = np.ascontiguousarray(weight).reshape(1, C_out, C_in * int(np.prod(K)))
    y = matmul_forward(w_flat, col, acc).reshape((B, C_out) + O[3 - nd:])
    dw_flat, dcol = matmul_backward(w_flat, col, np.ascontiguousarray(grad_out).reshape(B, C_out, int(np.prod(O))), acc)
    dx = col2im_3d(dcol, C_in, dims, K, S, P, D, O).reshape(x.shape)
    return y, dx, dw_flat.reshape(weight.shape)


def conv_transpose_nd_forward_backward(x, weight, grad_out, stride, padding, dilation, acc=np.float32):
    """conv_transpose{1,2,3}d of the reference's fallback (aakaar/__init__.py:398-519): weight
    (C_in, C_out, *K); col = W_flat^T @ x, then the fold; and (dx, dweight) for a given dy (the fold's
    backward is the unfold, src/bindings.cpp:1066-1078)."""
    nd = weight.ndim - 2
    K, S, P, D = _pad3(weight.shape[2:], 1), _pad3(stride, 1), _pad3(padding, 0), _pad3(dilation, 1)
    win = _pad3(x.shape[2:], 1)                       # the input positions are the WINDOW positions of the fold
    out_dims = tuple((win[i] - 1) * S[i] - 2 * P[i] + D[i] * (K[i] - 1) + 1 for i in range(3))
    B, C_in, C_out = x.shape[0], weight.shape[0], weight.shape[1]
    kk = int(np.prod(K))
    w_t = np.ascontiguousarray(np.ascontiguousarray(weight).reshape(C_in, C_out * kk).T)[None]   # (1, C_out*kk, C_in)
    x_flat = np.ascontiguousarray(x).reshape(B, C_in, int(np.prod(win)))
    col = matmul_forward(w_t, x_flat, acc)                                                        # (B, C_out*kk, L_in)
    y = col2im_3d(col, C_out, out_dims, K, S, P, D, win).reshape((B, C_out) + out_dims[3 - nd:])
    dcol = im2col_3d(np.asarray(grad_out).reshape((B, C_out) + out_dims), K, S, P, D, win)
    dw_t, dx_flat = matmul_backward(w_t, x_flat, dcol, acc)
    dw = np.ascontiguousarray(dw_t[0].T).reshape(weight.shape)
    return y, dx_flat.reshape(x.shape), dw


# ---------------------------------------------------------------- Linear training step support

def linear_forward(x, w, bias, acc=np.float32):
    """y = x @ W + b with W (in, out) and b (1, out)."""
    y = matmul_forward(np.ascontiguousarray(x), np.ascontiguousarray(w), acc)
    return (y + bias).astype(np.float32) if bias is not None else y


def tanh(x):
    return np.tanh(x.astype(np.float32))


def tanh_backward(grad, out):
    return (grad * (1.0 - out * out)).astype(np.float32)


def mse_loss(pred, target):
    """sum((p - t)^2) / n, composed as sub, mul, sum_all, div like aakaar.mse_loss."""
    d = (pred - target).astype(np.float32)
    return np.float32((d * d).astype(np.float32).sum(dtype=np.float32) / np.float32(d.size))


def sgd_step(param, grad, lr):
    """Plain SGD (no momentum / weight decay): p -= lr * g."""
    return (param - np.float32(lr) * grad).astype(np.float32)


def mlp_step(x, target, w1, b1, w2, b2, lr, acc=np.float32):
    """One Linear -> tanh -> Linear -> MSE -> backward -> SGD step.

    Returns (loss, (w1', b1', w2', b2'), grads dict). Gradient flow follows the reference's
    autograd: matmul node backward, bias gradient = sum over rows (keepdim), tanh' = 1 - t^2.
    """
    z1 = linear_forward(x, w1, b1, acc)
    h = tanh(z1)
    y = linear_forward(h, w2, b2, acc)
    loss = mse_loss(y, target)
    n = np.float32(y.size)
    dy = (np.float32(2.0) * (y - target) / n).astype(np.float32)
    dh, dw2 = matmul_backward(h, w2, dy, acc)
    db2 = reduce_grad_to_shape(dy, b2.shape, 0, acc)
    dz1 = tanh_backward(dh, h)
    _, dw1 = matmul_backward(x, w1, dz1, acc)
    db1 = reduce_grad_to_shape(dz1, b1.shape, 0, acc)
    new = (sgd_step(w1, dw1, lr), sgd_step(b1, db1, lr), sgd_step(w2, dw2, lr), sgd_step(b2, db2, lr))
    return loss, new, {"w1": dw1, "b1": db1, "w2": dw2, "b2": db2, "y": y}
