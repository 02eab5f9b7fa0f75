"""aakaar_b200 - the fp32 matmul path of the Aakaar tensor library, rebuilt for NVIDIA B200.

Same Python surface as the reference package for this path (``aakaar/__init__.py:160-168, 222-268``):
``matmul`` / ``Tensor.__matmul__``, ``from_numpy``, ``set_tf32`` / ``is_tf32_enabled``,
``synchronize``, ``no_grad``, ``mse_loss``, plus ``nn.Linear`` and ``optim.SGD``. The work is done
by hand-written sm_100a kernels (TMA + tcgen05, TF32 or 3xTF32 split products) behind the C ABI of
``include/akr_b200.h``. There is no CPU implementation: importing works anywhere the native module
was built, computing needs a B200.

Differences from the reference, all supersets:
* operands may be transposed / sliced views - no ``.contiguous()`` needed (the reference raises);
* the backward pass reduces broadcast-batch gradients inside the GEMM;
* ``set_tf32(False)`` (the default) is a 3xTF32 split with fp32-level accuracy on tensor cores.
"""
from __future__ import annotations

import contextlib

__version__ = "0.1.0"

try:
    from . import _C  # pybind11 module over the C ABI (aakaar_b200/csrc/host)
except ImportError as exc:  # pragma: no cover - exercised only on a broken install
    raise ImportError(
        "aakaar_b200: the native module is not built. Run `python -m aakaar_b200._build` "
        "(needs nvcc with sm_100a support); there is no pure-Python or CPU fallback."
    ) from exc

Tensor = _C.Tensor


def matmul(a, b):
    """``a @ b`` with N-D batch broadcasting; both tensors must live on the same device."""
    if a.device != b.device:
        raise RuntimeError("Both tensors must be on the same device!")
    return _C.cuda_matmul(a, b)


def add(a, b):
    if a.device != b.device:
        raise RuntimeError("Both tensors must be on the same device!")
    return a + b


def sub(a, b):
    if a.device != b.device:
        raise RuntimeError("Both tensors must be on the same device!")
    return a - b


@contextlib.contextmanager
def no_grad():
    prev = _C._is_grad_enabled()
    _C._set_grad_enabled(False)
    try:
        yield
    finally:
        _C._set_grad_enabled(prev)


def is_grad_enabled():
    return _C._is_grad_enabled()


def mse_loss(pred, target):
    """Mean squared error as one fused reduction (the reference composes sub, mul, sum, div)."""
    return _C._mse_fused(pred, target)


def im2col_1d(x, kernel_size, stride, padding, dilation, out_length):
    """(B, C, L) -> (B, C*kernel_size, L_out) sliding windows (aakaar/__init__.py:285-288)."""
    return _C.im2col_1d(x, kernel_size, stride, padding, dilation, out_length)


def im2col_2d(x, KH, KW, SH, SW, PH, PW, DH, DW, OH, OW):
    """(B, C, H, W) -> (B, C*KH*KW, OH*OW) sliding windows (aakaar/__init__.py:325-328)."""
    return _C.im2col_2d(x, KH, KW, SH, SW, PH, PW, DH, DW, OH, OW)


def conv1d(x, weight, stride=1, padding=0, dilation=1):
    """Conv1d forward + backward as unfold + matmul, the reference's path without cuDNN
    (aakaar/__init__.py:289-307): ``[1, C_out, C_in*K] @ [B, C_in*K, L_out]`` is ONE batched launch with the
    weights broadcast (stride 0), and the weight gradient is summed over the batch inside its GEMM."""
    C_out, C_in, K = weight.shape
    B, _, L_in = x.shape
    L_out = (L_in + 2 * padding - dilation * (K - 1) - 1) // stride + 1
    if L_out <= 0:
        raise ValueError(f"conv1d: computed output length {L_out} <= 0")
    col = im2col_1d(x, K, stride, padding, dilation, L_out)
    w_flat = weight.reshape([1, C_out, C_in * K])
    return matmul(w_flat, col)


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


def conv2d(x, weight, stride=(1, 1), padding=(0, 0), dilation=(1, 1)):
    """Conv2d forward + backward as unfold + matmul (aakaar/__init__.py:330-352)."""
    (SH, SW), (PH, PW), (DH, DW) = _pair(stride), _pair(padding), _pair(dilation)
    C_out, C_in, KH, KW = weight.shape
    B, _, H, W = x.shape
    OH = (H + 2 * PH - DH * (KH - 1) - 1) // SH + 1
    OW = (W + 2 * PW - DW * (KW - 1) - 1) // SW + 1
    if OH <= 0 or OW <= 0:
        raise ValueError(f"conv2d: computed output size ({OH},{OW}) <= 0")
    col = im2col_2d(x, KH, KW, SH, SW, PH, PW, DH, DW, OH, OW)
    w_flat = weight.reshape([1, C_out, C_in * KH * KW])
    return matmul(w_flat, col).reshape([B, C_out, OH, OW])


def _triple(v):
    return (v, v, v) if isinstance(v, int) else tuple(v)


def im2col_3d(x, kernel_size, stride, padding, dilation, out_size):
    """(B, C, D, H, W) -> (B, C*KD*KH*KW, OD*OH*OW) sliding windows (aakaar/__init__.py:354-363)."""
    (KD, KH, KW), (SD, SH, SW), (PD, PH, PW) = kernel_size, stride, padding
    (DD, DH, DW), (OD, OH, OW) = dilation, out_size
    return _C.im2col_3d(x, KD, KH, KW, SD, SH, SW, PD, PH, PW, DD, DH, DW, OD, OH, OW)


def conv3d(x, weight, stride=(1, 1, 1), padding=(0, 0, 0), dilation=(1, 1, 1)):
    """Conv3d forward + backward as unfold + matmul (aakaar/__init__.py:365-388):
    ``[1, C_out, C_in*KD*KH*KW] @ [B, C_in*KD*KH*KW, OD*OH*OW]`` in one broadcast-batched launch."""
    (SD, SH, SW), (PD, PH, PW), (DD, DH, DW) = _triple(stride), _triple(padding), _triple(dilation)
    C_out, C_in, KD, KH, KW = weight.shape
    B, _, D, H, W = x.shape
    OD = (D + 2 * PD - DD * (KD - 1) - 1) // SD + 1
    OH = (H + 2 * PH - DH * (KH - 1) - 1) // SH + 1
    OW = (W + 2 * PW - DW * (KW - 1) - 1) // SW + 1
    if OD <= 0 or OH <= 0 or OW <= 0:
        raise ValueError(f"conv3d: computed output size ({OD},{OH},{OW}) <= 0")
    col = im2col_3d(x, (KD, KH, KW), (SD, SH, SW), (PD, PH, PW), (DD, DH, DW), (OD, OH, OW))
    w_flat = weight.reshape([1, C_out, C_in * KD * KH * KW])
    return matmul(w_flat, col).reshape([B, C_out, OD, OH, OW])


def col2im_1d(col, C, L_in, stride, padding, dilation, out_length):
    """(B, C*K, L_out) columns summed back into (B, C, L_in): the adjoint of im2col_1d
    (aakaar/__init__.py:390-395)."""
    return _C.col2im_1d(col, C, L_in, stride, padding, dilation, out_length)


def col2im_2d(col, C, H_in, W_in, stride, padding, dilation, out_size, kernel_size=None):
    """Adjoint of im2col_2d (aakaar/__init__.py:441-446). The reference infers a square kernel from the row
    count; `kernel_size` lifts that restriction."""
    (SH, SW), (PH, PW), (DH, DW), (OH, OW) = stride, padding, dilation, out_size
    KH, KW = kernel_size if kernel_size is not None else (0, 0)
    return _C.col2im_2d(col, C, H_in, W_in, SH, SW, PH, PW, DH, DW, OH, OW, KH, KW)


def col2im_3d(col, C, D_in, H_in, W_in, stride, padding, dilation, out_size, kernel_size=None):
    """Adjoint of im2col_3d (aakaar/__init__.py:448-453)."""
    (SD, SH, SW), (PD, PH, PW), (DD, DH, DW), (OD, OH, OW) = stride, padding, dilation, out_size
    KD, KH, KW = kernel_size if kernel_size is not None else (0, 0, 0)
    return _C.col2im_3d(col, C, D_in, H_in, W_in, SD, SH, SW, PD, PH, PW, DD, DH, DW, OD, OH, OW, KD, KH, KW)


def _no_output_padding(name, output_padding):
    if output_padding != 0 and any(_triple(output_padding)):
        raise NotImplementedError(f"{name}: output_padding != 0 is not yet implemented.")


def conv_transpose1d(x, weight, stride=1, padding=0, output_padding=0, dilation=1):
    """Transposed convolution, weight ``(in_channels, out_channels, K)`` (aakaar/__init__.py:398-439): the
    flattened weights, read as a TRANSPOSED VIEW (no copy), times x in one broadcast-batched launch, then the
    fold. output_padding is not supported (as in the reference)."""
    _no_output_padding("conv_transpose1d", output_padding)
    Cin_t, Cout_t, K = weight.shape
    B, C_in_x, L_in = x.shape
    if C_in_x != Cin_t:
        raise ValueError(f"conv_transpose1d: expected {Cin_t} input channels, got {C_in_x}")
    L_out = (L_in - 1) * stride - 2 * padding + dilation * (K - 1) + 1
    w_t = weight.reshape([Cin_t, Cout_t * K]).transpose(0, 1)          # (Cout_t*K, Cin_t), strided view
    col = matmul(w_t, x)                                               # (B, Cout_t*K, L_in)
    return col2im_1d(col, Cout_t, L_out, stride, padding, dilation, L_in)


def conv_transpose2d(x, weight, stride=(1, 1), padding=(0, 0), output_padding=(0, 0), dilation=(1, 1)):
    """2-D transposed convolution, weight ``(in_channels, out_channels, KH, KW)`` (aakaar/__init__.py:456-486)."""
    _no_output_padding("conv_transpose2d", output_padding)
    (SH, SW), (PH, PW), (DH, DW) = _pair(stride), _pair(padding), _pair(dilation)
    Cin_t, Cout_t, KH, KW = weight.shape
    B, C_in_x, H_in, W_in = x.shape
    if C_in_x != Cin_t:
        raise ValueError(f"conv_transpose2d: expected {Cin_t} input channels, got {C_in_x}")
    OH = (H_in - 1) * SH - 2 * PH + DH * (KH - 1) + 1
    OW = (W_in - 1) * SW - 2 * PW + DW * (KW - 1) + 1
    w_t = weight.reshape([Cin_t, Cout_t * KH * KW]).transpose(0, 1)
    col = matmul(w_t, x.reshape([B, Cin_t, H_in * W_in]))              # (B, Cout_t*KH*KW, H_in*W_in)
    return col2im_2d(col, Cout_t, OH, OW, (SH, SW), (PH, PW), (DH, DW), (H_in, W_in), (KH, KW))


def conv_transpose3d(x, weight, stride=(1, 1, 1), padding=(0, 0, 0), output_padding=(0, 0, 0), dilation=(1, 1, 1)):
    """3-D transposed convolution, weight ``(in_channels, out_channels, KD, KH, KW)`` (aakaar/__init__.py:489-519)."""
    _no_output_padding("conv_transpose3d", output_padding)
    (SD, SH, SW), (PD, PH, PW), (DD, DH, DW) = _triple(stride), _triple(padding), _triple(dilation)
    Cin_t, Cout_t, KD, KH, KW = weight.shape
    B, C_in_x, D_in, H_in, W_in = x.shape
    if C_in_x != Cin_t:
        raise ValueError(f"conv_transpose3d: expected {Cin_t} input channels, got {C_in_x}")
    OD = (D_in - 1) * SD - 2 * PD + DD * (KD - 1) + 1
    OH = (H_in - 1) * SH - 2 * PH + DH * (KH - 1) + 1
    OW = (W_in - 1) * SW - 2 * PW + DW * (KW - 1) + 1
    w_t = weight.reshape([Cin_t, Cout_t * KD * KH * KW]).transpose(0, 1)
    col = matmul(w_t, x.reshape([B, Cin_t, D_in * H_in * W_in]))
    return col2im_3d(col, Cout_t, OD, OH, OW, (SD, SH, SW), (PD, PH, PW), (DD, DH, DW), (D_in, H_in, W_in),
                     (KD, KH, KW))


def from_numpy(array, device: str = "cuda", requires_grad: bool = False):
    return _C.from_numpy(array, device, requires_grad)


def zero_grad_all(parameters):
    for p in parameters:
        p.zero_grad()


def set_tf32(enabled: bool = True):
    """True: single-pass TF32 products. False (default): 3xTF32 split, fp32-accurate results."""
    _C._set_tf32_enabled(bool(enabled))


def is_tf32_enabled():
    return _C._get_tf32_enabled()


def synchronize():
    """Block until all queued GPU work is done; raises if a kernel aborted on a bounded wait."""
    _C._synchronize()


def is_available():
    return _C.is_available()


def device_count():
    return _C.device_count()


def empty_cache():
    _C.empty_cache()


from . import nn, optim, losses  # noqa: E402

__all__ = [
    "Tensor", "matmul", "add", "sub", "no_grad", "is_grad_enabled", "mse_loss", "from_numpy",
    "zero_grad_all", "set_tf32", "is_tf32_enabled", "synchronize", "is_available", "device_count",
    "empty_cache", "nn", "optim", "losses", "conv1d", "conv2d", "conv3d", "im2col_1d", "im2col_2d", "im2col_3d",
    "col2im_1d", "col2im_2d", "col2im_3d", "conv_transpose1d", "conv_transpose2d", "conv_transpose3d",
]
