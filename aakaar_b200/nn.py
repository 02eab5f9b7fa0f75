"""``nn.Linear`` (aakaar/nn.py:5-18) on the fused GEMM + bias epilogue, and ``nn.Conv1d`` / ``nn.Conv2d``
(aakaar/nn.py:20-134) on the unfold + matmul path. float32 only."""
from __future__ import annotations

import numpy as np

from . import _C


class Linear:
    """y = x @ W + b with W stored ``(in_features, out_features)`` and b ``(1, out_features)``.

    Initialisation follows the reference: ``np.random.uniform(-1/sqrt(in), 1/sqrt(in))`` for the
    weight (so ``np.random.seed`` reproduces the reference's weights) and zeros for the bias.
    The bias add runs in the GEMM epilogue instead of a separate broadcast-add kernel.
    """

    def __init__(self, in_features, out_features, device="cuda", bias=True):
        limit = 1.0 / np.sqrt(in_features)
        w = np.random.uniform(-limit, limit, (in_features, out_features)).astype(np.float32)
        self.weight = _C.from_numpy(w, device, True)
        self.bias = _C.from_numpy(np.zeros((1, out_features), dtype=np.float32), device, True) if bias else None
        self.in_features = in_features
        self.out_features = out_features

    def __call__(self, x):
        return _C.linear(x, self.weight, self.bias)

    def parameters(self):
        return [self.weight] if self.bias is None else [self.weight, self.bias]


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


def _triple(v):
    return (v, v, v) if isinstance(v, int) else tuple(v)


class _ConvNd:
    """Shared part of the convolution modules: weights ``(out, in, *kernel)`` (``(in, out, *kernel)`` for the
    transposed ones) and bias ``(1, out, 1[, 1[, 1]])`` drawn as the reference draws them (uniform
    +-1/sqrt(fan_in) with fan_in = in_channels * kernel volume, weight first, then bias), so ``np.random.seed``
    gives the reference's parameters."""

    def _init(self, in_channels, out_channels, kernel, bias, device, dtype, transposed=False):
        if dtype != "float32":
            raise RuntimeError("aakaar_b200 convolutions are float32 only")
        self.in_channels, self.out_channels = in_channels, out_channels
        limit = 1.0 / np.sqrt(in_channels * int(np.prod(kernel)))
        lead = (in_channels, out_channels) if transposed else (out_channels, in_channels)
        w = np.random.uniform(-limit, limit, lead + tuple(kernel)).astype(np.float32)
        self.weight = _C.from_numpy(w, device, True)
        self.has_bias = bias
        self.bias = None
        if bias:
            b = np.random.uniform(-limit, limit, (1, out_channels) + (1,) * len(kernel)).astype(np.float32)
            self.bias = _C.from_numpy(b, device, True)

    def parameters(self):
        return [self.weight, self.bias] if self.has_bias else [self.weight]


class Conv1d(_ConvNd):
    """y = conv1d(x, weight) + bias; x ``(batch, in_channels, length)``."""

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, bias=True,
                 device="cuda", dtype="float32"):
        self.kernel_size, self.stride, self.padding, self.dilation = kernel_size, stride, padding, dilation
        self._init(in_channels, out_channels, (kernel_size,), bias, device, dtype)

    def __call__(self, x):
        from . import conv1d
        if len(x.shape) != 3:
            raise ValueError(f"Conv1d expects input of shape (batch, in_channels, length), got {x.shape}")
        if x.shape[1] != self.in_channels:
            raise ValueError(f"Conv1d: expected {self.in_channels} input channels, got {x.shape[1]}")
        out = conv1d(x, self.weight, self.stride, self.padding, self.dilation)
        return out + self.bias if self.has_bias else out


class Conv2d(_ConvNd):
    """y = conv2d(x, weight) + bias; x ``(batch, in_channels, H, W)``."""

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, bias=True,
                 device="cuda", dtype="float32"):
        self.kernel_size = _pair(kernel_size)
        self.stride, self.padding, self.dilation = _pair(stride), _pair(padding), _pair(dilation)
        self._init(in_channels, out_channels, self.kernel_size, bias, device, dtype)

    def __call__(self, x):
        from . import conv2d
        if len(x.shape) != 4:
            raise ValueError(f"Conv2d expects input of shape (batch, in_channels, H, W), got {x.shape}")
        if x.shape[1] != self.in_channels:
            raise ValueError(f"Conv2d: expected {self.in_channels} input channels, got {x.shape[1]}")
        out = conv2d(x, self.weight, self.stride, self.padding, self.dilation)
        return out + self.bias if self.has_bias else out


class Conv3d(_ConvNd):
    """y = conv3d(x, weight) + bias; x ``(batch, in_channels, D, H, W)`` (aakaar/nn.py:139-200)."""

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, bias=True,
                 device="cuda", dtype="float32"):
        self.kernel_size = _triple(kernel_size)
        self.stride, self.padding, self.dilation = _triple(stride), _triple(padding), _triple(dilation)
        self._init(in_channels, out_channels, self.kernel_size, bias, device, dtype)

    def __call__(self, x):
        from . import conv3d
        if len(x.shape) != 5:
            raise ValueError(f"Conv3d expects input of shape (batch, in_channels, D, H, W), got {x.shape}")
        if x.shape[1] != self.in_channels:
            raise ValueError(f"Conv3d: expected {self.in_channels} input channels, got {x.shape[1]}")
        out = conv3d(x, self.weight, self.stride, self.padding, self.dilation)
        return out + self.bias if self.has_bias else out


class _ConvTransposeNd(_ConvNd):
    _fn, _rank, _what = None, 0, ""

    def __call__(self, x):
        import aakaar_b200 as ak
        if len(x.shape) != self._rank + 2:
            raise ValueError(f"{type(self).__name__} expects input of shape {self._what}, got {x.shape}")
        if x.shape[1] != self.in_channels:
            raise ValueError(f"{type(self).__name__}: expected {self.in_channels} input channels, got {x.shape[1]}")
        out = getattr(ak, self._fn)(x, self.weight, self.stride, self.padding, self.output_padding, self.dilation)
        return out + self.bias if self.has_bias else out


class ConvTranspose1d(_ConvTransposeNd):
    """Transposed Conv1d, weight ``(in_channels, out_channels, K)`` (aakaar/nn.py:202-268)."""
    _fn, _rank, _what = "conv_transpose1d", 1, "(batch, in_channels, length)"

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, output_padding=0, dilation=1,
                 bias=True, device="cuda", dtype="float32"):
        self.kernel_size, self.stride, self.padding = kernel_size, stride, padding
        self.output_padding, self.dilation = output_padding, dilation
        self._init(in_channels, out_channels, (kernel_size,), bias, device, dtype, transposed=True)


class ConvTranspose2d(_ConvTransposeNd):
    """Transposed Conv2d, weight ``(in_channels, out_channels, KH, KW)`` (aakaar/nn.py:270-326)."""
    _fn, _rank, _what = "conv_transpose2d", 2, "(batch, in_channels, H, W)"

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, output_padding=0, dilation=1,
                 bias=True, device="cuda", dtype="float32"):
        self.kernel_size = _pair(kernel_size)
        self.stride, self.padding, self.dilation = _pair(stride), _pair(padding), _pair(dilation)
        self.output_padding = _pair(output_padding)
        self._init(in_channels, out_channels, self.kernel_size, bias, device, dtype, transposed=True)


class ConvTranspose3d(_ConvTransposeNd):
    """Transposed Conv3d, weight ``(in_channels, out_channels, KD, KH, KW)`` (aakaar/nn.py:328-382)."""
    _fn, _rank, _what = "conv_transpose3d", 3, "(batch, in_channels, D, H, W)"

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, output_padding=0, dilation=1,
                 bias=True, device="cuda", dtype="float32"):
        self.kernel_size = _triple(kernel_size)
        self.stride, self.padding, self.dilation = _triple(stride), _triple(padding), _triple(dilation)
        self.output_padding = _triple(output_padding)
        self._init(in_channels, out_channels, self.kernel_size, bias, device, dtype, transposed=True)
