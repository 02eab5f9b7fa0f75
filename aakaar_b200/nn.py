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


class _ConvNd:
    """Shared part of Conv1d / Conv2d: weights ``(out, in, *kernel)`` and bias ``(1, out, 1[, 1])`` drawn as the
    reference draws them (uniform +-1/sqrt(fan_in), weight first, then bias), so ``np.random.seed`` gives the
    reference's parameters."""

    def _init(self, in_channels, out_channels, kernel, bias, device, dtype):
        if dtype != "float32":
            raise RuntimeError("aakaar_b200 convolutions are float32 only")
        self.in_channels, self.out_channels = in_channels, out_channels
        limit = 1.0 / np.sqrt(in_channels * int(np.prod(kernel)))
        w = np.random.uniform(-limit, limit, (out_channels, in_channels) + tuple(kernel)).astype(np.float32)
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
