"""``nn.Linear`` of the reference (aakaar/nn.py:5-18) on the fused GEMM + bias epilogue."""
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
