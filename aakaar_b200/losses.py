"""``losses.MSELoss`` of the reference (aakaar/losses.py:40-48)."""
from __future__ import annotations

from . import _C


class MSELoss:
    def __call__(self, pred, target):
        return _C._mse_fused(pred, target)
