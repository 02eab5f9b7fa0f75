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
    "empty_cache", "nn", "optim", "losses",
]
