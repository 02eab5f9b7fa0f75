"""``optim.SGD`` of the reference (aakaar/optim.py:5-50) on the fused update kernel."""
from __future__ import annotations

from . import _C, no_grad


class SGD:
    def __init__(self, parameters, lr=0.01, momentum=0.0, weight_decay=0.0, dampening=0.0, nesterov=False):
        if nesterov and (momentum <= 0 or dampening != 0):
            raise ValueError("Nesterov momentum requires momentum > 0 and dampening == 0")
        self.parameters = list(parameters)
        self.lr = lr
        self.momentum = momentum
        self.weight_decay = weight_decay
        self.dampening = dampening
        self.nesterov = nesterov
        self._velocity = [None] * len(self.parameters)

    def step(self):
        with no_grad():
            for i, p in enumerate(self.parameters):
                if p.grad is None:
                    continue
                grad = p.grad if p.grad.is_contiguous() else p.grad.contiguous()
                if not p.is_contiguous():
                    raise ValueError("SGD.step: parameters must be contiguous")
                initialized = self._velocity[i] is not None
                if self.momentum != 0 and self._velocity[i] is None:
                    self._velocity[i] = grad * 0.0
                _C._sgd_step_fused(p, grad, self._velocity[i], self.lr, self.momentum, self.weight_decay,
                                   self.dampening, int(self.nesterov), int(self.momentum != 0), int(initialized))

    def zero_grad(self):
        for p in self.parameters:
            p.zero_grad()
