"""``optim.SGD`` (aakaar/optim.py:5-50) and ``optim.Muon`` (aakaar/optim.py:516-568) of the reference.

SGD runs on the fused update kernel. Muon's Newton-Schulz chain is three launches per iteration: the
transposed operand of ``X^T X`` is read in place and the scalar multiplies and adds of
``b * A + c * (A @ A)`` and ``a * X + X @ B`` are folded into the epilogue of their products."""
from __future__ import annotations

from . import _C, no_grad


def _fused_update(p, grad, velocity, lr, momentum, weight_decay, dampening, nesterov, has_momentum, initialized):
    """The fused update on `p`. A parameter that is a view (transposed, sliced) takes it on a dense copy that
    is written back through the view's strides - the reference's unfused fallback for such parameters
    (aakaar/optim.py:24-48: ``p.copy_(p - update * lr)``), same arithmetic."""
    if p.is_contiguous():
        _C._sgd_step_fused(p, grad, velocity, lr, momentum, weight_decay, dampening, nesterov, has_momentum, initialized)
        return
    dense = p.contiguous()
    _C._sgd_step_fused(dense, grad, velocity, lr, momentum, weight_decay, dampening, nesterov, has_momentum, initialized)
    p.copy_(dense)


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
        """One update of every parameter that has a gradient: the contiguous ones in ONE launch
        (the reference launches its kernel once per parameter), views through the dense-copy fallback."""
        with no_grad():
            ps, gs, vs, inits = [], [], [], []
            for i, p in enumerate(self.parameters):
                if p.grad is None:
                    continue
                grad = p.grad if p.grad.is_contiguous() else p.grad.contiguous()
                initialized = self._velocity[i] is not None
                if self.momentum != 0 and self._velocity[i] is None:
                    # the first step writes v = g without reading it (vel_init = 0): no fill needed
                    self._velocity[i] = _C._empty_like(grad)
                if p.is_contiguous():
                    ps.append(p)
                    gs.append(grad)
                    vs.append(self._velocity[i])
                    inits.append(int(initialized))
                else:
                    _fused_update(p, grad, self._velocity[i], self.lr, self.momentum, self.weight_decay,
                                  self.dampening, int(self.nesterov), int(self.momentum != 0), int(initialized))
            if ps:
                _C._sgd_step_multi(ps, gs, vs if self.momentum != 0 else [], inits, self.lr, self.momentum,
                                   self.weight_decay, self.dampening, int(self.nesterov), int(self.momentum != 0))

    def zero_grad(self):
        for p in self.parameters:
            p.zero_grad()


class Muon:
    """Momentum, then an orthogonalised update for 2-D parameters (Newton-Schulz iteration); other
    parameters take the plain momentum update. Same arguments and arithmetic as the reference."""

    def __init__(self, parameters, lr=0.02, momentum=0.95, ns_steps=5, weight_decay=0.0):
        self.parameters = list(parameters)
        self.lr = lr
        self.momentum = momentum
        self.ns_steps = ns_steps
        self.weight_decay = weight_decay
        self._buf = [None] * len(self.parameters)

    @staticmethod
    def _newton_schulz_orthogonalize(G, steps):
        norm = (float(_C._mean_square(G).item()) * G.size) ** 0.5
        X = G * (1.0 / (norm + 1e-7))
        a, b, c = 3.4445, -4.7750, 2.0315
        for _ in range(steps):
            A = _C.cuda_matmul(X.transpose(0, 1), X)         # X^T X, the transposed view read in place
            B = _C.matmul_axpby(A, A, c, b, A)               # b * A + c * (A @ A)
            X = _C.matmul_axpby(X, B, 1.0, a, X)             # a * X + X @ B
        return X

    def step(self):
        with no_grad():
            for i, p in enumerate(self.parameters):
                if p.grad is None:
                    continue
                grad = p.grad
                if self.weight_decay != 0:
                    grad = grad + p * self.weight_decay
                if self._buf[i] is None:
                    self._buf[i] = grad
                else:
                    self._buf[i] = self._buf[i] * self.momentum + grad * (1 - self.momentum)
                if len(p.shape) == 2:
                    update = self._newton_schulz_orthogonalize(self._buf[i], self.ns_steps)
                else:
                    update = self._buf[i]
                upd = update if update.is_contiguous() else update.contiguous()
                _fused_update(p, upd, None, self.lr, 0.0, 0.0, 0.0, 0, 0, 0)        # p -= lr * update

    def zero_grad(self):
        for p in self.parameters:
            p.zero_grad()
