"""Finite-difference checks of attribution scores against actual parameter perturbations
(reference ``bergson/utils/gradcheck.py:10-114``)."""

from __future__ import annotations

from contextlib import contextmanager

import torch
from torch import nn


def _xor_swap_(a: torch.Tensor, b: torch.Tensor) -> None:
    """Exchange the contents of two equally-shaped tensors in place, without a temporary,
    through XOR on their byte views."""
    av, bv = a.view(torch.uint8), b.view(torch.uint8)
    av.bitwise_xor_(bv)
    bv.bitwise_xor_(av)
    av.bitwise_xor_(bv)


class FiniteDiff:
    """``with fd.perturbed(sign): loss = f()`` evaluates ``f`` at ``theta + sign * eps * d``
    for a direction dict ``d`` (parameter name -> tensor); ``derivative(f)`` is the central
    difference ``(f(+) - f(-)) / (2 eps)``."""

    def __init__(self, model: nn.Module, direction: dict[str, torch.Tensor], eps: float = 1e-3):
        self.model, self.direction, self.eps = model, direction, eps
        self.params = dict(model.named_parameters())

    @contextmanager
    def perturbed(self, sign: float = 1.0):
        moved = {}
        with torch.no_grad():
            for name, d in self.direction.items():
                p = self.params[name]
                new = (p + sign * self.eps * d.to(p)).contiguous()
                _xor_swap_(p.data, new)  # p now holds the perturbed values, `new` the originals
                moved[name] = new
        try:
            yield
        finally:
            with torch.no_grad():
                for name, old in moved.items():
                    _xor_swap_(self.params[name].data, old)

    def derivative(self, fn) -> float:
        with self.perturbed(+1.0):
            hi = float(fn())
        with self.perturbed(-1.0):
            lo = float(fn())
        return (hi - lo) / (2 * self.eps)


def compute_effect(model: nn.Module, grads: dict[str, torch.Tensor], fn, eps: float = 1e-3) -> tuple[float, float]:
    """(finite-difference directional derivative of ``fn`` along ``grads``, its first-order
    prediction ``sum <grad_fn, grads>`` if ``fn`` is differentiable else nan)."""
    fd = FiniteDiff(model, grads, eps).derivative(fn)
    try:
        loss = fn()
        names = [n for n in grads]
        g = torch.autograd.grad(loss, [dict(model.named_parameters())[n] for n in names], allow_unused=True)
        pred = sum(float((a * grads[n].to(a)).sum()) for n, a in zip(names, g) if a is not None)
    except RuntimeError:
        pred = float("nan")
    return fd, pred
