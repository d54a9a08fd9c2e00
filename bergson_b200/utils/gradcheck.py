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
    """Two ways to move a model along a direction and back, bit for bit.

    * Direction given up front: ``with fd.perturbed(sign): loss = f()`` evaluates ``f`` at
      ``theta + sign * eps * d`` for a direction dict ``d`` (parameter name -> tensor);
      ``derivative(f)`` is the central difference ``(f(+) - f(-)) / (2 eps)``.
    * Direction taken from the gradients of a backward pass that has just run (the reference's
      protocol): ``store(step)`` turns every ``.grad`` buffer into ``theta + step * grad``
      (normalised first by the module's entry of ``normalizers``) and clears ``.grad``;
      ``with fd.apply():`` swaps those values into the model and back; ``clear()`` drops them.
    """

    def __init__(self, model: nn.Module, direction: dict[str, torch.Tensor] | None = None, eps: float = 1e-3, *,
                 normalizers: dict | None = None):
        self.model, self.direction, self.eps = model, direction or {}, eps
        self.normalizers = normalizers or {}
        self.params: dict[str, torch.Tensor] = {} if direction is None else dict(model.named_parameters())

    # -- gradients of the last backward pass as the direction --------------------------------

    def store(self, step_size: float) -> None:
        """``theta + step_size * grad`` for every parameter with a gradient, computed inside
        the gradient buffer (no extra memory); ``.grad`` is set to None."""
        used = 0
        stored: dict[str, torch.Tensor] = {}
        with torch.no_grad():
            for name, p in self.model.named_parameters():
                g = p.grad
                if g is None:
                    continue
                norm = self.normalizers.get(name.removesuffix(".weight")) if name.endswith(".weight") else None
                if norm is not None:
                    norm.normalize_weight(g)
                    used += 1
                torch.add(p.data, g, alpha=step_size, out=g)
                stored[name] = g
                p.grad = None
        if used != len(self.normalizers):
            raise ValueError(f"Expected {len(self.normalizers)} normalized gradients, but got {used}.")
        self.params = stored

    def swap(self) -> None:
        """Exchange the stored values with the model's parameters (twice = no change)."""
        with torch.no_grad():
            for name, p in self.model.named_parameters():
                buf = self.params.get(name)
                if buf is not None and buf is not p:
                    assert buf.shape == p.shape
                    _xor_swap_(buf, p.data)

    @contextmanager
    def apply(self):
        self.swap()
        try:
            yield self
        finally:
            self.swap()

    def clear(self) -> None:
        self.params.clear()

    # -- an explicit direction -----------------------------------------------------------------

    @contextmanager
    def perturbed(self, sign: float = 1.0):
        moved = {}
        named = dict(self.model.named_parameters())
        with torch.no_grad():
            for name, d in self.direction.items():
                p = named[name]
                new = (p + sign * self.eps * d.to(p)).contiguous()
                _xor_swap_(p.data, new)  # p now holds the perturbed values, `new` the originals
                moved[name] = new
        try:
            yield
        finally:
            with torch.no_grad():
                for name, old in moved.items():
                    _xor_swap_(named[name].data, old)

    def derivative(self, fn) -> float:
        def value() -> float:
            v = fn()
            return float(v.detach() if isinstance(v, torch.Tensor) else v)

        with self.perturbed(+1.0):
            hi = value()
        with self.perturbed(-1.0):
            lo = value()
        return (hi - lo) / (2 * self.eps)


def compute_effect(model: nn.Module, grads, fn=None, eps: float | None = None, *, normalizers: dict | None = None, x=None,
                   y=None):
    """Two forms.

    ``compute_effect(model, grads: dict, fn, eps)`` -> (finite-difference directional derivative of
    ``fn`` along ``grads``, its first-order prediction ``sum <grad_fn, grads>``, nan if ``fn`` is not
    differentiable).

    ``compute_effect(model, x, y, eps=, normalizers=)`` with token tensors (the reference's form):
    the change of the loss on ``y`` after moving the base model's parameters by ``eps`` along the
    (normalised) gradient of the loss on ``x``, divided by ``eps`` and by the parameter count.
    """
    if not isinstance(grads, dict):
        return _effect_of_example(model, grads if x is None else x, fn if y is None else y, eps, normalizers)
    eps = 1e-3 if eps is None else eps
    fd = FiniteDiff(model, grads, eps).derivative(fn)
    try:
        loss = fn()
        names = [n for n in grads]
        g = torch.autograd.grad(loss, [dict(model.named_parameters())[n] for n in names], allow_unused=True)
        pred = sum(float((a * grads[n].to(a)).sum()) for n, a in zip(names, g) if a is not None)
    except RuntimeError:
        pred = float("nan")
    return fd, pred


def _effect_of_example(model, x, y, eps, normalizers):
    fd = FiniteDiff(getattr(model, "base_model", model), normalizers=normalizers)
    dtype = next(model.parameters()).dtype
    eps = eps or torch.finfo(dtype).eps
    with torch.no_grad():
        before = model(y, labels=y).loss
    model(x, labels=x).loss.backward()
    fd.store(eps)
    model.zero_grad()
    with fd.apply(), torch.no_grad():
        after = model(y, labels=y).loss
    fd.clear()
    # For small eps the difference is an inner product of two gradients, whose size grows with the
    # number of parameters.
    n = sum(p.numel() for p in model.parameters())
    return (after - before) / (eps * n)
