"""Gradient transformations: ``(init, update)`` pairs over parameter trees, composed with
``chain``.  Every update is written with ordinary differentiable tensor operations;
``inplace=True`` switches the moment updates and the final scaling to their in-place forms."""

from __future__ import annotations

from typing import NamedTuple

import torch

from .pytree import tree_map
from .typing import GradientTransformation


class EmptyState(NamedTuple):
    pass


class ScaleByAdamState(NamedTuple):
    mu: object
    nu: object
    count: object


class TraceState(NamedTuple):
    trace: object


class ScaleByScheduleState(NamedTuple):
    count: torch.Tensor


def chain(*transformations: GradientTransformation) -> GradientTransformation:
    inits = [t.init for t in transformations]
    updates = [t.update for t in transformations]

    def init(params):
        return tuple(fn(params) for fn in inits)

    def update(grads, state, *, params=None, inplace=True):
        new_state = []
        for fn, s in zip(updates, state):
            grads, s = fn(grads, s, params=params, inplace=inplace)
            new_state.append(s)
        return grads, tuple(new_state)

    return GradientTransformation(init, update)


def identity() -> GradientTransformation:
    return GradientTransformation(lambda params: EmptyState(), lambda u, s, *, params=None, inplace=True: (u, s))


def scale(step_size: float) -> GradientTransformation:
    def update(updates, state, *, params=None, inplace=True):
        fn = (lambda g: g.mul_(step_size)) if inplace else (lambda g: g.mul(step_size))
        return tree_map(fn, updates), state

    return GradientTransformation(lambda params: EmptyState(), update)


def scale_by_schedule(schedule) -> GradientTransformation:
    def init(params):
        return ScaleByScheduleState(count=torch.zeros((), dtype=torch.int64))

    def update(updates, state, *, params=None, inplace=True):
        step_size = schedule(state.count)
        fn = (lambda g: g.mul_(step_size)) if inplace else (lambda g: g.mul(step_size))
        return tree_map(fn, updates), ScaleByScheduleState(count=state.count + 1)

    return GradientTransformation(init, update)


def scale_by_neg_lr(lr) -> GradientTransformation:
    if callable(lr):
        return scale_by_schedule(lambda count: -lr(count))
    return scale(-lr)


def add_decayed_weights(weight_decay: float = 0.0) -> GradientTransformation:
    if weight_decay == 0.0:
        return identity()

    def update(updates, state, *, params=None, inplace=True):
        assert params is not None, "weight decay needs the parameters"
        if inplace:
            fn = lambda g, p: g.add_(p.detach(), alpha=weight_decay)  # noqa: E731
        else:
            fn = lambda g, p: g.add(p, alpha=weight_decay)  # noqa: E731
        return tree_map(fn, updates, params), state

    return GradientTransformation(lambda params: EmptyState(), update)


def _moment(grads, moments, decay: float, order: int, inplace: bool):
    if order == 1:
        if inplace:
            return tree_map(lambda g, t: t.mul_(decay).add_(g, alpha=1 - decay), grads, moments)
        return tree_map(lambda g, t: t.mul(decay).add(g, alpha=1 - decay), grads, moments)
    if inplace:
        return tree_map(lambda g, t: t.mul_(decay).addcmul_(g, g, value=1 - decay), grads, moments)
    return tree_map(lambda g, t: t.mul(decay).addcmul(g, g, value=1 - decay), grads, moments)


def scale_by_adam(b1: float = 0.9, b2: float = 0.999, eps: float = 1e-8, eps_root: float = 0.0,
                  moment_requires_grad: bool = False) -> GradientTransformation:
    def init(params):
        zeros = lambda p: torch.zeros_like(p, requires_grad=moment_requires_grad)  # noqa: E731
        count = tree_map(lambda p: torch.zeros((), dtype=torch.int64, device=p.device), params)
        return ScaleByAdamState(mu=tree_map(zeros, params), nu=tree_map(zeros, params), count=count)

    def update(grads, state, *, params=None, inplace=True):
        mu = _moment(grads, state.mu, b1, 1, inplace)
        nu = _moment(grads, state.nu, b2, 2, inplace)
        count = tree_map(lambda c: c + 1, state.count)
        mu_hat = tree_map(lambda t, c: t.div(1 - b1**c), mu, count)
        nu_hat = tree_map(lambda t, c: t.div(1 - b2**c), nu, count)
        if inplace:
            out = tree_map(lambda m, v: m.div_(v.add_(eps_root).sqrt_().add_(eps)), mu_hat, nu_hat)
        else:
            out = tree_map(lambda m, v: m.div(v.add(eps_root).sqrt().add(eps)), mu_hat, nu_hat)
        return out, ScaleByAdamState(mu=mu, nu=nu, count=count)

    return GradientTransformation(init, update)


def trace(momentum: float = 0.9, dampening: float = 0.0, nesterov: bool = False,
          moment_requires_grad: bool = False) -> GradientTransformation:
    """Heavy-ball momentum as ``torch.optim.SGD`` applies it: the first step stores the
    gradient itself, later steps ``t = momentum t + (1 - dampening) g``."""
    if momentum == 0.0:
        return identity()
    first = [True]

    def init(params):
        return TraceState(trace=tree_map(lambda p: torch.zeros_like(p, requires_grad=moment_requires_grad), params))

    def update(grads, state, *, params=None, inplace=True):
        scale_g = 1.0 if first[0] else 1.0 - dampening
        first[0] = False
        if inplace:
            new = tree_map(lambda g, t: t.mul_(momentum).add_(g, alpha=scale_g), grads, state.trace)
            out = tree_map(lambda g, t: g.add_(t, alpha=momentum), grads, new) if nesterov else new
        else:
            new = tree_map(lambda g, t: t.mul(momentum).add(g, alpha=scale_g), grads, state.trace)
            out = tree_map(lambda g, t: g.add(t, alpha=momentum), grads, new) if nesterov else new
        return out, TraceState(trace=new)

    return GradientTransformation(init, update)
