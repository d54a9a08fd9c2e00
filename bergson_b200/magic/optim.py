"""Functional, twice-differentiable optimizers.

The reference builds its optimizers from the third-party ``torchopt`` package
(``bergson/magic/trainer.py:1072-1096``) plus an in-repo Muon
(``bergson/magic/optim.py:27-269``).  This module provides the same update rules as
self-contained ``GradientTransformation(init, update)`` pairs whose state is a plain
nested dict of tensors, so that a training step can be differentiated with respect to
gradients, parameters and optimizer state to any order:

* ``adamw``: ``m = b1 m + (1-b1) g``, ``v = b2 v + (1-b2) g^2``, bias-corrected,
  ``u = m_hat / (sqrt(v_hat + eps_root) + eps) + wd * p``, step ``-lr(count) * u``;
* ``sgd``: ``g += wd * p``, heavy-ball ``t = g + momentum * t``, step ``-lr(count) * t``;
* ``muon``: 2-D params: Nesterov momentum, 5 quintic Newton-Schulz iterations
  (a, b, c = 3.4445, -4.7750, 2.0315), lr ratio ``0.2 sqrt(max(A, B))``, decoupled
  weight decay; other params: AdamW.

On CUDA, the non-traced (``inplace=True``) AdamW step runs as one multi-tensor kernel launch
(``GradientTransformation.step_inplace``: moments, bias correction, weight decay and the
parameter write in a single pass, with an optional device-side gradient coefficient so that
global-norm clipping needs no pass of its own); ``global_norm_coef`` computes that
coefficient with one multi-tensor reduction.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Callable

import torch
from torch import Tensor

Params = dict[str, Tensor]
OptState = dict[str, Any]
Schedule = Callable[[int], float]

NS_EPS = 1e-7
NS_COEFFS = (3.4445, -4.7750, 2.0315)
NS_STEPS = 5


@dataclass
class GradientTransformation:
    init: Callable[[Params], OptState]
    update: Callable[..., tuple[Params, OptState]]
    # Optional fused in-place step ``(grads, state, params, coef) -> (params, state) | None``;
    # None means "not applicable to these tensors", and the caller uses ``update``.
    step_inplace: Callable[..., tuple[Params, OptState] | None] | None = None
    # Optional fused out-of-place step that stays in the autograd graph (one launch forward,
    # one for its vector-Jacobian product): ``(grads, state, params) -> (params, state) | None``.
    step_traced: Callable[..., tuple[Params, OptState] | None] | None = None


_FUSED_DTYPES = (torch.float32, torch.bfloat16, torch.float16)


def _native():
    from ..ops import native

    return native if native.available() else None


def _fusable(tensors: list[Tensor]) -> bool:
    """One CUDA device, one element type the kernels take, contiguous, outside autograd."""
    if not tensors or _native() is None:
        return False
    first = tensors[0]
    return first.is_cuda and first.dtype in _FUSED_DTYPES and all(
        t.device == first.device and t.dtype == first.dtype and t.is_contiguous() and not t.requires_grad
        for t in tensors)


class _AdamWStepFn(torch.autograd.Function):
    """``(p, g, mu, nu) -> (p', mu', nu')`` for a whole parameter list in one launch; the
    backward is the step's vector-Jacobian product, also one launch.  Differentiable once:
    that is what a metagradient needs from the optimizer (the second-order terms live in the
    graph of ``g``)."""

    @staticmethod
    def forward(ctx, hp: tuple, n: int, *tensors: Tensor):
        ps, gs, ms, vs = (list(tensors[i * n : (i + 1) * n]) for i in range(4))
        po, mo, vo = _native().adamw_traced_fwd(ps, gs, ms, vs, *hp)
        ctx.save_for_backward(*gs, *ms, *vs)
        ctx.hp, ctx.n = hp, n
        return (*po, *mo, *vo)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, *cots):
        n = ctx.n
        saved = ctx.saved_tensors
        gs, ms, vs = list(saved[:n]), list(saved[n : 2 * n]), list(saved[2 * n :])
        cp, cm, cv = list(cots[:n]), list(cots[n : 2 * n]), list(cots[2 * n :])
        dp, dg, dm, dv = _native().adamw_traced_bwd(gs, ms, vs, cp, cm, cv, *ctx.hp)
        return (None, None, *dp, *dg, *dm, *dv)


def global_norm_coef(grads: list[Tensor], max_norm: float, *, reduce=None) -> Tensor | None:
    """``min(1, max_norm / (||grads||_2 + 1e-6))`` as a device scalar, from one multi-tensor
    sum-of-squares launch (partials added in a fixed order).  ``reduce`` (e.g. an all-reduce
    over ranks holding shards) is applied to the squared norm first.  None when the tensors
    are not eligible for the kernel."""
    if not _fusable(grads):
        return None
    out = torch.empty(2, device=grads[0].device, dtype=torch.float32)
    _native().multi_sumsq(grads, out, False, 0.0 if reduce is not None else float(max_norm))
    if reduce is None:
        return out[1:2]
    sq = reduce(out[0:1])
    return (max_norm / (sq.sqrt() + 1e-6)).clamp(max=1.0)


def apply_updates(params: Params, updates: Params, *, inplace: bool = False) -> Params:
    """``p + u`` per key (keys without an update are passed through)."""
    if inplace and params and not any(p.requires_grad for p in params.values()):
        keys = [k for k in params if updates.get(k) is not None]
        torch._foreach_add_([params[k] for k in keys], [updates[k].to(params[k].dtype) for k in keys])
        return dict(params)
    out = {}
    for k, p in params.items():
        u = updates.get(k)
        if u is None:
            out[k] = p
        elif inplace:
            out[k] = p.add_(u.to(p.dtype))
        else:
            out[k] = p + u.to(p.dtype)
    return out


def _lr_of(schedule: Schedule | float, count: Tensor) -> float:
    return float(schedule(int(count))) if callable(schedule) else float(schedule)


# --------------------------------------------------------------------------- #
# pytree helpers for the nested-dict optimizer state
# --------------------------------------------------------------------------- #


def tree_flatten_with_path(tree: Any, prefix: tuple = ()) -> list[tuple[tuple, Any]]:
    """Leaves of a nested dict / list with their key paths, dict keys in sorted order."""
    if isinstance(tree, dict):
        out = []
        for k in sorted(tree, key=str):
            out += tree_flatten_with_path(tree[k], prefix + (k,))
        return out
    if isinstance(tree, (list, tuple)):
        out = []
        for i, v in enumerate(tree):
            out += tree_flatten_with_path(v, prefix + (i,))
        return out
    return [(prefix, tree)]


def tree_iter(tree: Any):
    for _, leaf in tree_flatten_with_path(tree):
        yield leaf


def tree_map(fn: Callable, tree: Any, *rest: Any) -> Any:
    if isinstance(tree, dict):
        return {k: tree_map(fn, v, *(r[k] for r in rest)) for k, v in tree.items()}
    if isinstance(tree, (list, tuple)):
        return type(tree)(tree_map(fn, v, *(r[i] for r in rest)) for i, v in enumerate(tree))
    return fn(tree, *rest)


def tree_unflatten_like(tree: Any, leaves: list) -> Any:
    """Rebuild a tree of ``tree``'s structure from ``leaves`` in flatten order."""
    it = iter(leaves)

    def build(node):
        if isinstance(node, dict):
            vals = {k: None for k in node}
            for k in sorted(node, key=str):
                vals[k] = build(node[k])
            return vals
        if isinstance(node, (list, tuple)):
            return type(node)(build(v) for v in node)
        return next(it)

    return build(tree)


# --------------------------------------------------------------------------- #
# AdamW
# --------------------------------------------------------------------------- #


def _adam_direction(g, m, v, count: int, b1, b2, eps, eps_root, inplace: bool):
    if inplace:
        m = m.mul_(b1).add_(g, alpha=1 - b1)
        v = v.mul_(b2).addcmul_(g, g, value=1 - b2)
    else:
        m = m * b1 + g * (1 - b1)
        v = v * b2 + g * g * (1 - b2)
    m_hat = m / (1 - b1**count)
    v_hat = v / (1 - b2**count)
    return m_hat / ((v_hat + eps_root).sqrt() + eps), m, v


def adamw(lr: Schedule | float, betas=(0.9, 0.999), eps: float = 1e-8, eps_root: float = 0.0,
          weight_decay: float = 0.0) -> GradientTransformation:
    b1, b2 = betas

    def init(params: Params) -> OptState:
        return {
            "mu": {k: torch.zeros_like(p, dtype=torch.float32 if p.dtype != torch.float64 else p.dtype) for k, p in params.items()},
            "nu": {k: torch.zeros_like(p, dtype=torch.float32 if p.dtype != torch.float64 else p.dtype) for k, p in params.items()},
            "count": torch.zeros((), dtype=torch.long),
        }

    def update_foreach(grads: Params, state: OptState, params: Params):
        """In-place multi-tensor step for the untraced path: a handful of fused launches
        instead of a dozen small kernels per parameter."""
        count = state["count"] + 1
        step_lr = _lr_of(lr, state["count"])
        t = int(count)
        keys = [k for k in params if grads.get(k) is not None]
        mus, nus = [state["mu"][k] for k in keys], [state["nu"][k] for k in keys]
        gs = [grads[k].to(state["mu"][k].dtype) for k in keys]
        torch._foreach_mul_(mus, b1)
        torch._foreach_add_(mus, gs, alpha=1 - b1)
        torch._foreach_mul_(nus, b2)
        torch._foreach_addcmul_(nus, gs, gs, value=1 - b2)
        denom = torch._foreach_div(nus, 1 - b2**t)
        torch._foreach_add_(denom, eps_root)
        torch._foreach_sqrt_(denom)
        torch._foreach_add_(denom, eps)
        direction = torch._foreach_div(mus, 1 - b1**t)
        torch._foreach_div_(direction, denom)
        if weight_decay:
            torch._foreach_add_(direction, [params[k].to(d.dtype) for k, d in zip(keys, direction)], alpha=weight_decay)
        torch._foreach_mul_(direction, -step_lr)
        updates = {k: None for k in params}
        updates.update(dict(zip(keys, direction)))
        return updates, {"mu": state["mu"], "nu": state["nu"], "count": count}

    def step_inplace(grads: Params, state: OptState, params: Params, coef: Tensor | None = None):
        keys = [k for k in params if grads.get(k) is not None]
        ps, gs = [params[k] for k in keys], [grads[k] for k in keys]
        mus, nus = [state["mu"][k] for k in keys], [state["nu"][k] for k in keys]
        if not (_fusable(ps + gs) and all(t.dtype == torch.float32 and t.is_contiguous() for t in mus + nus)):
            return None
        t = int(state["count"]) + 1
        _native().adamw_multi(ps, mus, nus, gs, _lr_of(lr, state["count"]), b1, b2, eps, eps_root, weight_decay, t,
                              1.0, coef)
        return dict(params), {"mu": state["mu"], "nu": state["nu"], "count": state["count"] + 1}

    def step_traced(grads: Params, state: OptState, params: Params):
        keys = [k for k in params if grads.get(k) is not None]
        ps, gs = [params[k] for k in keys], [grads[k] for k in keys]
        mus, nus = [state["mu"][k] for k in keys], [state["nu"][k] for k in keys]
        first = ps[0] if ps else None
        if (first is None or _native() is None or not first.is_cuda or first.dtype not in _FUSED_DTYPES
                or not all(t.device == first.device and t.dtype == first.dtype for t in ps + gs)
                or not all(t.dtype == torch.float32 and t.device == first.device for t in mus + nus)):
            return None
        hp = (_lr_of(lr, state["count"]), b1, b2, eps, eps_root, weight_decay, int(state["count"]) + 1)
        n = len(keys)
        out = _AdamWStepFn.apply(hp, n, *(t.contiguous() for t in ps + gs + mus + nus))
        new_params, mu, nu = dict(params), dict(state["mu"]), dict(state["nu"])
        for i, k in enumerate(keys):
            new_params[k], mu[k], nu[k] = out[i], out[n + i], out[2 * n + i]
        return new_params, {"mu": mu, "nu": nu, "count": state["count"] + 1}

    def update(grads: Params, state: OptState, *, params: Params, inplace: bool = False):
        if inplace and not any(g is not None and g.requires_grad for g in grads.values()):
            return update_foreach(grads, state, params)
        count = state["count"] + 1
        step_lr = _lr_of(lr, state["count"])
        t = int(count)
        updates, mu, nu = {}, {}, {}
        for k, p in params.items():
            g = grads.get(k)
            if g is None:
                mu[k], nu[k], updates[k] = state["mu"][k], state["nu"][k], None
                continue
            d, mu[k], nu[k] = _adam_direction(g.to(state["mu"][k].dtype), state["mu"][k], state["nu"][k], t, b1, b2,
                                              eps, eps_root, inplace)
            if weight_decay:
                d = d + weight_decay * p
            updates[k] = -step_lr * d
        return updates, {"mu": mu, "nu": nu, "count": count}

    return GradientTransformation(init, update, step_inplace, step_traced)


# --------------------------------------------------------------------------- #
# SGD with heavy-ball momentum
# --------------------------------------------------------------------------- #


def sgd(lr: Schedule | float, momentum: float = 0.0, weight_decay: float = 0.0) -> GradientTransformation:
    def init(params: Params) -> OptState:
        return {"trace": {k: torch.zeros_like(p) for k, p in params.items()}, "count": torch.zeros((), dtype=torch.long)}

    def update(grads: Params, state: OptState, *, params: Params, inplace: bool = False):
        step_lr = _lr_of(lr, state["count"])
        updates, trace = {}, {}
        for k, p in params.items():
            g = grads.get(k)
            if g is None:
                trace[k], updates[k] = state["trace"][k], None
                continue
            if weight_decay:
                g = g + weight_decay * p
            t = state["trace"][k]
            t = t.mul_(momentum).add_(g) if inplace else t * momentum + g
            trace[k] = t
            updates[k] = -step_lr * t
        return updates, {"trace": trace, "count": state["count"] + 1}

    return GradientTransformation(init, update)


# --------------------------------------------------------------------------- #
# Muon
# --------------------------------------------------------------------------- #


def zeropower_via_newtonschulz(grad: Tensor) -> Tensor:
    """Quintic Newton-Schulz orthogonalisation ``X <- aX + (bA + cA^2)X``, ``A = XX^T``,
    on the Frobenius-normalised matrix (transposed so that rows <= columns)."""
    if grad.ndim != 2:
        raise ValueError("Input tensor gradient must be a 2D matrix")
    a, b, c = NS_COEFFS
    if (grad.is_cuda and grad.dtype in (torch.bfloat16, torch.float16) and grad.size(0) % 8 == 0
            and grad.size(1) % 8 == 0 and _native() is not None):
        return _newtonschulz_on_kernel(grad, a, b, c)
    x = grad.T if grad.size(0) > grad.size(1) else grad
    x = x / x.norm().clamp(min=NS_EPS)
    for _ in range(NS_STEPS):
        gram = x @ x.T
        poly = torch.addmm(gram, gram, gram, beta=b, alpha=c)
        x = torch.addmm(x, poly, x, beta=a)
    return x.T if grad.size(0) > grad.size(1) else x


def _newtonschulz_on_kernel(grad: Tensor, a: float, b: float, c: float) -> Tensor:
    """The same iteration with its three products per step on the tcgen05 GEMM (twice
    differentiable through ``_GemmFn``).  The matrix stays in its own storage orientation: a
    tall matrix iterates ``X <- aX + X (bA + cA^2)`` with ``A = X^T X``, which is the transpose
    of the wide form, so no transposed copy is made."""
    import sys

    import bergson_b200.ops  # noqa: F401 - makes sure the submodule is loaded

    gemm = sys.modules["bergson_b200.ops.linear"]._GemmFn.apply
    tall = grad.size(0) > grad.size(1)
    x = (grad / grad.norm().clamp(min=NS_EPS)).contiguous()
    for _ in range(NS_STEPS):
        gram = gemm(x, x, True, True, None) if tall else gemm(x, x, False, False, None)
        poly = b * gram + c * gemm(gram, gram, False, True, None)
        x = a * x + (gemm(x, poly, False, True, None) if tall else gemm(poly, x, False, True, None))
    return x


def adjust_lr(lr: float, mode: str | None, shape) -> float:
    A, B = shape[:2]
    if mode is None or mode == "original":
        return lr * math.sqrt(max(1, A / B))
    if mode == "match_rms_adamw":
        return lr * 0.2 * math.sqrt(max(A, B))
    return lr


def muon(lr: Schedule | float, momentum: float = 0.95, dampening: float = 0.0, weight_decay: float = 0.1,
         adamw_betas: tuple[float | None, float] = (None, 0.999), adamw_eps: float = 1e-8, adamw_eps_root: float = 0.0, *,
         moment_requires_grad: bool = False) -> GradientTransformation:
    """Argument order and defaults of the reference (``bergson/magic/optim.py:27-37``): the first
    AdamW beta defaults to ``momentum``; Nesterov momentum needs a positive ``momentum`` and no
    dampening; ``moment_requires_grad`` makes the initial momentum buffers leaves of the graph."""
    if not (callable(lr) or lr >= 0.0):
        raise ValueError(f"Invalid learning rate: {lr}")
    if not weight_decay >= 0.0:
        raise ValueError(f"Invalid weight_decay value: {weight_decay}")
    if momentum <= 0.0 or dampening != 0.0:
        raise ValueError("Nesterov momentum requires a momentum and zero dampening")
    b1, b2 = adamw_betas
    if b1 is None:
        b1 = momentum

    def init(params: Params) -> OptState:
        for p in params.values():
            if p.ndim > 2:
                raise ValueError(f"Muon does not support parameters with more than 2 dimensions, got shape {p.shape}")
        return {
            "trace": {k: torch.zeros_like(p, requires_grad=moment_requires_grad) for k, p in params.items() if p.ndim == 2},
            "mu": {k: torch.zeros_like(p) for k, p in params.items() if p.ndim != 2},
            "nu": {k: torch.zeros_like(p) for k, p in params.items() if p.ndim != 2},
            "count": torch.zeros((), dtype=torch.long),
        }

    def update(grads: Params, state: OptState, *, params: Params, inplace: bool = False):
        count = state["count"] + 1
        step_lr = _lr_of(lr, state["count"])
        first = int(state["count"]) == 0
        updates = {}
        trace, mu, nu = dict(state["trace"]), dict(state["mu"]), dict(state["nu"])
        for k, p in params.items():
            g = grads.get(k)
            if g is None:
                updates[k] = None
                continue
            if p.ndim > 2:
                raise ValueError(f"Muon does not support parameters with more than 2 dimensions, got shape {p.shape}")
            if p.ndim == 2:
                t = state["trace"][k]
                t = t + g if first else t * momentum + g
                trace[k] = t
                d = zeropower_via_newtonschulz(g + momentum * t).to(g.dtype) * adjust_lr(1.0, "match_rms_adamw", p.shape)
                if weight_decay:
                    d = d + weight_decay * p.detach()
            else:
                d, mu[k], nu[k] = _adam_direction(g, state["mu"][k], state["nu"][k], int(count), b1, b2, adamw_eps,
                                                  adamw_eps_root, False)
                if weight_decay:
                    d = d + weight_decay * p.detach()
            updates[k] = -step_lr * d
        return updates, {"trace": trace, "mu": mu, "nu": nu, "count": count}

    return GradientTransformation(init, update)
