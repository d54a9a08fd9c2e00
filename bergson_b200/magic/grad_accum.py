"""Micro-batched gradients and the memory-bounded VJP through one training step
(reference ``bergson/magic/grad_accum.py:29-337``).

``grads = sum_i c_i * grad(L_i)`` with ``c_i = denom_i / denom``; differentiating a step
therefore splits into (A) the VJP through reduce / clip / optimizer update, which yields a
cotangent on the combined gradient, and (B) one double backward per micro-batch against
that cotangent, each graph freed before the next.
"""

from __future__ import annotations

from collections.abc import Callable
from typing import Any

import torch
import torch.distributed as dist
from torch import nn

from ..distributed import grad_tree


def maybe_get_cuda_rng_state() -> torch.Tensor:
    if torch.cuda.is_available() and torch.cuda.is_initialized():
        return torch.cuda.random.get_rng_state()
    return torch.zeros(16, dtype=torch.uint8)


def maybe_set_cuda_rng_state(state: torch.Tensor) -> None:
    if torch.cuda.is_available() and torch.cuda.is_initialized():
        torch.cuda.random.set_rng_state(state.cpu())


def rng_snapshot():
    return torch.random.get_rng_state(), maybe_get_cuda_rng_state()


def rng_restore(snapshot) -> None:
    torch.random.set_rng_state(snapshot[0])
    maybe_set_cuda_rng_state(snapshot[1])


def loss_denom(batch: dict) -> float:
    """Denominator of the "mean" loss reduction: supervised-token count, at least 1."""
    mask = batch.get("shift_loss_mask")
    if mask is not None:
        return max(float(mask.sum()), 1.0)
    labels = batch.get("labels")
    if labels is not None:
        return max(float((labels[:, 1:] != -100).sum()), 1.0)
    return float(batch["input_ids"].shape[1] - 1)


def split_batch(inputs: dict, n: int) -> list[dict]:
    """Up to ``n`` micro-batches along dim 0; non-batch entries are shared."""
    bs = next(v for v in inputs.values() if isinstance(v, torch.Tensor) and v.ndim >= 1).shape[0]
    n = max(1, min(n, bs))
    sizes = [bs // n + (1 if i < bs % n else 0) for i in range(n)]
    out, off = [], 0
    for size in sizes:
        out.append({
            k: v[off : off + size] if isinstance(v, torch.Tensor) and v.ndim >= 1 and v.shape[0] == bs else v
            for k, v in inputs.items()
        })
        off += size
    return out


def _loss_of(outputs) -> torch.Tensor:
    loss = outputs.loss if hasattr(outputs, "loss") else outputs
    assert isinstance(loss, torch.Tensor), "Loss must be a Tensor"
    return loss


def accumulate_grads(call_model: Callable[[dict, dict], Any], params: dict, inputs: dict, grad_accum_steps: int, *,
                     create_graph: bool, rng_snapshots: list | None = None, loss_scale: float = 1.0) -> tuple[dict, float]:
    """Full-batch gradient as the sum of rescaled micro-batch gradients.
    ``call_model(params, micro_batch)`` runs the forward pass with ``params``.  ``loss_scale``
    multiplies the differentiated loss (``1 / world`` under parameter sharding, where the
    gradient reduction over ranks is a sum); the returned loss value is unscaled."""
    total = loss_denom(inputs)
    grads: dict | None = None
    loss_value = 0.0
    for mb in split_batch(inputs, grad_accum_steps):
        if rng_snapshots is not None:
            rng_snapshots.append(rng_snapshot())
        loss = _loss_of(call_model(params, mb))
        coef = loss_denom(mb) / total
        loss_value += float(loss.detach()) * coef
        g = grad_tree(loss * (coef * loss_scale), params, create_graph=create_graph)
        if grads is None:
            grads = dict(g)
        else:
            for k, v in g.items():
                if v is not None:
                    grads[k] = v if grads[k] is None else grads[k] + v
    assert grads is not None
    return grads, loss_value


def microbatch_step_vjp(call_model, apply_update, fwd_state, inputs: dict[str, Any], param_grads: dict,
                        opt_grads: list, data_weights: torch.Tensor, *, model_training: bool = False,
                        loss_scale: float = 1.0,
                        fsdp: bool = False, max_grad_norm: float | None = None, grad_accum_steps: int = 1,
                        double_backward_batch_size: int | None = None):
    """Returns ``(param_cotangents, opt_cotangents, weight_cotangent)`` of one step."""
    flat_in = fwd_state.differentiable_tensors()
    keys = list(param_grads)
    n_params, n_in = len(keys), len(flat_in)

    # Stage 0: gradient values (no graph); remember where each micro-batch's RNG started.
    rng_restore((fwd_state.cpu_rng_state, fwd_state.cuda_rng_state))
    snaps: list = []
    detached = {k: v.detach().requires_grad_(True) for k, v in fwd_state.params.items()}
    g0, _ = accumulate_grads(call_model, detached, inputs, grad_accum_steps, create_graph=False, rng_snapshots=snaps,
                             loss_scale=loss_scale)
    g_vars = {k: v.detach().clone().requires_grad_(True) for k, v in g0.items() if v is not None}

    # Stage A: VJP through reduce / clip / update only.
    nxt = apply_update(fwd_state, g_vars, inplace=False, trace=True, fsdp=fsdp, max_grad_norm=max_grad_norm)
    res = list(torch.autograd.grad(nxt.differentiable_tensors(), flat_in + list(g_vars.values()),
                                   grad_outputs=list(param_grads.values()) + opt_grads, allow_unused=True))
    zero = lambda c, ref: c if c is not None else torch.zeros_like(ref)  # noqa: E731
    p_cot = [zero(res[i], flat_in[i]).clone() for i in range(n_params)]
    o_cot = [zero(res[i], flat_in[i]) for i in range(n_params, n_in)]
    g_cot = {k: zero(c, g_vars[k]) for k, c in zip(g_vars, res[n_in:])}
    del g0, g_vars, nxt, res

    ex_w = inputs.get("example_weight")
    ex_cot = torch.zeros_like(ex_w) if ex_w is not None else None

    # Stage B: one double backward per micro-batch.
    total = loss_denom(inputs)
    work = list(zip(split_batch(inputs, grad_accum_steps), snaps))
    if double_backward_batch_size is not None and not model_training:
        work = [(sub, s) for mb, s in work
                for sub in split_batch(mb, -(-mb["input_ids"].shape[0] // double_backward_batch_size))]
    index = {k: i for i, k in enumerate(keys)}
    off = 0
    for mb, snap in work:
        rng_restore(snap)
        params = fwd_state.params
        loss = _loss_of(call_model(params, mb))
        mg = grad_tree(loss * (loss_denom(mb) / total * loss_scale), params, create_graph=True)
        gk = [k for k, v in mg.items() if v is not None and k in g_cot]
        targets = [params[k] for k in gk]
        mb_w = mb.get("example_weight")
        if mb_w is not None:
            targets.append(mb_w)
        contrib = torch.autograd.grad([mg[k] for k in gk], targets, grad_outputs=[g_cot[k] for k in gk],
                                      allow_unused=True)
        for i, k in enumerate(gk):
            if contrib[i] is not None:
                p_cot[index[k]] = p_cot[index[k]] + contrib[i]
        if mb_w is not None and contrib[-1] is not None and ex_cot is not None:
            n = mb_w.shape[0]
            ex_cot[off : off + n] = ex_cot[off : off + n] + contrib[-1]
        if mb_w is not None:
            off += mb_w.shape[0]
        del mg, contrib, loss

    w_cot = torch.zeros_like(data_weights)
    if ex_w is not None and ex_cot is not None and float(ex_cot.abs().sum()) > 0:
        if ex_w is data_weights:
            w_cot = w_cot + ex_cot
        else:
            (dw,) = torch.autograd.grad(ex_w, data_weights, grad_outputs=ex_cot, allow_unused=True)
            if dw is not None:
                w_cot = w_cot + dw
    if dist.is_initialized() and not fsdp:
        # A document contributes to 1/world of the averaged gradient.
        w_cot = w_cot / dist.get_world_size()
    return {k: p_cot[i] for i, k in enumerate(keys)}, o_cot, w_cot
