"""Collectives that are differentiable to any order.

Each is a linear map whose transpose is another collective of this module, so the
backward of one is an application of the other and autograd can differentiate a training
step twice (gradient synchronisation inside ``create_graph=True``) without special cases:

* ``all_reduce_sum``        backward: ``all_reduce_sum``
* ``all_gather_rows``       backward: ``reduce_scatter_rows`` (sum)
* ``reduce_scatter_rows``   backward: ``all_gather_rows``

The reference gets the first from a custom autograd function
(``bergson/magic/trainer.py:80-96``) and the other two by patching DTensor's
redistribute backward (``bergson/magic/dtensor_patch.py``).
"""

from __future__ import annotations

import torch
import torch.distributed as dist
from torch import Tensor


def _world(group) -> int:
    return dist.get_world_size(group) if dist.is_initialized() else 1


def _is_gloo(group) -> bool:
    return dist.get_backend(group) == "gloo"


def _all_gather_raw(shard: Tensor, group) -> Tensor:
    w = _world(group)
    shard = shard.contiguous()
    if _is_gloo(group):  # Gloo has no fused all-gather into one tensor
        parts = [torch.empty_like(shard) for _ in range(w)]
        dist.all_gather(parts, shard, group=group)
        return torch.cat(parts, dim=0)
    out = torch.empty((w * shard.shape[0], *shard.shape[1:]), dtype=shard.dtype, device=shard.device)
    dist.all_gather_into_tensor(out, shard, group=group)
    return out


def _reduce_scatter_raw(full: Tensor, group) -> Tensor:
    w = _world(group)
    rows = full.shape[0] // w
    if _is_gloo(group):  # Gloo has no reduce-scatter: all-reduce and keep this rank's rows
        tmp = full.clone()
        dist.all_reduce(tmp, op=dist.ReduceOp.SUM, group=group)
        r = dist.get_rank(group)
        return tmp[r * rows : (r + 1) * rows].clone()
    out = torch.empty((rows, *full.shape[1:]), dtype=full.dtype, device=full.device)
    dist.reduce_scatter_tensor(out, full.contiguous(), op=dist.ReduceOp.SUM, group=group)
    return out


class _AllReduceSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, group):
        ctx.group = group
        out = x.clone()
        dist.all_reduce(out, op=dist.ReduceOp.SUM, group=group)
        return out

    @staticmethod
    def backward(ctx, g: Tensor):
        return _AllReduceSum.apply(g, ctx.group), None


class _AllGatherRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, shard: Tensor, group):
        ctx.group = group
        return _all_gather_raw(shard, group)

    @staticmethod
    def backward(ctx, g: Tensor):
        return _ReduceScatterRows.apply(g, ctx.group), None


class _ReduceScatterRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, full: Tensor, group):
        ctx.group = group
        return _reduce_scatter_raw(full, group)

    @staticmethod
    def backward(ctx, g: Tensor):
        return _AllGatherRows.apply(g, ctx.group), None


class _AllGatherRowsStarted(torch.autograd.Function):
    """``all_gather_rows`` whose data movement was started earlier: the forward only hands out
    the gathered tensor, the backward is the same reduce-scatter."""

    @staticmethod
    def forward(ctx, shard: Tensor, gathered: Tensor, group):
        ctx.group = group
        return gathered.view_as(gathered)

    @staticmethod
    def backward(ctx, g: Tensor):
        return _ReduceScatterRows.apply(g, ctx.group), None, None


def start_all_gather_rows(shard: Tensor, group=None):
    """Begin ``all_gather_rows(shard)`` without waiting for it: returns a handle for
    ``finish_all_gather_rows``.  The shard must not change until then."""
    w = _world(group)
    src = shard.detach().contiguous()
    if _is_gloo(group):
        parts = [torch.empty_like(src) for _ in range(w)]
        return dist.all_gather(parts, src, group=group, async_op=True), parts, src
    out = torch.empty((w * src.shape[0], *src.shape[1:]), dtype=src.dtype, device=src.device)
    return dist.all_gather_into_tensor(out, src, group=group, async_op=True), out, src


def finish_all_gather_rows(shard: Tensor, handle, group=None) -> Tensor:
    """The gathered tensor of a started all-gather, attached to ``shard``'s autograd history."""
    work, out, _src = handle
    work.wait()
    gathered = torch.cat(out, dim=0) if isinstance(out, list) else out
    return _AllGatherRowsStarted.apply(shard, gathered, group)


def all_reduce_sum(x: Tensor, group=None) -> Tensor:
    if not dist.is_initialized() or _world(group) == 1:
        return x
    return _AllReduceSum.apply(x, group)


def all_gather_rows(shard: Tensor, group=None) -> Tensor:
    """Concatenate every rank's ``[r, ...]`` shard along dim 0."""
    if not dist.is_initialized() or _world(group) == 1:
        return shard
    return _AllGatherRows.apply(shard, group)


def reduce_scatter_rows(full: Tensor, group=None) -> Tensor:
    """Sum over ranks and keep this rank's block of rows (dim 0 divisible by world)."""
    if not dist.is_initialized() or _world(group) == 1:
        return full
    return _ReduceScatterRows.apply(full, group)
