"""Parameter sharding for the twice-differentiable trainer.

Every trainable parameter is stored as this rank's block of rows (dim 0 padded to a
multiple of the world size).  ``gather_params`` rebuilds the full tensors with the
differentiable all-gather of ``collectives``; its backward is a reduce-scatter, so
parameter gradients come back sharded (summed over ranks), and the backward of that is
again an all-gather: the whole step stays differentiable to any order.  The reference
reaches the same behaviour with DTensor ``Shard(0)`` parametrisations and a patched
redistribute backward (``bergson/magic/fsdp.py:20-87``, ``dtensor_patch.py``).
"""

from __future__ import annotations

import torch
import torch.distributed as dist
from torch import Tensor

from .collectives import all_gather_rows


def shallow_copy(tensors: dict[str, Tensor]) -> dict[str, Tensor]:
    """New tensor objects sharing storage (so in-place state edits do not alias the module)."""
    return {k: v.detach().clone() if v.device.type == "meta" else v.detach().view_as(v) for k, v in tensors.items()}


def _world() -> tuple[int, int]:
    if dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


def shard_param(full: Tensor) -> Tensor:
    """This rank's rows of ``full`` (zero-padded so that dim 0 divides evenly)."""
    rank, world = _world()
    if world == 1 or full.ndim == 0:
        return full
    rows = -(-full.shape[0] // world)
    pad = rows * world - full.shape[0]
    if pad:
        full = torch.cat([full, full.new_zeros(pad, *full.shape[1:])])
    return full[rank * rows : (rank + 1) * rows].clone()


def gather_param(shard: Tensor, full_shape: torch.Size) -> Tensor:
    """Differentiable inverse of ``shard_param``.  Its adjoint is a *summing* reduce-scatter;
    the trainer averages over ranks by scaling each rank's loss with ``1 / world`` instead,
    which keeps second-order terms correctly scaled as well."""
    _, world = _world()
    if world == 1 or len(full_shape) == 0:
        return shard
    return all_gather_rows(shard)[: full_shape[0]]


def simple_fsdp(params: dict[str, Tensor]) -> tuple[dict[str, Tensor], dict[str, torch.Size]]:
    """Shard a parameter dict; returns ``(shards, full_shapes)``."""
    shapes = {k: p.shape for k, p in params.items()}
    return {k: shard_param(p) for k, p in params.items()}, shapes


def gather_params(shards: dict[str, Tensor], shapes: dict[str, torch.Size]) -> dict[str, Tensor]:
    return {k: gather_param(s, shapes[k]) for k, s in shards.items()}
