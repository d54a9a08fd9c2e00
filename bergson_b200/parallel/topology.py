"""Process topology: ``world = data_parallel x tensor_parallel``.

Ranks ``[k * tp, (k + 1) * tp)`` form tensor-parallel group k (they hold shards of one model
replica and see the same data); ranks with equal position inside their group form a
data-parallel group.  With ``tp == 1`` everything degenerates to plain data parallelism.
"""

from __future__ import annotations

import torch.distributed as dist

_tp_size = 1
_tp_group = None
_dp_group = None


def init_topology(tp_size: int = 1) -> None:
    """Create the groups (collective: every rank must call it with the same ``tp_size``)."""
    global _tp_size, _tp_group, _dp_group
    _tp_size, _tp_group, _dp_group = 1, None, None
    if tp_size <= 1 or not dist.is_initialized():
        return
    world, rank = dist.get_world_size(), dist.get_rank()
    if world % tp_size:
        raise ValueError(f"world size {world} is not a multiple of tensor_parallel={tp_size}")
    _tp_size = tp_size
    for k in range(world // tp_size):
        ranks = list(range(k * tp_size, (k + 1) * tp_size))
        g = dist.new_group(ranks)
        if rank in ranks:
            _tp_group = g
    for j in range(tp_size):
        ranks = list(range(j, world, tp_size))
        g = dist.new_group(ranks)
        if rank in ranks:
            _dp_group = g


def reset_topology() -> None:
    global _tp_size, _tp_group, _dp_group
    _tp_size, _tp_group, _dp_group = 1, None, None


def tp_size() -> int:
    return _tp_size


def tp_group():
    return _tp_group


def tp_rank() -> int:
    return dist.get_rank() % _tp_size if _tp_size > 1 else 0


def data_rank_world() -> tuple[int, int]:
    """(rank, world) for data sharding: tensor-parallel peers count as one."""
    if not dist.is_initialized():
        return 0, 1
    return dist.get_rank() // _tp_size, dist.get_world_size() // _tp_size
