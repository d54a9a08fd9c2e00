"""Tensor parallelism for the in-tree Llama family (attribution passes).

Megatron-style: q/k/v and gate/up projections are split along their output features
(whole heads per rank), o_proj and down_proj along their input features; the block input
is copied into the group (backward: all-reduce of the input gradient) and the block output
is all-reduced (backward: identity).  Module names are unchanged, so stores and normaliser
keys do not depend on the parallel layout.

On GPUs with peer memory the same sharding runs *sequence-parallel*: the residual stream is
split over tokens between blocks and both collectives move into the GEMM kernels
(all-gather -> GEMM for the column-parallel projections, GEMM -> reduce-scatter for the
row-parallel ones; see ``sequence_parallel``).

Per-example projected gradients need no gathering: ``P_out (G^T A) P_in^T`` is a sum over
the shards of the split dimension, so each rank projects with its *slice* of the projection
matrix and the ``[N, p, p]`` blocks are summed over the group (one all-reduce of the row
accumulator per batch).  The reference has no tensor parallelism.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn
from torch import Tensor

from . import topology


class _CopyToGroup(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g: Tensor):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromGroup(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, group):
        x = x.contiguous()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g: Tensor):
        return g, None


def copy_to_group(x: Tensor, group) -> Tensor:
    return x if group is None else _CopyToGroup.apply(x, group)


def reduce_from_group(x: Tensor, group) -> Tensor:
    return x if group is None else _ReduceFromGroup.apply(x, group)


def _shard_linear(lin: nn.Linear, dim: str, rank: int, size: int) -> nn.Linear:
    full = lin.out_features if dim == "out" else lin.in_features
    if full % size:
        raise ValueError(f"feature size {full} is not divisible by tensor_parallel={size}")
    step = full // size
    lo, hi = rank * step, (rank + 1) * step
    w = lin.weight.data[lo:hi] if dim == "out" else lin.weight.data[:, lo:hi]
    from ..ops.linear import Linear

    new = Linear(w.shape[1], w.shape[0], bias=False, device=w.device, dtype=w.dtype)
    new.weight = nn.Parameter(w.clone().contiguous(), requires_grad=lin.weight.requires_grad)
    if lin.bias is not None:
        raise ValueError("tensor parallelism supports bias-free projections only")
    new._tp_shard = (dim, lo, hi, full)  # read by the collectors to slice projections / scales
    return new


def apply_tensor_parallel(model, group=None):
    """Shard a ``LlamaForCausalLM`` in place over ``group`` (default: the topology's)."""
    from ..models.llama import LlamaForCausalLM

    group = group if group is not None else topology.tp_group()
    if group is None:
        return model
    if not isinstance(model, LlamaForCausalLM):
        raise NotImplementedError("tensor parallelism is implemented for the in-tree Llama family")
    size, rank = dist.get_world_size(group), dist.get_rank(group)
    for layer in model.model.layers:
        att, mlp = layer.self_attn, layer.mlp
        if att.num_heads % size or att.kv_heads % size:
            raise ValueError(f"heads ({att.num_heads}/{att.kv_heads}) are not divisible by tensor_parallel={size}")
        for name in ("q_proj", "k_proj", "v_proj"):
            setattr(att, name, _shard_linear(getattr(att, name), "out", rank, size))
        att.o_proj = _shard_linear(att.o_proj, "in", rank, size)
        att.num_heads //= size
        att.kv_heads //= size
        att.tp_group = group
        for name in ("gate_proj", "up_proj"):
            setattr(mlp, name, _shard_linear(getattr(mlp, name), "out", rank, size))
        mlp.down_proj = _shard_linear(mlp.down_proj, "in", rank, size)
        mlp.tp_group = group
    # With peer memory the blocks run sequence-parallel with the collectives inside the GEMMs
    # (``sequence_parallel``); the all-reduce path above remains for everything else (CPU / gloo,
    # odd token counts, trainable sharded weights, hook-based collectors).
    import os

    from .sequence_parallel import SeqParallel

    sp = SeqParallel(group)
    if os.environ.get("BERGSON_B200_DISABLE_PEER", "0") != "1" and sp.available():
        model._seq_parallel = sp
    return model
