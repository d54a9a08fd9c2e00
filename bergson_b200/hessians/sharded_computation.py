"""Row-sharded linear algebra for Kronecker factors.

Factors are stored row-sharded (``shard_bounds``: rank 0 takes the remainder).  The
reference applies a sharded factor with one broadcast per rank per product
(``bergson/hessians/sharded_computation.py:160-255``).  Here a product needs the whole
factor exactly once: ``gather_rows`` assembles it with a single all-gather into local
memory (cached by the caller when it is reused across batches), and the product is one
local GEMM.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
from torch import Tensor

from ..utils.utils import get_device


def shard_bounds(dim: int, rank: int, world_size: int) -> tuple[int, int]:
    """``[start, end)`` of ``rank``'s rows: sizes are ``[base + rem, base, ..., base]``."""
    base, rem = divmod(dim, world_size)
    if rank == 0:
        return 0, base + rem
    start = rem + rank * base
    return start, start + base


class ShardedMul:
    """Products and scalings with row-sharded matrices; every rank ends with the full
    result.  Without a process group the "shard" is the whole matrix."""

    def __init__(self):
        self.dist = dist.is_initialized() and dist.get_world_size() > 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.world_size = dist.get_world_size() if dist.is_initialized() else 1
        self.device = torch.device(get_device(self.rank))

    def shard_bounds(self, dim: int, rank: int | None = None) -> tuple[int, int]:
        return shard_bounds(dim, self.rank if rank is None else rank, self.world_size)

    def _init_covariance_dict(self, activation_covariance_dict, gradient_covariance_dict, dtype, target_info):
        """Zeroed row shards of ``A^T A`` ([I(+1)] square) and ``G^T G`` ([O] square)."""
        for name, (_, (o, i), bias) in target_info.items():
            i_full = i + (1 if bias else 0)
            lo, hi = self.shard_bounds(i_full)
            activation_covariance_dict[name] = torch.zeros(hi - lo, i_full, device=self.device, dtype=dtype)
            lo, hi = self.shard_bounds(o)
            gradient_covariance_dict[name] = torch.zeros(hi - lo, o, device=self.device, dtype=dtype)

    def gather_rows(self, shard: Tensor, full_rows: int) -> Tensor:
        """Full ``[full_rows, b]`` matrix from every rank's row shard (one all-gather;
        uneven shards are padded to the largest)."""
        if not self.dist:
            return shard
        sizes = [self.shard_bounds(full_rows, r) for r in range(self.world_size)]
        biggest = max(hi - lo for lo, hi in sizes)
        padded = shard
        if shard.shape[0] < biggest:
            padded = torch.zeros(biggest, *shard.shape[1:], device=shard.device, dtype=shard.dtype)
            padded[: shard.shape[0]] = shard
        out = torch.empty(self.world_size * biggest, *shard.shape[1:], device=shard.device, dtype=shard.dtype)
        dist.all_gather_into_tensor(out, padded.contiguous())
        if all(hi - lo == biggest for lo, hi in sizes):
            return out
        return torch.cat([out[r * biggest : r * biggest + (hi - lo)] for r, (lo, hi) in enumerate(sizes)], dim=0)

    def _matmul(self, vector_nsa: Tensor, matrix_cb: Tensor) -> Tensor:
        """``x [n, s, a] @ M [a, b]`` where ``matrix_cb`` is this rank's rows of ``M``."""
        a = vector_nsa.shape[2]
        lo, hi = self.shard_bounds(a)
        assert matrix_cb.shape[0] == hi - lo, (
            f"Vector shape {vector_nsa.shape} not compatible with matrix shape {matrix_cb.shape} "
            f"and world_size {self.world_size}"
        )
        full = self.gather_rows(matrix_cb, a)
        return vector_nsa.to(full.dtype) @ full

    def _transpose_matmul(self, vector_nsa: Tensor, matrix_cb: Tensor) -> Tensor:
        """``x [n, s, a] @ M^T`` with ``M [b, a]`` row-sharded along ``b``."""
        if not self.dist:
            return vector_nsa.to(matrix_cb.dtype) @ matrix_cb.T
        full = self.gather_rows(matrix_cb, matrix_cb.shape[1])
        return vector_nsa.to(full.dtype) @ full.T

    def global_mean(self, x_shard: Tensor, full_numel: int) -> Tensor:
        total = x_shard.sum()
        if self.dist:
            dist.all_reduce(total, op=dist.ReduceOp.SUM)
        return total / full_numel

    def scale_rows_in_place(self, matrix_noi: Tensor, inverse_eigvals_ci: Tensor) -> None:
        """``matrix[:, rows_r, :] *= shard_r`` for every rank's shard."""
        full = self.gather_rows(inverse_eigvals_ci, matrix_noi.shape[1])
        matrix_noi.mul_(full)
