"""Scores index gradients against query gradients:
``scores[b, q] = sum_m <g_b[m], q_q[m]>``, optionally divided by ``||g_b||`` (cosine;
the queries are normalised once up front) and reduced with ``max`` over queries
(reference ``bergson/score/scorer.py:9-115``).

On CUDA with 16-bit scoring dtype the inner products run in the tcgen05 TN GEMM over
the concatenated module dimension; otherwise per-module ``torch`` GEMMs are used.
"""

from __future__ import annotations

from collections.abc import Callable

import torch
from torch import Tensor

from .score_writer import ScoreWriter


class GatheredQueries:
    """Query rows kept sharded over the ranks of a process group, in a symmetric peer-memory
    heap.  ``scores(rows)`` is one kernel: the score GEMM whose query operand is read, tile by
    tile, straight from the owning ranks' memory over NVLink (an all-gather fused into the
    GEMM's operand loads), so no rank ever holds a gathered copy of the queries.

    ``local_rows`` is this rank's ``[n_r, D]`` slice (``shard_bounds`` order: rank 0 takes the
    remainder); the heap region is sized for the largest slice and zero-padded."""

    def __init__(self, local_rows: Tensor, num_queries: int, dtype: torch.dtype, group=None):
        import torch.distributed as dist

        from ..hessians.sharded_computation import shard_bounds
        from ..parallel.peer import PeerHeap

        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.num_queries = num_queries
        bounds = [shard_bounds(num_queries, r, self.world) for r in range(self.world)]
        self.per_rank = max(hi - lo for lo, hi in bounds)
        lo, hi = bounds[self.rank]
        assert local_rows.shape[0] == hi - lo, (local_rows.shape, lo, hi)
        self.dim = local_rows.shape[1]
        self.heap = PeerHeap(self.per_rank * self.dim, dtype, group=group)
        view = self.heap.local.view(self.per_rank, self.dim)
        view.zero_()
        view[: hi - lo] = local_rows.to(view.device, dtype)
        # Output column of query q (global order) in the [B, world * per_rank] product.
        cols = torch.cat([torch.arange(b_lo, b_hi) - b_lo + r * self.per_rank for r, (b_lo, b_hi) in enumerate(bounds)])
        self.columns = cols.to(view.device)
        self.identity = self.world * self.per_rank == num_queries
        self.heap.barrier()  # every rank's slice is in place before anyone reads it

    def scores(self, rows: Tensor) -> Tensor:
        from ..parallel.peer import gathered_scores

        out = gathered_scores(rows, self.heap, 0, self.per_rank)
        return out if self.identity else out.index_select(1, self.columns)


class Scorer:
    def __init__(
        self,
        query_grads: dict[str, Tensor],
        modules: list[str],
        writer: ScoreWriter,
        device: torch.device,
        dtype: torch.dtype,
        *,
        unit_normalize: bool = False,
        score_mode: str = "individual",
        attribute_tokens: bool = False,
        index_transform: Callable[[dict[str, Tensor]], dict[str, Tensor]] | None = None,
        query_offset: int = 0,
        gathered: GatheredQueries | None = None,
    ):
        """``gathered``: the queries live sharded over the ranks (``query_grads`` then holds only
        this rank's slice, already laid out as concatenated rows inside ``gathered``); scoring
        goes through the fused all-gather + GEMM kernel."""
        self.device, self.dtype, self.modules = device, dtype, modules
        self.unit_normalize = unit_normalize
        self.score_mode = score_mode
        self.attribute_tokens = attribute_tokens
        self.writer = writer
        # Concatenated-row scoring (``score_rows``) is valid when no per-module transform
        # has to run on the index gradients first.
        self.supports_rows = index_transform is None
        self.index_transform = index_transform if index_transform is not None else (lambda g: g)
        self.query_offset = query_offset
        # [dim_m, n_queries] per module, ready for g @ q^T
        self.gathered = gathered
        self.query_grads_t = {} if gathered is not None else {
            m: query_grads[m].to(device=device, dtype=dtype).T for m in modules}
        self._module_dims = {m: query_grads[m].shape[1] for m in modules}
        self._q_cat: Tensor | None = None
        self._layout: dict[str, tuple[int, int]] | None = None

    def __call__(self, indices: list[int], mod_grads: dict[str, Tensor]):
        self.writer(indices, self.score(mod_grads), query_offset=self.query_offset)

    def set_row_layout(self, offsets: dict[str, tuple[int, int]], total: int) -> bool:
        """Tell the scorer how a producer lays out concatenated rows: ``offsets`` maps module
        names to their ``[lo, hi)`` columns of a ``total``-wide row.  The query operand of
        ``score_rows`` is then assembled in that layout, with zero columns for modules that
        this scorer does not score, so the producer's module set may be a superset of
        ``self.modules`` in any order.  Returns False when concatenated-row scoring cannot
        be used: a scored module is missing from the rows or has another width, or cosine
        scoring would see the norm of columns outside ``self.modules``."""
        if not self.supports_rows:
            return False
        if self.gathered is not None:
            # The sharded query rows were laid out in ``self.modules`` order when they were
            # placed in the heap; the producer must use exactly that layout.
            lo = 0
            for m in self.modules:
                if offsets.get(m) != (lo, lo + self._module_dims[m]):
                    return False
                lo += self._module_dims[m]
            return lo == total and set(offsets) == set(self.modules)
        for m in self.modules:
            if m not in offsets or offsets[m][1] - offsets[m][0] != self.query_grads_t[m].shape[0]:
                return False
        if self.unit_normalize and set(offsets) != set(self.modules):
            return False
        n_q = next(iter(self.query_grads_t.values())).shape[1] if self.modules else 0
        q = torch.zeros(n_q, total, device=self.device, dtype=self.dtype)
        for m in self.modules:
            lo, hi = offsets[m]
            q[:, lo:hi] = self.query_grads_t[m].T
        self._q_cat = q
        return True

    def _q_rows(self) -> Tensor:
        """Queries as ``[n_queries, row width]`` (K-major operand of the fused GEMM); module
        order ``self.modules`` unless ``set_row_layout`` gave another layout."""
        if self._q_cat is None:
            self._q_cat = torch.cat([self.query_grads_t[m].T for m in self.modules], dim=1).contiguous()
        return self._q_cat

    @torch.inference_mode()
    def score_rows(self, rows: Tensor) -> Tensor:
        """Score concatenated rows ``[B, row width]`` laid out as ``_q_rows`` describes."""
        from ..ops import attribution

        if self.gathered is not None:
            rows = rows.to(self.device, self.dtype).contiguous()
            scores = self.gathered.scores(rows)
            sq = rows.float().pow(2).sum(1) if self.unit_normalize else None
        else:
            scores, sq = attribution.score_rows(rows.to(self.device), self._q_rows(), self.dtype, self.unit_normalize)
        if self.unit_normalize:
            scores = scores / sq.sqrt().clamp_min_(1e-12).unsqueeze(1)
        if self.score_mode == "nearest":
            return scores.max(dim=-1, keepdim=True).values
        return scores

    @torch.inference_mode()
    def score(self, index_grads: dict[str, Tensor]) -> Tensor:
        if self.gathered is not None:
            return self.score_rows(torch.cat([index_grads[m].to(self.device, self.dtype) for m in self.modules], dim=1))
        index_grads = self.index_transform(index_grads)
        scores = sq = None
        for m in self.modules:
            g = index_grads[m].to(self.device, self.dtype, non_blocking=True)
            part = g @ self.query_grads_t[m]
            scores = part if scores is None else scores.add_(part)
            if self.unit_normalize:
                n = g.pow(2).sum(dim=1)
                sq = n if sq is None else sq.add_(n)
        assert scores is not None, "Scorer requires at least one module"
        if self.unit_normalize:
            scores.div_(sq.sqrt().clamp_min_(1e-12).unsqueeze(1))
        if self.score_mode == "nearest":
            return scores.max(dim=-1, keepdim=True).values
        return scores
