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
    ):
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
        self.query_grads_t = {m: query_grads[m].to(device=device, dtype=dtype).T for m in modules}
        self._q_cat: Tensor | None = None

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

        scores, sq = attribution.score_rows(rows.to(self.device), self._q_rows(), self.dtype, self.unit_normalize)
        if self.unit_normalize:
            scores = scores / sq.sqrt().clamp_min_(1e-12).unsqueeze(1)
        if self.score_mode == "nearest":
            return scores.max(dim=-1, keepdim=True).values
        return scores

    @torch.inference_mode()
    def score(self, index_grads: dict[str, Tensor]) -> Tensor:
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
