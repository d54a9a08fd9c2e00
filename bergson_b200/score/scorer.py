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

    def _q_rows(self) -> Tensor:
        """Queries as ``[n_queries, sum_m dim_m]`` (K-major operand of the fused GEMM)."""
        if self._q_cat is None:
            self._q_cat = torch.cat([self.query_grads_t[m].T for m in self.modules], dim=1).contiguous()
        return self._q_cat

    @torch.inference_mode()
    def score_rows(self, rows: Tensor) -> Tensor:
        """Score concatenated rows ``[B, sum_m dim_m]`` (module order = ``self.modules``)."""
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
