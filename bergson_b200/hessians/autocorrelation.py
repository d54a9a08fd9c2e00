"""Autocorrelation Hessian: the mean outer product of the projected per-example gradient
blocks of every module, ``H_m = (1/R) sum_r vec(P_r,m)^T vec(P_r,m)``.

One pass over the data.  On CUDA the blocks come from the taps on the layers' own GEMMs
(the batch's rows land in one fp32 accumulator) and all modules' Grams advance with one
batched product per batch (``hessians.gram.GramAccumulator``); modules that the fused path
does not cover, and CPU runs, contribute their blocks through the generic hook expressions.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from pathlib import Path

import torch.nn as nn
from datasets import Dataset
from torch import Tensor

from ..collector.collector import HookCollectorBase
from ..data import column_offsets
from .gram import GramAccumulator


@dataclass(kw_only=True)
class AutocorrelationCollector(HookCollectorBase):
    data: Dataset
    path: str

    def setup(self) -> None:
        if self.processor.projection_target == "global":
            raise AssertionError(
                "An autocorrelation Hessian is fitted per module; projection_target='global' folds every module "
                "into one vector, for which no per-module statistic exists.")
        self.sizes = {name: math.prod(shape) for name, shape in self.shapes().items()}
        self.gram = GramAccumulator(self.sizes)
        self._pending: dict[str, Tensor] = {}
        spans = column_offsets(self.sizes)
        self.enable_fused({n: lo for n, (lo, _) in spans.items()}, sum(self.sizes.values()))

    @HookCollectorBase.split_attention_heads
    def backward_hook(self, module: nn.Module, g: Tensor):
        if self.compute_gradient_fused(module, g):
            return
        block = self._compute_gradient(module, g)
        if self._fused_enabled:
            self.mod_grads[module._name] = block  # merged into the batch's rows in process_batch
        else:
            self._pending[module._name] = block

    def process_batch(self, indices: list[int], **kwargs):
        if self._fused_enabled:
            self.gram.add_rows(self.fused_rows().clamp(self.lo, self.hi))
            self.mod_grads.clear()
        elif self._pending:
            self.gram.add_blocks(self._pending)
            self._pending = {}

    def teardown(self):
        self.gram.finish(self.processor, self.num_rows(self.data), self.rank)
        if self.rank == 0:
            self.processor.save(Path(self.path))
