"""Autocorrelation (dense Gram) Hessian: ``H_m = (1/R) sum_rows vec(P)^T vec(P)``
(reference ``bergson/hessians/autocorrelation.py:15-63``)."""

from __future__ import annotations

import math
from dataclasses import dataclass
from pathlib import Path

import torch.nn as nn
from datasets import Dataset
from torch import Tensor

from ..collector.collector import HookCollectorBase
from ..process_autocorrelation import process_autocorrelation_matrices


@dataclass(kw_only=True)
class AutocorrelationCollector(HookCollectorBase):
    data: Dataset
    path: str

    def setup(self) -> None:
        assert self.processor.projection_target != "global", (
            "Autocorrelation Hessian fitting requires per-module projection; projection_target='global' "
            "sums all modules into a single key and has no per-module Hessian."
        )

    @HookCollectorBase.split_attention_heads
    def backward_hook(self, module: nn.Module, g: Tensor):
        name: str = module._name
        P = self._compute_gradient(module, g).float()
        if name in self.processor.hessians:
            self.processor.hessians[name].addmm_(P.mT, P)
        else:
            self.processor.hessians[name] = P.mT @ P

    def process_batch(self, indices: list[int], **kwargs):
        return

    def teardown(self):
        sizes = {n: math.prod(s) for n, s in self.shapes().items()}
        if self.processor.hessians:
            process_autocorrelation_matrices(
                self.processor, self.processor.hessians, self.num_rows(self.data), sizes, self.rank
            )
        if self.rank == 0:
            self.processor.save(Path(self.path))
