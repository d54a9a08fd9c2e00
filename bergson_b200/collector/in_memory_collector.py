"""Collector that keeps everything in host memory: gradients (via an in-memory
``Builder``), optional on-the-fly scores, optional autocorrelation Grams
(reference ``bergson/collector/in_memory_collector.py:24-183``)."""

from __future__ import annotations

import math
from dataclasses import dataclass
from dataclasses import field as dc_field

import torch
import torch.distributed as dist
from datasets import Dataset
from torch import Tensor, nn

from ..builder import Builder
from ..config import IndexConfig, PreprocessConfig
from ..process_autocorrelation import process_autocorrelation_matrices
from ..score.scorer import Scorer
from ..utils.utils import numpy_to_tensor
from .collector import HookCollectorBase
from .gradient_collectors import resolve_save_dtype


@dataclass(kw_only=True)
class InMemoryCollector(HookCollectorBase):
    data: Dataset
    cfg: IndexConfig
    skip_hessians: bool = True
    mod_grads: dict = dc_field(default_factory=dict)
    preprocess_cfg: PreprocessConfig = dc_field(default_factory=PreprocessConfig)
    builder: Builder | None = None
    scorer: Scorer | None = None
    gradients: dict[str, torch.Tensor] = dc_field(default_factory=dict)
    scores: list | torch.Tensor | None = None

    def __post_init__(self):
        if self.filter_modules is None:
            self.filter_modules = self.cfg.filter_modules
        super().__post_init__()

    def setup(self) -> None:
        assert isinstance(self.model.device, torch.device), "Model device is not set correctly"
        self.attribute_tokens = self.cfg.attribute_tokens
        if self.processor.projection_target == "global":
            assert self.skip_hessians, (
                "projection_target='global' sums all modules into a single key, so per-module "
                "autocorrelation statistics are undefined."
            )
        if self.cfg.attribute_tokens:
            assert self.preprocess_cfg.aggregation == "none", "attribute_tokens is incompatible with reduce mode."
        self.save_dtype = resolve_save_dtype(self.model, self.cfg)
        self.lo = torch.finfo(self.save_dtype).min
        self.hi = torch.finfo(self.save_dtype).max
        self.per_doc_losses = torch.zeros(len(self.data), device=self.model.device, dtype=torch.float32)
        self.gradients, self.scores = {}, None
        if self.builder is None and self.scorer is None:
            sizes = {n: math.prod(s) for n, s in self.shapes().items()}
            self.builder = Builder(self.data, sizes, self.save_dtype, self.preprocess_cfg,
                                   attribute_tokens=self.cfg.attribute_tokens)

    def teardown(self) -> None:
        if dist.is_initialized():
            dist.reduce(self.per_doc_losses, dst=0)
        sizes = {n: math.prod(s) for n, s in self.shapes().items()}
        if self.processor.hessians:
            process_autocorrelation_matrices(
                self.processor, self.processor.hessians, self.num_rows(self.data), sizes, self.rank
            )
        if self.builder is not None:
            self.builder.teardown()
            buf, off = self.builder.grad_buffer, 0
            for name, dim in sizes.items():
                self.gradients[name] = numpy_to_tensor(buf[:, off : off + dim])
                off += dim
        if self.scorer is not None:
            self.scores = self.scorer.writer.scores

    @HookCollectorBase.split_attention_heads
    def backward_hook(self, module: nn.Module, g: Tensor) -> None:
        name: str = module._name
        P = self._compute_gradient(module, g)
        if not self.skip_hessians:
            P = P.float()
            if name in self.processor.hessians:
                self.processor.hessians[name].addmm_(P.mT, P)
            else:
                self.processor.hessians[name] = P.mT @ P
        if self.accumulate_global_projection(name, P):
            return
        if self.scorer is not None or self.preprocess_cfg.aggregation != "none":
            self.mod_grads[name] = P.to(dtype=self.save_dtype)
        else:
            self.mod_grads[name] = P.to(device="cpu", dtype=self.save_dtype, non_blocking=True)

    def process_batch(self, indices: list[int], **kwargs) -> None:
        losses = kwargs.get("losses")
        assert losses is not None, "losses must be provided in kwargs"
        self.finalize_global_projection()
        if self.builder is not None:
            self.builder(indices, self.mod_grads)
        if self.scorer is not None:
            self.scorer(indices, self.mod_grads)
        self.mod_grads.clear()
        idx = torch.as_tensor(indices, device=self.per_doc_losses.device)
        self.per_doc_losses[idx] = losses.detach().to(self.per_doc_losses.dtype)
