"""A collector whose outputs stay in memory: the gradient rows (``.gradients``), scores
against a query set (``.scores``) and, on request, the autocorrelation Hessian of the rows.

It is a thin arrangement of three sinks that each receive every batch's blocks:

* a ``Builder`` without a path (rows gathered in a host array; created unless a builder or a
  scorer is passed in),
* a ``Scorer`` (its writer keeps the score matrix),
* a ``GramAccumulator`` when ``skip_hessians`` is False.

Nothing here touches the disk; ``teardown`` reduces the per-document losses to rank 0, finishes
the Gram statistics and exposes the per-module views of the row buffer.
"""

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
from ..data import column_offsets
from ..hessians.gram import GramAccumulator
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
        # the index configuration's module filter applies unless the caller gave one
        self.filter_modules = self.filter_modules if self.filter_modules is not None else self.cfg.filter_modules
        super().__post_init__()

    # ------------------------------------------------------------------ lifecycle

    def setup(self) -> None:
        if not isinstance(self.model.device, torch.device):
            raise AssertionError("Model device is not set correctly")
        cfg, pre = self.cfg, self.preprocess_cfg
        self.attribute_tokens = cfg.attribute_tokens
        if cfg.attribute_tokens and pre.aggregation != "none":
            raise AssertionError("attribute_tokens is incompatible with reduce mode.")
        wants_gram = not self.skip_hessians
        if wants_gram and self.processor.projection_target == "global":
            raise AssertionError("Autocorrelation statistics are per module; projection_target='global' keeps a "
                                 "single combined vector, so skip_hessians must stay True.")
        self.save_dtype = resolve_save_dtype(self.model, cfg)
        info = torch.finfo(self.save_dtype)
        self.lo, self.hi = info.min, info.max
        self.sizes = {name: math.prod(shape) for name, shape in self.shapes().items()}
        self.gram = GramAccumulator(self.sizes) if wants_gram else None
        self.per_doc_losses = torch.zeros(len(self.data), device=self.model.device, dtype=torch.float32)
        self.gradients, self.scores = {}, None
        if self.builder is None and self.scorer is None:
            self.builder = Builder(self.data, self.sizes, self.save_dtype, pre, attribute_tokens=cfg.attribute_tokens)
        # blocks stay on the device when something there consumes them (scorer, aggregate row)
        self._keep_on_device = self.scorer is not None or pre.aggregation != "none"

    def teardown(self) -> None:
        if dist.is_initialized():
            dist.reduce(self.per_doc_losses, dst=0)
        if self.gram is not None:
            self.gram.finish(self.processor, self.num_rows(self.data), self.rank)
        if self.builder is not None:
            self.builder.teardown()
            rows = self.builder.grad_buffer
            self.gradients = {name: numpy_to_tensor(rows[:, lo:hi]) for name, (lo, hi) in column_offsets(self.sizes).items()}
        if self.scorer is not None:
            self.scores = self.scorer.writer.scores

    # ------------------------------------------------------------------ per batch

    @HookCollectorBase.split_attention_heads
    def backward_hook(self, module: nn.Module, g: Tensor) -> None:
        name: str = module._name
        block = self._compute_gradient(module, g)
        if self.gram is not None:
            self.gram.add_blocks({name: block})
        if self.accumulate_global_projection(name, block):
            return
        if self._keep_on_device:
            self.mod_grads[name] = block.to(dtype=self.save_dtype)
        else:
            self.mod_grads[name] = block.to(device="cpu", dtype=self.save_dtype, non_blocking=True)

    def process_batch(self, indices: list[int], **kwargs) -> None:
        if (losses := kwargs.get("losses")) is None:
            raise AssertionError("losses must be provided in kwargs")
        self.finalize_global_projection()
        for sink in (self.builder, self.scorer):
            if sink is not None:
                sink(indices, self.mod_grads)
        self.mod_grads.clear()
        where = torch.as_tensor(indices, device=self.per_doc_losses.device)
        self.per_doc_losses[where] = losses.detach().to(self.per_doc_losses.dtype)
