"""Concrete collectors: store builder / scorer feed, query-time traces, streaming
(training callback) collection (reference ``bergson/collector/gradient_collectors.py``)."""

from __future__ import annotations

import math
from collections import defaultdict
from dataclasses import dataclass, field

import torch
import torch.distributed as dist
import torch.nn as nn
from datasets import Dataset, Value
from torch import Tensor

from ..builder import Builder
from ..config import IndexConfig, PreprocessConfig
from ..gradients import AdamNormalizer
from ..data import column_offsets
from ..score.scorer import Scorer
from ..utils.utils import convert_precision_to_torch, get_gradient_dtype
from .collector import HookCollectorBase


def resolve_save_dtype(model: nn.Module, cfg: IndexConfig | None) -> torch.dtype:
    """Row dtype: ``cfg.store_dtype`` if set, else the model's gradient dtype."""
    if cfg is not None and getattr(cfg, "store_dtype", "auto") != "auto":
        return convert_precision_to_torch(cfg.store_dtype)
    return get_gradient_dtype(model)


@dataclass(kw_only=True)
class GradientCollector(HookCollectorBase):
    """Per-example gradients -> gradient store (``Builder``) or on-the-fly ``Scorer``.

    With ``skip_index=True`` nothing is written and ``mod_grads`` holds the last
    batch's blocks for inspection."""

    data: Dataset
    cfg: IndexConfig
    mod_grads: dict = field(default_factory=dict)
    preprocess_cfg: PreprocessConfig = field(default_factory=PreprocessConfig)
    builder: Builder | None = None
    scorer: Scorer | None = None
    skip_index: bool = False

    def setup(self) -> None:
        assert isinstance(self.model.device, torch.device), "Model device is not set correctly"
        self.attribute_tokens = self.cfg.attribute_tokens
        if self.cfg.attribute_tokens:
            assert self.preprocess_cfg.aggregation == "none", "attribute_tokens is incompatible with reduce mode."
        from ..parallel import topology

        self._tp = topology.tp_size()
        self._tp_writer = topology.tp_rank() == 0
        if self._tp > 1:
            assert self.processor.projection_dim and self.processor.projection_target == "per_module", (
                "tensor parallelism needs per-module projection (the blocks are summed over the group)")
            assert not any(isinstance(n, AdamNormalizer) for n in self.processor.normalizers.values()), (
                "elementwise (Adam) normalisation does not commute with the sum over tensor-parallel shards")
        self.save_dtype = resolve_save_dtype(self.model, self.cfg)
        self.lo = torch.finfo(self.save_dtype).min
        self.hi = torch.finfo(self.save_dtype).max
        self.per_doc_losses = torch.zeros(len(self.data), device=self.model.device, dtype=torch.float32)
        self.save_index = self.scorer is None and not self.skip_index
        self.grad_sizes = {name: math.prod(s) for name, s in self.shapes().items()}
        if self.save_index:
            self.builder = Builder(
                self.data, self.grad_sizes, self.save_dtype, self.preprocess_cfg,
                attribute_tokens=self.cfg.attribute_tokens, path=self.cfg.partial_run_path,
            )
        else:
            self.builder = None
        # The fused kernels feed either the asynchronous store writer or the scorer.
        wants_fused = getattr(self.cfg, "fused_collection", True) and (
            (self.builder is not None and self.builder.supports_async_rows)
            or (self.scorer is not None and not self.scorer.attribute_tokens
                and getattr(self.scorer, "supports_rows", False))
        )
        if wants_fused and self.processor.projection_target == "per_module":
            spans = column_offsets(self.grad_sizes)
            total = sum(self.grad_sizes.values())
            # The scorer's modules may be a subset of the collected ones, in another order:
            # it assembles its query operand in this collector's column layout, or declines.
            if self.scorer is None or self.scorer.set_row_layout(spans, total):
                self.enable_fused({n: lo for n, (lo, _) in spans.items()}, total,
                                  token_rows=self.builder is not None and self._tp == 1)

    @HookCollectorBase.split_attention_heads
    def backward_hook(self, module: nn.Module, g: Tensor):
        if self.compute_gradient_fused(module, g):
            return
        name: str = module._name
        P = self._compute_gradient(module, g)
        if self.accumulate_global_projection(name, P):
            return
        if self._fused_enabled or self._tp > 1:
            self.mod_grads[name] = P  # merged / reduced in process_batch
        elif self.save_index and self.preprocess_cfg.aggregation == "none":
            self.mod_grads[name] = P.to(device="cpu", dtype=self.save_dtype, non_blocking=True)
        else:
            self.mod_grads[name] = P.to(dtype=self.save_dtype)

    def process_batch(self, indices: list[int], **kwargs):
        losses = kwargs.get("losses")
        assert losses is not None, "losses must be provided in kwargs"
        if self._tp > 1:
            self._reduce_over_tensor_parallel_group()
        if self._fused_enabled:
            rows = self.fused_rows()
            if self._tp > 1:
                dist.all_reduce(rows, group=self._tp_group())
            if self.builder is not None and self._tp_writer:
                self.builder.write_rows_async(indices, rows, self.lo, self.hi)
            if self.scorer is not None:
                self.scorer.writer(indices, self.scorer.score_rows(rows.clamp(self.lo, self.hi)),
                                   query_offset=self.scorer.query_offset)
        else:
            self.finalize_global_projection()
            if self.builder and self._tp_writer:
                self.builder(indices, self.mod_grads)
            if self.scorer:
                self.scorer(indices, self.mod_grads)
        self.mod_grads.clear()
        idx = torch.as_tensor(indices, device=self.per_doc_losses.device)
        self.per_doc_losses[idx] = losses.detach().to(self.per_doc_losses.dtype)

    def _tp_group(self):
        from ..parallel import topology

        return topology.tp_group()

    def _reduce_over_tensor_parallel_group(self) -> None:
        """Torch-path blocks are partial sums over the group's shards: add them up, then
        clamp / cast as the single-rank path does."""
        if self._fused_enabled:
            return  # the fused accumulator is reduced as a whole
        for name, P in self.mod_grads.items():
            P = P.float().contiguous()
            dist.all_reduce(P, group=self._tp_group())
            self.mod_grads[name] = P.clamp_(self.lo, self.hi).to(self.save_dtype)

    def teardown(self):
        if dist.is_initialized():
            if self._tp > 1:
                self.per_doc_losses /= self._tp  # every rank of a group holds the same losses
            dist.reduce(self.per_doc_losses, dst=0)
        if self.builder:
            self.builder.teardown()
        if self.rank != 0:
            return
        if self.preprocess_cfg.aggregation != "none" and self.builder is not None:
            self.data = Dataset.from_list([{"query_index": i} for i in range(self.builder.grad_buffer.shape[0])])
        else:
            if self.cfg.drop_columns and "input_ids" in self.data.column_names:
                self.data = self.data.remove_columns(["input_ids"])
            self.data = self.data.add_column(
                "loss", self.per_doc_losses.cpu().numpy(), feature=Value("float32"), new_fingerprint="loss"
            )
        self.data.save_to_disk(str(self.cfg.partial_run_path / "data.hf"))
        self.processor.save(self.cfg.partial_run_path)


@dataclass(kw_only=True)
class TraceCollector(HookCollectorBase):
    """Query-time collector: keeps every batch's blocks in per-module lists."""

    mod_grads: dict = field(default_factory=lambda: defaultdict(list))
    device: torch.device | str
    dtype: torch.dtype

    def setup(self) -> None:
        self.save_dtype = get_gradient_dtype(self.model)
        self.lo = torch.finfo(self.save_dtype).min
        self.hi = torch.finfo(self.save_dtype).max

    @HookCollectorBase.split_attention_heads
    def backward_hook(self, module: nn.Module, g: Tensor):
        P = self._compute_gradient(module, g)
        self.mod_grads[module._name].append(P.to(self.device, self.dtype, non_blocking=True))

    def process_batch(self, indices: list[int], **kwargs):
        return

    def teardown(self):
        return


@dataclass(kw_only=True)
class StreamingGradientCollector(HookCollectorBase):
    """Leaves each micro-step's blocks (on CPU, save dtype) in ``mod_grads`` for an
    external consumer such as the training callback."""

    mod_grads: dict = field(default_factory=dict)
    dtype: torch.dtype

    def setup(self) -> None:
        self.save_dtype = get_gradient_dtype(self.model)
        self.lo = torch.finfo(self.save_dtype).min
        self.hi = torch.finfo(self.save_dtype).max

    def teardown(self) -> None:
        pass

    def process_batch(self, indices: list[int], **kwargs) -> None:
        pass

    @HookCollectorBase.split_attention_heads
    def backward_hook(self, module: nn.Module, g: Tensor):
        P = self._compute_gradient(module, g)
        self.mod_grads[module._name] = P.to(device="cpu", dtype=self.save_dtype, non_blocking=True)
