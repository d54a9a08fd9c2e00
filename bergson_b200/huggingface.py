"""Gradient-store collection during HF ``Trainer`` training
(reference ``bergson/huggingface.py:31-430``).

``prepare_for_gradient_collection(trainer)`` threads each example's dataset index
(``_idx``) through the datasets and the collator; ``GradientCollectorCallback`` then
hooks the model for the whole run, writes every micro-step's per-example projected
gradients into ``<path>/train[/epoch_k]`` and, after each optimizer step, refreshes the
normalisers from the optimizer's second moments (optionally divided by ``lr^2`` so that
the stored row is the update the optimizer applied).
"""

from __future__ import annotations

import math
import os
from collections.abc import Sized
from functools import wraps
from itertools import chain
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist
from datasets import Dataset
from torch import Tensor

from .collector.gradient_collectors import StreamingGradientCollector
from .config import AttentionConfig
from .data import column_offsets, create_index
from .gradients import AdafactorNormalizer, AdamNormalizer, GradientProcessor, LayerAdapter
from .utils.utils import convert_dtype_to_torch

try:
    from transformers import TrainerCallback
except Exception:  # pragma: no cover - transformers is a soft dependency of this module

    class TrainerCallback:  # type: ignore[no-redef]
        pass


def _is_transposed(model, layer_name: str) -> bool:
    try:
        mod = model.get_submodule(layer_name)
    except AttributeError:
        return False
    return isinstance(mod, LayerAdapter.supported_modules) and LayerAdapter.weight_transposed(mod)


class GradientCollectorCallback(TrainerCallback):
    def __init__(self, path: Path, attention_cfgs: dict[str, AttentionConfig] | None = None, projection_dim: int = 16,
                 include_bias: bool = False, dtype: np.dtype = np.dtype(np.float16), accumulate_grads: bool = False,
                 use_optimizer_state: bool = True, scale_by_lr: bool = True, track_order: bool = False):
        """``accumulate_grads``: one store for all epochs (rows overwritten by the latest
        epoch) instead of ``train/epoch_k``; ``track_order``: save ``order.hf`` with
        ``(_idx, global_step, epoch)`` of every trained example."""
        super().__init__()
        self.path = Path(path)
        self.attention_cfgs = attention_cfgs or {}
        self.projection_dim, self.include_bias = projection_dim, include_bias
        self.dtype = np.dtype(dtype)
        self.torch_dtype = convert_dtype_to_torch(self.dtype)
        self.accumulate_grads = accumulate_grads
        self.use_optimizer_state, self.scale_by_lr = use_optimizer_state, scale_by_lr
        self.order: list[dict] | None = [] if track_order else None
        self.batch_indices: Tensor | None = None
        self.grad_sizes: dict[str, int] = {}
        self.collector: StreamingGradientCollector

    # -- store writes -----------------------------------------------------------------------

    def write_grads(self, grad_buffer: np.memmap):
        if not self.collector.mod_grads or self.batch_indices is None:
            return
        if torch.cuda.is_available():
            torch.cuda.synchronize()  # the blocks were copied to host asynchronously
        rows = self.batch_indices.numpy()
        for name, g in self.collector.mod_grads.items():
            lo, hi = self.grad_offsets[name]
            grad_buffer[rows, lo:hi] = g.to(self.torch_dtype).numpy()
        self.collector.mod_grads.clear()

    # -- Trainer events ---------------------------------------------------------------------

    def on_train_begin(self, args, state, control, *, model, **kwargs):
        if not hasattr(args, "__gradient_collection_enabled__"):
            raise RuntimeError("Gradient collection is not enabled. Call prepare_for_gradient_collection(trainer) first.")
        target_modules = None
        if type(model).__name__.startswith("Peft"):
            from .utils.peft import extract_peft_target_modules

            target_modules = extract_peft_target_modules(model)
        self.collector = StreamingGradientCollector(
            model=getattr(model, "base_model", model),
            processor=GradientProcessor({}, projection_dim=self.projection_dim or None, include_bias=self.include_bias),
            target_modules=target_modules, attention_cfgs=self.attention_cfgs, dtype=self.torch_dtype,
        )
        self.collector.save_dtype = self.torch_dtype
        self.collector.lo, self.collector.hi = torch.finfo(self.torch_dtype).min, torch.finfo(self.torch_dtype).max
        self.grad_sizes = {n: math.prod(s) for n, s in self.collector.shapes().items()}
        self.grad_offsets = column_offsets(self.grad_sizes)
        self.collector.__enter__()
        self.fwd_handle = model.register_forward_pre_hook(self.on_forward_begin, with_kwargs=True)

    def _epoch_dir(self, epoch: int) -> Path:
        return self.path / ("train" if self.accumulate_grads else f"train/epoch_{epoch}")

    def on_epoch_begin(self, args, state, control, *, train_dataloader, **kwargs):
        epoch = int(state.epoch or 0)
        if self.accumulate_grads and epoch > 0:
            return
        ds = train_dataloader.dataset
        if not isinstance(ds, Sized):
            raise ValueError("Dataset must be sized for gradient collection")
        self.train_grad_buffer = create_index(self._epoch_dir(epoch), num_grads=len(ds), grad_sizes=self.grad_sizes,
                                              dtype=self.dtype)

    def on_epoch_end(self, args, state, control, **kwargs):
        if (dist.get_rank() if dist.is_initialized() else 0) == 0:
            self.collector.processor.save(self._epoch_dir(int(state.epoch or 0) - 1))
        self.train_grad_buffer.flush()

    def on_forward_begin(self, module, args, kwargs: dict):
        idx = kwargs.pop("_idx", None)
        if module.training and idx is not None:
            self.batch_indices = idx.to("cpu", non_blocking=True)
        return args, kwargs

    def on_substep_end(self, args, state, control, **kwargs):
        self.write_grads(self.train_grad_buffer)

    def on_step_end(self, args, state, control, *, model=None, optimizer=None, **kwargs):
        self.on_substep_end(args, state, control)
        if self.order is not None:
            assert self.batch_indices is not None, "Batch indices are not available for training order tracking"
            epoch = int(state.epoch or 0)
            self.order.extend({"_idx": int(i), "global_step": state.global_step, "epoch": epoch}
                              for i in self.batch_indices.tolist())
        if self.use_optimizer_state and optimizer is not None and model is not None:
            self._refresh_normalizers(getattr(model, "base_model", model), optimizer)

    def _refresh_normalizers(self, model, optimizer) -> None:
        names = {p: n for n, p in model.named_parameters() if p.requires_grad}
        layers: dict[str, dict] = {}
        for group in optimizer.param_groups:
            for p in group["params"]:
                name = names.get(p)
                if name is None:
                    continue
                layer, _, kind = name.rpartition(".")
                if kind not in ("weight", "bias") or layer not in self.collector.target_info:
                    continue
                st = optimizer.state[p]
                rec = layers.setdefault(layer, {"lr": group["lr"]})
                if st.get("exp_avg_sq_row") is not None and kind == "weight":
                    rec["row"], rec["col"] = st["exp_avg_sq_row"], st.get("exp_avg_sq_col")
                elif st.get("exp_avg_sq") is not None:
                    rec[kind] = st["exp_avg_sq"]
        out = {}
        for layer, rec in layers.items():
            scale = rec["lr"] ** 2 if self.scale_by_lr else 1.0
            bias = rec["bias"] / scale if "bias" in rec and rec["bias"] is not None else None
            t = _is_transposed(model, layer)
            if "weight" in rec:
                w = rec["weight"].T.contiguous() if t else rec["weight"]
                out[layer] = AdamNormalizer(w / scale, bias)
            elif rec.get("row") is not None and rec.get("col") is not None:
                row, col = (rec["col"], rec["row"]) if t else (rec["row"], rec["col"])
                out[layer] = AdafactorNormalizer(row / scale, col / scale, bias)
        self.collector.processor.normalizers = out
        self.collector._fused_mats.clear()

    def on_train_end(self, args, state, control, **kwargs):
        self.collector.__exit__(None, None, None)
        self.fwd_handle.remove()
        if self.order is not None:
            self._save_order()

    def _save_order(self):
        os.makedirs(self.path, exist_ok=True)
        order = self.order or []
        if dist.is_initialized():
            gathered: list = [None] * dist.get_world_size()
            dist.all_gather_object(gathered, order)
            if dist.get_rank() != 0:
                return
            order = list(chain.from_iterable(o for o in gathered if o is not None))
        Dataset.from_list(order).save_to_disk(os.path.join(self.path, "order.hf"))


def prepare_for_gradient_collection(trainer):
    """Add an ``_idx`` column to the trainer's datasets, keep it through column pruning and
    collation, and mark the trainer as ready for ``GradientCollectorCallback``."""
    add_idx = lambda ex, idx: {"_idx": idx}  # noqa: E731
    trainer.train_dataset = trainer.train_dataset.map(add_idx, with_indices=True)
    if trainer.eval_dataset is not None:
        if isinstance(trainer.eval_dataset, dict):
            for k, d in trainer.eval_dataset.items():
                trainer.eval_dataset[k] = d.map(add_idx, with_indices=True)
        else:
            trainer.eval_dataset = trainer.eval_dataset.map(add_idx, with_indices=True)
    trainer._set_signature_columns_if_needed()
    trainer._signature_columns.append("_idx")
    if trainer.data_collator:
        inner = trainer.data_collator

        @wraps(inner)
        def collate(features):
            batch = inner(features)
            batch.setdefault("_idx", torch.tensor([f["_idx"] for f in features]))
            return batch

        trainer.data_collator = collate
    trainer.args.__gradient_collection_enabled__ = True
    return trainer
