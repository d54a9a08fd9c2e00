"""Autocorrelation Hessians whose modules are owned by different ranks.

Every rank computes per-example gradient blocks for all modules of its own batch; the
block of module ``m`` is sent to the rank that owns ``m``'s Gram matrix, which adds
``P^T P``.  This lets the set of ``[d, d]`` Grams exceed one device's memory
(reference ``bergson/collector/dist_autocorrelation_gradient_collector.py``).

The exchange is one ``all_to_all_single`` of the flattened fp32 blocks per batch.  Batch
sizes may differ between ranks, so a first small all-to-all carries the element counts.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.distributed as dist
import torch.nn as nn
from datasets import Dataset, Value
from torch import Tensor

from ..config import IndexConfig
from ..process_autocorrelation import process_autocorrelation_matrices
from ..utils.utils import get_gradient_dtype
from .collector import HookCollectorBase


def assign_modules(names: list[str], world: int) -> dict[str, int]:
    """Contiguous blocks of modules per rank; the first ``len % world`` ranks get one more."""
    base, rem = divmod(len(names), world)
    out, i = {}, 0
    for r in range(world):
        n = base + (1 if r < rem else 0)
        for name in names[i : i + n]:
            out[name] = r
        i += n
    return out


def _add_gram(hessians: dict[str, Tensor], name: str, g: Tensor) -> None:
    g = g.float()
    if name in hessians:
        hessians[name].addmm_(g.mT, g)
    else:
        hessians[name] = g.mT @ g


def exchange_hessian_gradients(mod_grads: dict[str, Tensor], hessians: dict[str, Tensor],
                               module_to_rank: dict[str, int], owned_modules: set[str], rank: int) -> None:
    """Accumulate ``P^T P`` of this batch on the owning ranks."""
    for name, g in mod_grads.items():
        if name in owned_modules:
            _add_gram(hessians, name, g)
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return
    world = dist.get_world_size()
    names = list(mod_grads)
    device = next(iter(mod_grads.values())).device
    width = {n: mod_grads[n].shape[-1] for n in names}
    empty = torch.empty(0, device=device, dtype=torch.float32)
    send = [empty if dest == rank else
            torch.cat([mod_grads[n].flatten().float() for n in names if module_to_rank[n] == dest] or [empty])
            for dest in range(world)]
    send_sizes = torch.tensor([t.numel() for t in send], device=device, dtype=torch.int64)
    recv_sizes = torch.empty_like(send_sizes)
    dist.all_to_all_single(recv_sizes, send_sizes)
    recv_list = recv_sizes.tolist()
    recv = torch.empty(sum(recv_list), device=device, dtype=torch.float32)
    dist.all_to_all_single(recv, torch.cat(send), output_split_sizes=recv_list, input_split_sizes=send_sizes.tolist())
    mine = [n for n in names if module_to_rank[n] == rank]
    total_width = sum(width[n] for n in mine)
    off = 0
    for src, size in enumerate(recv_list):
        part = recv[off : off + size]
        off += size
        if size == 0 or src == rank or total_width == 0:
            continue
        rows = size // total_width  # the sender's batch size
        p = 0
        for n in mine:
            cnt = rows * width[n]
            _add_gram(hessians, n, part[p : p + cnt].view(rows, width[n]))
            p += cnt


@dataclass(kw_only=True)
class GradientCollectorWithDistributedAutocorrelationMatrices(HookCollectorBase):
    data: Dataset
    cfg: IndexConfig
    skip_hessians: bool = False
    mod_grads: dict = field(default_factory=dict)

    def setup(self) -> None:
        assert not self.skip_hessians, "this collector always estimates autocorrelation Hessians"
        self.attribute_tokens = self.cfg.attribute_tokens
        self.save_dtype = get_gradient_dtype(self.model)
        self.lo, self.hi = torch.finfo(self.save_dtype).min, torch.finfo(self.save_dtype).max
        self.per_doc_losses = torch.zeros(len(self.data), device=self.model.device, dtype=torch.float32)
        names = list(self.shapes())
        world = dist.get_world_size() if dist.is_initialized() else 1
        assert len(names) >= world, "Each rank must own at least one module"
        self.module_to_rank = assign_modules(names, world)
        self.owned_modules = {n for n, r in self.module_to_rank.items() if r == self.rank}

    @HookCollectorBase.split_attention_heads
    def backward_hook(self, module: nn.Module, g: Tensor):
        self.mod_grads[module._name] = self._compute_gradient(module, g)

    def process_batch(self, indices: list[int], **kwargs):
        losses = kwargs.get("losses")
        assert losses is not None, "losses must be provided in kwargs"
        exchange_hessian_gradients(self.mod_grads, self.processor.hessians, self.module_to_rank, self.owned_modules,
                                   self.rank)
        self.mod_grads.clear()
        idx = torch.as_tensor(indices, device=self.per_doc_losses.device)
        self.per_doc_losses[idx] = losses.detach().to(self.per_doc_losses.dtype)

    def teardown(self):
        if dist.is_initialized():
            dist.reduce(self.per_doc_losses, dst=0)
        sizes = {n: math.prod(s) for n, s in self.shapes().items()}
        if self.processor.hessians:
            process_autocorrelation_matrices(self.processor, self.processor.hessians, self.num_rows(self.data), sizes,
                                             self.rank)
        if self.rank == 0:
            data = self.data
            if self.cfg.drop_columns and "input_ids" in data.column_names:
                data = data.remove_columns(["input_ids"])
            data = data.add_column("loss", self.per_doc_losses.cpu().numpy(), feature=Value("float32"),
                                   new_fingerprint="loss")
            data.save_to_disk(str(self.cfg.partial_run_path / "data.hf"))
            self.processor.save(self.cfg.partial_run_path)
