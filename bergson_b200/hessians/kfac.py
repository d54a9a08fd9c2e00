"""Kronecker-factor collectors: K-FAC covariances, trace-weighted K-FAC (TKFAC) and
Shampoo second moments.

Per batch and module, with ``a`` the masked activations ``[T, I(+1)]`` and ``g`` the
masked output gradients ``[T, O]`` (reference ``bergson/hessians/{kfac,tkfac,shampoo}.py``):

* kfac:    ``A += a^T a``                      ``S += g^T g``
* tkfac:   ``A += tr(g^T g) a^T a``            ``S += tr(a^T a) g^T g``
* shampoo: ``M = g^T a``; ``A += M^T M``;  ``S += M M^T``;  ``A /= tr(A)`` at the end

The reference all-reduces every update and keeps its row slice.  Every update is a sum
over (rank, batch) units, so this implementation accumulates the full fp32 matrices
locally and performs one reduce-scatter to row shards in ``teardown`` — through the
fused SYRK kernel's peer-memory epilogue when a symmetric heap is available, else with
``torch.distributed.reduce_scatter``-equivalent collectives.  On CUDA with 16-bit
activations the K-FAC products run in the tcgen05 SYRK kernel, which reads the
activations once in their own dtype with fp32 accumulation.
"""

from __future__ import annotations

import os
from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn as nn
from safetensors.torch import save_file
from torch import Tensor

from ..collector.collector import HookCollectorBase
from ..ops import attribution
from ..utils.utils import assert_type
from .sharded_computation import ShardedMul


@dataclass(kw_only=True)
class _FactorCollector(HookCollectorBase):
    dtype: torch.dtype
    path: str
    method: str = "kfac"

    def setup(self) -> None:
        self.shard_computer = ShardedMul()
        self.A_full: dict[str, Tensor] = {}
        self.S_full: dict[str, Tensor] = {}

    # -- helpers --------------------------------------------------------------------------

    def _masked(self, x: Tensor) -> Tensor:
        mask = self._current_collection_mask
        assert mask is not None, "Collection mask not set."
        return x[mask]

    def _acc(self, store: dict[str, Tensor], name: str, d: int, device) -> Tensor:
        if name not in store:
            store[name] = torch.zeros(d, d, device=device, dtype=torch.float32)
        return store[name]

    def _gram_into(self, acc: Tensor, x: Tensor, full: Tensor | None = None, scale: float | Tensor | None = None):
        """``acc += scale * x^T x`` for masked rows ``x``.  When the unmasked tensor
        ``full`` is given and the fused kernel applies, the Gram of all rows is taken in
        place and the few masked-out rows are subtracted."""
        if scale is None and attribution.gram_fused_ok(x):
            attribution.gram_accumulate(acc, x)
            return
        xf = x.to(self.dtype if self.dtype != torch.bfloat16 else torch.float32)
        upd = (xf.mT @ xf).float()
        acc.add_(upd if scale is None else upd * scale)

    # -- hooks ----------------------------------------------------------------------------

    def forward_hook(self, module: nn.Module, a: Tensor) -> None:
        a_bi = self._masked(a)
        if module._collect_bias:
            a_bi = torch.cat([a_bi, a_bi.new_ones(a_bi.shape[0], 1)], dim=1)
        if self.method == "kfac":
            name = assert_type(str, module._name)
            self._gram_into(self._acc(self.A_full, name, a_bi.shape[1], a.device), a_bi)
        else:
            module._inputs = a_bi

    def backward_hook(self, module: nn.Module, g: Tensor) -> None:
        name = assert_type(str, module._name)
        g_bo = self._masked(g)
        S = self._acc(self.S_full, name, g_bo.shape[1], g.device)
        if self.method == "kfac":
            self._gram_into(S, g_bo)
            return
        a_bi = module._inputs
        A = self._acc(self.A_full, name, a_bi.shape[1], g.device)
        wd = self.dtype if self.dtype != torch.bfloat16 else torch.float32
        if self.method == "tkfac":
            gg = (g_bo.to(wd).mT @ g_bo.to(wd)).float()
            aa = (a_bi.to(wd).mT @ a_bi.to(wd)).float()
            S.add_(gg * aa.diagonal().sum())
            A.add_(aa * gg.diagonal().sum())
        elif self.method == "shampoo":
            M = (g_bo.to(wd).mT @ a_bi.to(wd)).float()  # [O, I]
            A.add_(M.mT @ M)
            S.add_(M @ M.mT)
        else:
            raise ValueError(self.method)

    def process_batch(self, indices: list[int], **kwargs) -> None:
        pass

    # -- flush ----------------------------------------------------------------------------

    def _row_shards(self, store: dict[str, Tensor]) -> dict[str, Tensor]:
        """Sum over ranks and keep this rank's rows.  On NVLink-connected GPUs the reduction
        is done by the covariance kernel's epilogue pushing rows into their owners' peer
        memory; otherwise (CPU, single rank, no symmetric memory) by NCCL / Gloo."""
        sc = self.shard_computer
        names = [n for n in self.target_info if n in store]
        if sc.dist and names and store[names[0]].is_cuda:
            try:
                return self._row_shards_peer(store, names)
            except Exception as e:  # noqa: BLE001 - fall back to the library collective
                self.logger.warning(f"peer-memory reduce-scatter unavailable ({e}); using all_reduce")
        out = {}
        for name in names:
            full = store[name]
            if sc.dist:
                dist.all_reduce(full, op=dist.ReduceOp.SUM)
            lo, hi = sc.shard_bounds(full.shape[0])
            out[name] = full[lo:hi].to(self.dtype).contiguous()
        return out

    def _row_shards_peer(self, store: dict[str, Tensor], names: list[str]) -> dict[str, Tensor]:
        from ..parallel.peer import PeerHeap, symmetric_memory_available
        from ..ops import native
        from .sharded_computation import shard_bounds

        if not symmetric_memory_available():
            raise RuntimeError("symmetric memory not available")
        world, rank = self.shard_computer.world_size, self.shard_computer.rank
        # Same offsets on every rank: regions are sized for the largest (rank 0) shard.
        offsets, total = {}, 0
        for n in names:
            d = store[n].shape[0]
            offsets[n] = total
            total += (shard_bounds(d, 0, world)[1]) * d
        heap = PeerHeap(total, torch.float32)
        heap.local.zero_()
        heap.barrier()
        dummy: dict[int, Tensor] = {}
        for n in names:
            full = store[n].contiguous()
            d = full.shape[0]
            bounds = [shard_bounds(d, r, world) for r in range(world)]
            x = dummy.setdefault(d, torch.zeros(64, d, device=full.device, dtype=torch.bfloat16))
            native.cov_syrk(x, [heap.ptr(r, offsets[n]) for r in range(world)], [b[0] for b in bounds] + [d], full,
                            True, 0)
        heap.barrier()
        out = {}
        for n in names:
            d = store[n].shape[0]
            lo, hi = shard_bounds(d, rank, world)
            out[n] = heap.local[offsets[n] : offsets[n] + (hi - lo) * d].view(hi - lo, d).to(self.dtype).clone()
        heap.barrier()
        return out

    def teardown(self) -> None:
        attribution.gram_finalize(self.A_full)
        attribution.gram_finalize(self.S_full)
        A = self._row_shards(self.A_full)
        S = self._row_shards(self.S_full)
        if self.method == "shampoo":
            sc = self.shard_computer
            for name, shard in A.items():
                lo, _ = sc.shard_bounds(shard.shape[1])
                rows = torch.arange(shard.shape[0], device=shard.device)
                tr = shard[rows, rows + lo].sum()
                if sc.dist:
                    dist.all_reduce(tr, op=dist.ReduceOp.SUM)
                shard.div_(tr)
        a_dir = os.path.join(self.path, "activation_sharded")
        g_dir = os.path.join(self.path, "gradient_sharded")
        os.makedirs(a_dir, exist_ok=True)
        os.makedirs(g_dir, exist_ok=True)
        self.logger.info(f"Saving sharded covariance matrices to {a_dir} and {g_dir}")
        save_file({k: v.cpu() for k, v in A.items()}, os.path.join(a_dir, f"shard_{self.rank}.safetensors"))
        save_file({k: v.cpu() for k, v in S.items()}, os.path.join(g_dir, f"shard_{self.rank}.safetensors"))


@dataclass(kw_only=True)
class CovarianceCollector(_FactorCollector):
    """K-FAC: ``A = sum a^T a``, ``S = sum g^T g`` over collected positions."""

    method: str = "kfac"
