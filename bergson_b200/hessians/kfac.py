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
fused SYRK kernel's peer-memory epilogue on CUDA ranks (``BERGSON_B200_DISABLE_PEER=1`` on every
rank selects library all-reduces instead; CPU ranks always use them).  On CUDA with 16-bit
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

    def with_batch(self, collection_mask: Tensor | None = None):
        """Row indices of collected / skipped positions are computed once per batch (one
        host synchronisation) and reused by every hook."""
        super().with_batch(collection_mask)
        if collection_mask is not None:
            flat = collection_mask.reshape(-1)
            self._keep_idx = flat.nonzero(as_tuple=True)[0]
            self._drop_idx = (~flat).nonzero(as_tuple=True)[0]
        return self

    def _masked(self, x: Tensor) -> Tensor:
        assert self._current_collection_mask is not None, "Collection mask not set."
        return x.reshape(-1, x.shape[-1]).index_select(0, self._keep_idx)

    def _acc(self, store: dict[str, Tensor], name: str, d: int, device) -> Tensor:
        if name not in store:
            store[name] = torch.zeros(d, d, device=device, dtype=torch.float32)
        return store[name]

    def _gram_into(self, acc: Tensor, x3d: Tensor, ones_column: bool = False) -> None:
        """``acc += X^T X`` over the collected positions of ``x3d [N, S, D]``.

        Fused path: the SYRK kernel reads *all* rows in place (no compaction copy) and the
        Gram of the few skipped rows (each sequence's last position, padding) is subtracted."""
        x2 = x3d.reshape(-1, x3d.shape[-1])
        n_drop = self._drop_idx.numel()
        if not ones_column and attribution.gram_fused_ok(x2) and n_drop * 8 <= x2.shape[0]:
            attribution.gram_accumulate(acc, x2)
            if n_drop:
                xd = x2.index_select(0, self._drop_idx).float()
                acc.addmm_(xd.mT, xd, alpha=-1.0)
            return
        xk = self._masked(x3d)
        if ones_column:
            xk = torch.cat([xk, xk.new_ones(xk.shape[0], 1)], dim=1)
        xf = xk.to(self.dtype if self.dtype != torch.bfloat16 else torch.float32)
        acc.add_((xf.mT @ xf).float())

    # -- hooks ----------------------------------------------------------------------------

    def forward_hook(self, module: nn.Module, a: Tensor) -> None:
        if self.method == "kfac":
            name = assert_type(str, module._name)
            d = a.shape[-1] + (1 if module._collect_bias else 0)
            self._gram_into(self._acc(self.A_full, name, d, a.device), a, ones_column=bool(module._collect_bias))
            return
        a_bi = self._masked(a)
        if module._collect_bias:
            a_bi = torch.cat([a_bi, a_bi.new_ones(a_bi.shape[0], 1)], dim=1)
        module._inputs = a_bi

    def backward_hook(self, module: nn.Module, g: Tensor) -> None:
        name = assert_type(str, module._name)
        S = self._acc(self.S_full, name, g.shape[-1], g.device)
        if self.method == "kfac":
            self._gram_into(S, g)
            return
        g_bo = self._masked(g)
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
        # The choice is made from facts that are equal on every rank (backend, device type, one
        # environment switch), never from a per-rank try/except: ranks that disagreed would
        # wait for each other in different collectives.  A failure on the peer path is fatal.
        if sc.dist and names and store[names[0]].is_cuda and os.environ.get("BERGSON_B200_DISABLE_PEER") != "1":
            return self._row_shards_peer(store, names)
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
            raise RuntimeError(
                "the K-FAC reduce-scatter runs over a symmetric peer-memory heap, which this process group does not "
                "offer (needs the NCCL backend on CUDA); set BERGSON_B200_DISABLE_PEER=1 on every rank to use "
                "library all-reduces instead")
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
        from ..collector.collector import check_kernel_status

        check_kernel_status(next(self.model.parameters()).device)
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
