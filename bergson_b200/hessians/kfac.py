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
from torch import Tensor

from ..collector.collector import HookCollectorBase
from ..ops import attribution
from ..utils.streamed_safetensors import save_tensors
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
        self._final_batch = False
        self._flushed: set[tuple[str, str]] = set()
        self._flushed_in_gemm: set[tuple[str, str]] = set()
        self._peer = self._make_peer_regions() if self._peer_wanted() else None

    # -- peer-memory reduce-scatter ---------------------------------------------------------

    def _peer_wanted(self) -> bool:
        """Decided from facts that are the same on every rank (process group, device type, one
        environment switch) so that all ranks take the same branch; failures later are fatal."""
        sc = self.shard_computer
        dev = next(self.model.parameters()).device
        if not sc.dist or dev.type != "cuda" or os.environ.get("BERGSON_B200_DISABLE_PEER") == "1":
            return False
        from ..parallel.peer import symmetric_memory_available

        if not symmetric_memory_available():
            raise RuntimeError(
                "the K-FAC reduce-scatter runs over a symmetric peer-memory heap, which this process group does not "
                "offer (needs the NCCL backend on CUDA); set BERGSON_B200_DISABLE_PEER=1 on every rank to use "
                "library all-reduces instead")
        return True

    def _make_peer_regions(self):
        """One heap region per factor, sized for the largest (rank 0) row shard; zeroed, and a
        barrier passed, before any rank can add into it."""
        from ..parallel.peer import PeerHeap
        from .sharded_computation import shard_bounds

        world = self.shard_computer.world_size
        regions, total = {}, 0
        for name, (_, (o, i), bias) in self.target_info.items():
            for kind, d in (("A", i + (1 if bias else 0)), ("S", o)):
                regions[(kind, name)] = (total, d)
                total += shard_bounds(d, 0, world)[1] * d
        heap = PeerHeap(total, torch.float32)
        heap.local.zero_()
        heap.barrier()
        return heap, regions

    def on_batch_start(self, step: int, num_steps: int) -> None:
        self._final_batch = step == num_steps - 1

    def _push(self, key: tuple[str, str], x: Tensor | None, local: Tensor, local_upper: bool) -> None:
        """Add ``local`` (+ ``x^T x``) into the row owners' heap regions from inside the SYRK
        kernel (P2P ``red.global.add`` from the epilogue): GEMM -> reduce-scatter in one launch."""
        from ..ops import native
        from .sharded_computation import shard_bounds

        heap, regions = self._peer
        off, d = regions[key]
        world = self.shard_computer.world_size
        bounds = [shard_bounds(d, r, world) for r in range(world)]
        if x is None:
            x, rows = torch.zeros(64, d, device=local.device, dtype=torch.bfloat16), 0
        else:
            rows = -1
        native.cov_syrk(x, [heap.ptr(r, off) for r in range(world)], [b[0] for b in bounds] + [d], local, True, rows,
                        local_upper)
        self._flushed.add(key)

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

    def _gram_into(self, acc: Tensor, x3d: Tensor, ones_column: bool = False, key: tuple[str, str] | None = None) -> None:
        """``acc += X^T X`` over the collected positions of ``x3d [N, S, D]``.

        Fused path: the SYRK kernel reads *all* rows in place (no compaction copy) and the
        Gram of the few skipped rows (each sequence's last position, padding) is subtracted.
        On the run's last batch, with a peer heap, the same launch also folds in everything
        accumulated so far and adds the sum straight into the row owners' shards."""
        x2 = x3d.reshape(-1, x3d.shape[-1])
        n_drop = self._drop_idx.numel()
        if not ones_column and attribution.gram_fused_ok(x2) and n_drop * 8 <= x2.shape[0]:
            flush = self._peer is not None and self._final_batch and key is not None and key not in self._flushed
            if n_drop:
                xd = x2.index_select(0, self._drop_idx).float()
                acc.addmm_(xd.mT, xd, alpha=-1.0)
            if flush:
                self._push(key, x2.contiguous(), acc, local_upper=True)
                self._flushed_in_gemm.add(key)
            else:
                attribution.gram_accumulate(acc, x2)
            return
        xk = self._masked(x3d)
        if ones_column:
            xk = torch.cat([xk, xk.new_ones(xk.shape[0], 1)], dim=1)
        xf = xk.to(self.dtype if self.dtype != torch.bfloat16 else torch.float32)
        acc.add_((xf.mT @ xf).float())

    def _gram(self, x2: Tensor) -> Tensor:
        """``x2^T x2`` (fp32, full matrix) of already-compacted rows: SYRK kernel when the rows
        are 16-bit on CUDA, else a torch product in the working dtype."""
        d = x2.shape[1]
        if attribution.gram_fused_ok(x2):
            out = {"g": torch.zeros(d, d, device=x2.device, dtype=torch.float32)}
            attribution.gram_accumulate(out["g"], x2)
            attribution.gram_finalize(out)
            return out["g"]
        wd = self.dtype if self.dtype != torch.bfloat16 else torch.float32
        return (x2.to(wd).mT @ x2.to(wd)).float()

    # -- hooks ----------------------------------------------------------------------------

    def forward_hook(self, module: nn.Module, a: Tensor) -> None:
        if self.method == "kfac":
            name = assert_type(str, module._name)
            d = a.shape[-1] + (1 if module._collect_bias else 0)
            self._gram_into(self._acc(self.A_full, name, d, a.device), a, ones_column=bool(module._collect_bias),
                            key=("A", name))
            return
        a_bi = self._masked(a)
        if module._collect_bias:
            a_bi = torch.cat([a_bi, a_bi.new_ones(a_bi.shape[0], 1)], dim=1)
        module._inputs = a_bi

    def backward_hook(self, module: nn.Module, g: Tensor) -> None:
        name = assert_type(str, module._name)
        S = self._acc(self.S_full, name, g.shape[-1], g.device)
        if self.method == "kfac":
            self._gram_into(S, g, key=("S", name))
            return
        g_bo = self._masked(g)
        a_bi = module._inputs
        A = self._acc(self.A_full, name, a_bi.shape[1], g.device)
        wd = self.dtype if self.dtype != torch.bfloat16 else torch.float32
        if self.method == "tkfac":
            gg, aa = self._gram(g_bo), self._gram(a_bi)
            S.add_(gg * aa.diagonal().sum())
            A.add_(aa * gg.diagonal().sum())
        elif self.method == "shampoo":
            M = self._cross(g_bo, a_bi, wd)  # [O, I]
            A.add_(M.mT @ M)
            S.add_(M @ M.mT)
        else:
            raise ValueError(self.method)

    def _cross(self, g_bo: Tensor, a_bi: Tensor, wd) -> Tensor:
        """``g^T a`` ([O, I], fp32): both operands read along the tokens by the tcgen05 GEMM
        (MN-major) when they are 16-bit on CUDA."""
        from ..ops.functional import use_fused

        if (g_bo.dtype in (torch.bfloat16, torch.float16) and g_bo.dtype == a_bi.dtype and use_fused(g_bo, a_bi)
                and g_bo.shape[1] % 8 == 0 and a_bi.shape[1] % 8 == 0 and g_bo.shape[0] > 0):
            from ..ops import native

            return native.gemm(g_bo.contiguous(), a_bi.contiguous(), True, True, None, True)[0]
        return (g_bo.to(wd).mT @ a_bi.to(wd)).float()

    def process_batch(self, indices: list[int], **kwargs) -> None:
        pass

    # -- flush ----------------------------------------------------------------------------

    def _row_shards(self, store: dict[str, Tensor], kind: str) -> dict[str, Tensor]:
        """Sum over ranks and keep this rank's rows.  With a peer heap every factor reaches its
        owners through the SYRK kernel's epilogue: during the last batch for the factors that
        saw one (GEMM -> reduce-scatter), here for the rest (a pure push of the accumulator).
        Without one (CPU, single rank, opt-out) the sum is a library all-reduce."""
        sc = self.shard_computer
        names = [n for n in self.target_info if n in store]
        if self._peer is None:
            out = {}
            for name in names:
                full = store[name]
                if sc.dist:
                    dist.all_reduce(full, op=dist.ReduceOp.SUM)
                lo, hi = sc.shard_bounds(full.shape[0])
                out[name] = full[lo:hi].to(self.dtype).contiguous()
            return out
        for name in names:
            if (kind, name) not in self._flushed:
                self._push((kind, name), None, store[name].contiguous(), local_upper=False)
        return {}

    def _read_peer_shards(self, kind: str, names: list[str]) -> dict[str, Tensor]:
        from .sharded_computation import shard_bounds

        heap, regions = self._peer
        out = {}
        for n in names:
            off, d = regions[(kind, n)]
            lo, hi = shard_bounds(d, self.shard_computer.rank, self.shard_computer.world_size)
            out[n] = heap.local[off : off + (hi - lo) * d].view(hi - lo, d).to(self.dtype).clone()
        return out

    def teardown(self) -> None:
        from ..collector.collector import check_kernel_status

        check_kernel_status(next(self.model.parameters()).device)
        # Accumulators that were flushed from inside the last batch's SYRK launch are complete
        # in the owners' heap regions; the others are mirrored and reduced now.
        pending_a = {n: m for n, m in self.A_full.items() if ("A", n) not in self._flushed}
        pending_s = {n: m for n, m in self.S_full.items() if ("S", n) not in self._flushed}
        attribution.gram_finalize(pending_a)
        attribution.gram_finalize(pending_s)
        self.A_full.update(pending_a)
        self.S_full.update(pending_s)
        A = self._row_shards(self.A_full, "A")
        S = self._row_shards(self.S_full, "S")
        if self._peer is not None:
            heap = self._peer[0]
            heap.barrier()  # every rank's adds have landed
            n_fused = len(self._flushed_in_gemm)
            self.logger.info(f"factors reduced through peer memory: {n_fused} inside the last batch's SYRK launches, "
                             f"{len(self._flushed) - n_fused} pushed at teardown")
            A = self._read_peer_shards("A", [n for n in self.target_info if n in self.A_full])
            S = self._read_peer_shards("S", [n for n in self.target_info if n in self.S_full])
            heap.barrier()  # all ranks have read their shards before the heap is released
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
        # Written straight from the device, tensor by tensor, through pinned staging buffers.
        save_tensors({k: v.contiguous() for k, v in A.items()}, os.path.join(a_dir, f"shard_{self.rank}.safetensors"))
        save_tensors({k: v.contiguous() for k, v in S.items()}, os.path.join(g_dir, f"shard_{self.rank}.safetensors"))


@dataclass(kw_only=True)
class CovarianceCollector(_FactorCollector):
    """K-FAC: ``A = sum a^T a``, ``S = sum g^T g`` over collected positions."""

    method: str = "kfac"
