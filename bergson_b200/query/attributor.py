"""Store-resident querying (reference ``bergson/query/attributor.py:47-282``).

The whole store lives on the device as one ``[N, D]`` matrix (modules concatenated in
store order).  ``search`` is a chunked ``queries @ store^T`` on the tcgen05 TN GEMM with
a running top-k merge, so the ``[Q, N]`` score matrix is never materialised.  Cosine
scoring keeps the raw rows and multiplies score columns by the rows' inverse norms.
"""

from __future__ import annotations

import json
from contextlib import contextmanager
from pathlib import Path
from typing import Generator, Literal

import numpy as np
import torch
from torch import Tensor, nn

from ..collector.gradient_collectors import TraceCollector
from ..config import FaissConfig, InversionConfig
from ..data import column_offsets, load_gradients
from ..gradients import GradientProcessor
from ..hessians.preconditioner import DensePreconditioner, FactoredPreconditioner, load_preconditioner
from ..ops import attribution
from ..utils.utils import numpy_to_tensor


class TraceResult:
    """Filled in when the ``Attributor.trace`` context exits."""

    def __init__(self):
        self._indices: Tensor | None = None
        self._scores: Tensor | None = None

    @property
    def indices(self) -> Tensor:
        if self._indices is None:
            raise ValueError("No indices available. Exit the context manager first.")
        return self._indices

    @property
    def scores(self) -> Tensor:
        if self._scores is None:
            raise ValueError("No scores available. Exit the context manager first.")
        return self._scores


def merge_topk_across_ranks(scores: Tensor, indices: Tensor, k: int, *, largest: bool = True, group=None):
    """Every rank contributes its local top-k (``[Q, k_r]`` scores and *global* row indices,
    ``k_r`` may differ between ranks); all ranks receive the top-``k`` of the union.  Ties are
    resolved by rank order, then by the local order, so the result is the same on every rank."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    q = scores.shape[0]
    fill = float("-inf") if largest else float("inf")
    pad_s = scores.new_full((q, k), fill, dtype=torch.float32)
    pad_i = indices.new_full((q, k), -1)
    pad_s[:, : scores.shape[1]] = scores[:, :k].float()
    pad_i[:, : indices.shape[1]] = indices[:, :k]
    all_s = [torch.empty_like(pad_s) for _ in range(world)]
    all_i = [torch.empty_like(pad_i) for _ in range(world)]
    dist.all_gather(all_s, pad_s.contiguous(), group=group)
    dist.all_gather(all_i, pad_i.contiguous(), group=group)
    cat_s, cat_i = torch.cat(all_s, dim=1), torch.cat(all_i, dim=1)
    valid = int((cat_i[0] >= 0).sum())
    top_s, sel = torch.topk(cat_s, min(k, valid), dim=1, largest=largest)
    return top_s.to(scores.dtype), cat_i.gather(1, sel)


class Attributor:
    precondition: Literal["one-sided", "two-sided", "none"]

    def __init__(self, index_path, device: str = "cpu", dtype: torch.dtype = torch.float32, unit_norm: bool = False,
                 faiss_cfg: FaissConfig | None = None, inversion_cfg: InversionConfig | None = None,
                 hessian_path=None, ev_correction: bool = False, sharded: bool = False, group=None):
        """``sharded=True`` (needs an initialised process group): every rank keeps a contiguous
        slice of the store's rows resident; ``search`` runs on the slice and the per-rank top-k
        lists are merged across ranks, so every rank returns the global result."""
        self.device, self.dtype, self.unit_norm = device, dtype, unit_norm
        self.sharded = sharded
        self.group = group
        self.row_lo = 0
        if sharded:
            import torch.distributed as dist

            if not dist.is_initialized():
                raise RuntimeError("Attributor(sharded=True) needs torch.distributed to be initialised")
            if faiss_cfg:
                raise NotImplementedError("a sharded store uses exact search; omit faiss_cfg")
            self.shard_rank, self.shard_world = dist.get_rank(group), dist.get_world_size(group)
        self.inversion_cfg = inversion_cfg or InversionConfig()
        self.faiss_index = None
        index_path = Path(index_path)
        self.processor = GradientProcessor.load(index_path, map_location=device)
        if hessian_path is None:
            self.precondition, self.preconditioner = "none", None
        else:
            # cosine scoring applies H^-1/2 to both sides, inner-product scoring H^-1 to the query
            self.precondition = "two-sided" if unit_norm else "one-sided"
            self.preconditioner = load_preconditioner(
                hessian_path, inversion_cfg=self.inversion_cfg, power=-0.5 if unit_norm else -1.0,
                ev_correction=ev_correction, device=device,
            )
        with (index_path / "info.json").open() as f:
            grad_sizes = json.load(f)["grad_sizes"]
        self.ordered_modules = list(grad_sizes)
        self.offsets = column_offsets(grad_sizes)

        if faiss_cfg:
            from .faiss_index import FaissIndex

            if isinstance(self.preconditioner, FactoredPreconditioner):
                raise NotImplementedError("FAISS preconditioning is not supported for factored (EKFAC) Hessians; "
                                          "omit faiss or use the dense path.")
            h_inv = self.preconditioner.h_inv if isinstance(self.preconditioner, DensePreconditioner) else {}
            name = (f"faiss_{faiss_cfg.index_factory.replace(',', '_')}{'_cosine' if unit_norm else ''}"
                    f"{'_precondition' if self.precondition != 'none' else ''}")
            fpath = index_path / name
            if not (fpath / "config.yaml").exists():
                FaissIndex.create_index(index_path, fpath, faiss_cfg, device, unit_norm, h_inv)
            self.faiss_index = FaissIndex(fpath, device, mmap_index=faiss_cfg.mmap_index)
            self.N = self.faiss_index.ntotal
            self.ordered_modules = self.faiss_index.ordered_modules
            return

        mm = load_gradients(index_path)
        self.N = len(mm)
        if sharded:
            from ..hessians.sharded_computation import shard_bounds

            self.row_lo, hi = shard_bounds(self.N, self.shard_rank, self.shard_world)
            mm = mm[self.row_lo : hi]
        self.store = numpy_to_tensor(np.ascontiguousarray(mm)).to(device=device, dtype=dtype)
        self.inv_norms: Tensor | None = None
        if unit_norm:
            if self.preconditioner is not None:
                blocks = self.preconditioner.apply({n: self.store[:, lo:hi] for n, (lo, hi) in self.offsets.items()})
                self.store = torch.cat([blocks[n].to(dtype) for n in self.ordered_modules], dim=1).contiguous()
            norms = self.store.float().pow(2).sum(1).sqrt()
            inv = 1.0 / norms
            bad = ~torch.isfinite(inv)
            if bad.any():
                print("Warning: zero-norm rows in the index; their cosine scores are set to 0")
            self.inv_norms = torch.where(bad, torch.zeros_like(inv), inv)

    @classmethod
    def from_rows(cls, rows: Tensor, grad_sizes: dict[str, int], *, unit_norm: bool = False, sharded: bool = False,
                  row_offset: int = 0, total_rows: int | None = None, group=None,
                  processor: GradientProcessor | None = None) -> "Attributor":
        """An attributor over rows that are already on a device (``[n, sum(grad_sizes)]``, module
        blocks in ``grad_sizes`` order), without a store on disk.  With ``sharded`` the tensor is
        this rank's slice ``[row_offset, row_offset + n)`` of a store of ``total_rows`` rows."""
        self = cls.__new__(cls)
        self.device, self.dtype, self.unit_norm = str(rows.device), rows.dtype, unit_norm
        self.sharded, self.group, self.row_lo = sharded, group, row_offset
        self.inversion_cfg = InversionConfig()
        self.faiss_index = None
        self.processor = processor or GradientProcessor()
        self.precondition, self.preconditioner = "none", None
        self.ordered_modules = list(grad_sizes)
        self.offsets = column_offsets(grad_sizes)
        self.store = rows.contiguous()
        self.N = total_rows if total_rows is not None else rows.shape[0]
        self.inv_norms = None
        if sharded:
            import torch.distributed as dist

            self.shard_rank, self.shard_world = dist.get_rank(group), dist.get_world_size(group)
        if unit_norm:
            from ..ops.functional import use_fused

            if use_fused(self.store):
                from ..ops import native

                sq = torch.zeros(self.store.shape[0], device=self.store.device, dtype=torch.float32)
                native.row_sumsq(self.store, sq)
            else:
                sq = self.store.float().pow(2).sum(1)
            inv = sq.rsqrt()
            self.inv_norms = torch.where(torch.isfinite(inv), inv, torch.zeros_like(inv))
        return self

    @property
    def grads(self) -> dict[str, Tensor]:
        """Per-module views of the resident store (unit-normalised rows under ``unit_norm``)."""
        out = {n: self.store[:, lo:hi] for n, (lo, hi) in self.offsets.items()}
        if self.inv_norms is not None:
            out = {n: g * self.inv_norms[:, None].to(g.dtype) for n, g in out.items()}
        return out

    def search(self, queries: dict[str, Tensor], k: int | None, modules: set[str] | None = None, reverse: bool = False):
        """Top-``k`` (lowest if ``reverse``) rows for each query: ``(scores, indices)``,
        both ``[Q, k]``."""
        q = {n: queries[n].to(self.device, self.dtype) for n in self.ordered_modules}
        if self.preconditioner is not None:
            q = {n: g.to(self.dtype) for n, g in self.preconditioner.apply(q).items()}
        if self.unit_norm:
            norm = torch.cat(list(q.values()), dim=1).norm(dim=1, keepdim=True)
            q = {n: g / (norm + torch.finfo(norm.dtype).eps) for n, g in q.items()}
        if self.faiss_index:
            if modules:
                raise NotImplementedError("FAISS index does not implement module-specific search.")
            flat = torch.cat([q[n] for n in self.ordered_modules], dim=1).float().cpu().numpy()
            d, i = self.faiss_index.search(flat, k, reverse=reverse)
            return torch.from_numpy(d), torch.from_numpy(i)
        use = [n for n in self.ordered_modules if not modules or n in modules]
        k = min(k or self.N, self.N)
        if len(use) == len(self.ordered_modules):
            store, q_rows = self.store, torch.cat([q[n] for n in use], dim=1)
        else:
            cols = torch.cat([torch.arange(*self.offsets[n], device=self.store.device) for n in use])
            store, q_rows = self.store[:, cols].contiguous(), torch.cat([q[n] for n in use], dim=1)
        scores, idx = attribution.topk_scores(store, q_rows.contiguous(), min(k, store.shape[0]), largest=not reverse,
                                              inv_norms=self.inv_norms)
        if not self.sharded:
            return scores, idx
        return merge_topk_across_ranks(scores, idx + self.row_lo, k, largest=not reverse, group=self.group)

    @contextmanager
    def trace(self, module: nn.Module, k: int | None, *, modules: set[str] | None = None,
              reverse: bool = False) -> Generator[TraceResult, None, None]:
        """Collect the gradients of the backward passes run inside the block as queries and
        search the index with them on exit."""
        result = TraceResult()
        collector = TraceCollector(model=module, processor=self.processor, target_modules=modules,
                                   device=self.device, dtype=self.dtype)
        grads = collector.mod_grads
        with collector:
            yield result
        if not grads:
            raise ValueError("No grads collected. Did you forget to call backward?")
        queries = {n: torch.cat(grads[n], dim=0) for n in self.ordered_modules if n in grads}
        if any(v.isnan().any() for v in queries.values()):
            raise ValueError("NaN found in queries.")
        result._scores, result._indices = self.search(queries, k, modules, reverse)
