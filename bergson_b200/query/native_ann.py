"""In-tree inner-product indices for the factory strings the gradient store is queried with:
``Flat``, ``SQfp16``, ``IVF<n>``, ``IVF<n>,Flat``, ``IVF<n>,SQfp16`` and ``IVF<n>,PQ<m>`` /
``PQ<m>`` (8-bit product quantiser).

The search is built from dense matrix products so that it runs on the GPU the store was
built on: queries x centroids picks the ``nprobe`` inverted lists of every query, then each
probed list is scored as one ``queries-that-probe-it x list-rows`` product and merged into a
running top-k.  Rows are stored sorted by list (``vectors`` / ``codes``, ``ids``, ``offsets``)
so a list is one contiguous slice, on the device or memory-mapped from disk.

File layout of shard ``i`` under the index directory: ``<i>.ann.json`` (kind, sizes) and
``<i>.<part>.npy`` for every array, each readable with ``numpy.load(mmap_mode="r")``.
"""

from __future__ import annotations

import json
import re
from dataclasses import dataclass
from pathlib import Path

import numpy as np
import torch
from torch import Tensor

KMEANS_ITERS = 10
KMEANS_POINTS_PER_CENTROID = 256
PQ_CODES = 256
PQ_ITERS = 8


@dataclass
class Factory:
    nlist: int  # 0 = no inverted lists (every row is scanned)
    storage: str  # "fp32" | "fp16" | "pq"
    pq_m: int = 0

    @property
    def needs_training(self) -> bool:
        return self.nlist > 1 or self.storage == "pq"


def parse_factory(spec: str) -> Factory:
    """``"IVF1024,SQfp16"`` -> Factory(1024, "fp16"); raises ``ValueError`` for strings this
    backend does not implement (HNSW, OPQ, ...)."""
    parts = [p.strip() for p in spec.split(",") if p.strip()]
    nlist, storage, pq_m = 0, "fp32", 0
    for p in parts:
        if m := re.fullmatch(r"IVF(\d+)", p):
            nlist = int(m.group(1))
        elif p == "Flat":
            storage = "fp32"
        elif p in ("SQfp16", "SQ16"):
            storage = "fp16"
        elif m := re.fullmatch(r"PQ(\d+)(x8)?", p):
            storage, pq_m = "pq", int(m.group(1))
        else:
            raise ValueError(f"index_factory component {p!r} of {spec!r} is not implemented by the in-tree index "
                             "(supported: Flat, SQfp16, IVF<n>, PQ<m>, and IVF<n> combined with either)")
    if not parts:
        raise ValueError("empty index_factory")
    if nlist < 0 or (storage == "pq" and pq_m <= 0):
        raise ValueError(f"bad index_factory {spec!r}")
    return Factory(nlist, storage, pq_m)


def _kmeans(x: Tensor, k: int, iters: int, seed: int = 0) -> Tensor:
    """Lloyd's algorithm (L2) on ``x`` [n, d] fp32; empty clusters are re-seeded from the rows
    farthest from their centroid.  Returns [k, d]."""
    n = x.shape[0]
    g = torch.Generator(device="cpu").manual_seed(seed)
    if n <= k:
        reps = -(-k // max(n, 1))
        c = x.repeat(reps, 1)[:k].clone()
        return c + 1e-6 * torch.randn(c.shape, generator=g).to(c)
    c = x[torch.randperm(n, generator=g)[:k].to(x.device)].clone()
    x_sq = (x * x).sum(1)
    for _ in range(iters):
        d = x_sq[:, None] - 2 * (x @ c.T) + (c * c).sum(1)[None, :]
        dist, assign = d.min(1)
        sums = torch.zeros_like(c).index_add_(0, assign, x)
        counts = torch.bincount(assign, minlength=k).to(x.dtype)
        empty = counts == 0
        c = torch.where(empty[:, None], c, sums / counts.clamp_min(1)[:, None])
        n_empty = int(empty.sum())
        if n_empty:
            c[empty] = x[dist.topk(n_empty).indices]
    return c


class NativeIndex:
    """One shard.  ``train`` (if the factory needs it) -> ``add`` (once) -> ``search`` / ``save``."""

    def __init__(self, dim: int, factory: Factory, device: str | torch.device = "cpu"):
        self.dim = dim
        self.factory = factory
        self.device = torch.device(device)
        self.centroids: Tensor | None = None  # [nlist, d] fp32
        self.codebooks: Tensor | None = None  # [m, 256, d/m] fp32
        self.vectors = None  # fp32 / fp16 rows or uint8 codes, sorted by list (tensor or memmap)
        self.ids = None  # int64 original row of every stored row
        self.offsets = np.zeros(1, np.int64)  # [nlist + 1] list boundaries
        self.ntotal = 0
        self.nprobe = 10
        self.dense_scan: bool | None = None  # None: chosen per search from the number of probed lists
        self._row_list: Tensor | None = None
        if factory.storage == "pq" and dim % factory.pq_m:
            raise ValueError(f"PQ{factory.pq_m} needs the dimension ({dim}) to be a multiple of {factory.pq_m}")

    # ---------------------------------------------------------------- build
    @property
    def is_trained(self) -> bool:
        f = self.factory
        return (f.nlist <= 1 or self.centroids is not None) and (f.storage != "pq" or self.codebooks is not None)

    def train(self, x: np.ndarray | Tensor) -> None:
        x = torch.as_tensor(np.asarray(x) if not isinstance(x, Tensor) else x).to(self.device, torch.float32)
        f = self.factory
        if f.nlist > 1:
            cap = f.nlist * KMEANS_POINTS_PER_CENTROID
            sample = x if x.shape[0] <= cap else x[torch.randperm(x.shape[0], generator=torch.Generator().manual_seed(1))[:cap].to(x.device)]
            self.centroids = _kmeans(sample, f.nlist, KMEANS_ITERS)
        if f.storage == "pq":
            cap = PQ_CODES * KMEANS_POINTS_PER_CENTROID
            sample = x[:cap]
            if self.centroids is not None:
                sample = sample - self.centroids[self._assign(sample)]  # residuals, as stored
            sub = sample.view(sample.shape[0], f.pq_m, -1)
            self.codebooks = torch.stack([_kmeans(sub[:, j].contiguous(), PQ_CODES, PQ_ITERS, seed=j) for j in range(f.pq_m)])

    def _assign(self, x: Tensor) -> Tensor:
        """List of each row: the centroid with the largest inner product (the metric of the search)."""
        out = []
        for lo in range(0, x.shape[0], 65536):
            out.append((x[lo : lo + 65536] @ self.centroids.T).argmax(1))
        return torch.cat(out) if out else torch.zeros(0, dtype=torch.long, device=x.device)

    def _encode(self, x: Tensor) -> Tensor:
        f = self.factory
        if f.storage == "fp32":
            return x
        if f.storage == "fp16":
            return x.to(torch.float16)
        sub = x.view(x.shape[0], f.pq_m, -1)
        codes = torch.empty(x.shape[0], f.pq_m, dtype=torch.uint8, device=x.device)
        for j in range(f.pq_m):
            cb = self.codebooks[j]
            d = (cb * cb).sum(1)[None, :] - 2 * (sub[:, j] @ cb.T)
            codes[:, j] = d.argmin(1).to(torch.uint8)
        return codes

    def add(self, x: np.ndarray | Tensor) -> None:
        if self.ntotal:
            raise RuntimeError("NativeIndex.add may be called once per shard")
        if not self.is_trained:
            raise RuntimeError("train() the index before add()")
        x = torch.as_tensor(np.asarray(x) if not isinstance(x, Tensor) else x).to(self.device, torch.float32)
        n = x.shape[0]
        if self.factory.nlist > 1:
            lists = self._assign(x)
            order = torch.argsort(lists, stable=True)
            counts = torch.bincount(lists, minlength=self.factory.nlist)
            x = x[order]
            if self.factory.storage == "pq":
                x = x - self.centroids[lists[order]]
            self.ids = order
            self.offsets = np.concatenate([[0], np.cumsum(counts.cpu().numpy())]).astype(np.int64)
        else:
            self.ids = torch.arange(n, device=self.device)
            self.offsets = np.array([0, n], np.int64)
        self.vectors = self._encode(x)
        self.ntotal = n

    # ---------------------------------------------------------------- search
    def _rows(self, lo: int, hi: int) -> Tensor:
        """Stored rows [lo, hi) decoded to fp32 on the search device."""
        v = self.vectors[lo:hi]
        if not isinstance(v, Tensor):
            v = torch.from_numpy(np.array(v))  # a copy: the memory map is read-only
        v = v.to(self.device)
        if self.factory.storage != "pq":
            return v.to(torch.float32)
        m = self.factory.pq_m
        idx = v.long()  # [r, m]
        return torch.stack([self.codebooks[j][idx[:, j]] for j in range(m)], 1).reshape(v.shape[0], self.dim)

    def _scores(self, q: Tensor, lo: int, hi: int) -> Tensor:
        """fp32 inner products of ``q`` with stored rows [lo, hi).  16-bit rows on a GPU go through
        the tensor-core score GEMM (16-bit operands, fp32 accumulation and output) without being
        widened first; everything else is an fp32 product with the decoded rows."""
        v = self.vectors
        if self.factory.storage == "fp16" and isinstance(v, Tensor) and v.is_cuda and self.dim % 8 == 0:
            from ..ops import attribution

            return attribution.score_rows(q, v[lo:hi], torch.float16, False)[0]
        return q @ self._rows(lo, hi).T

    def _row_lists(self) -> Tensor:
        """Inverted list of every stored row (rows are sorted by list)."""
        if self._row_list is None:
            counts = torch.from_numpy(np.diff(self.offsets)).to(self.device)
            self._row_list = torch.repeat_interleave(torch.arange(len(counts), device=self.device), counts)
        return self._row_list

    def _ids(self, lo: int, hi: int) -> Tensor:
        i = self.ids[lo:hi]
        if not isinstance(i, Tensor):
            i = torch.from_numpy(np.array(i))
        return i.to(self.device)

    def search(self, q: np.ndarray | Tensor, k: int) -> tuple[np.ndarray, np.ndarray]:
        """Top ``k`` inner products per query: (scores [nq, k] descending, row ids, -1 / -inf where a
        query's probed lists hold fewer than ``k`` rows)."""
        q = torch.as_tensor(np.asarray(q) if not isinstance(q, Tensor) else q).to(self.device, torch.float32)
        nq = q.shape[0]
        k = max(1, min(k, max(self.ntotal, 1)))
        best_d = torch.full((nq, k), float("-inf"), device=self.device)
        best_i = torch.full((nq, k), -1, dtype=torch.long, device=self.device)
        if self.ntotal == 0 or nq == 0:
            return best_d.cpu().numpy(), best_i.cpu().numpy()

        def merge(rows: Tensor | None, scores: Tensor, ids: Tensor):
            nonlocal best_d, best_i
            kk = min(k, scores.shape[1])
            d, j = scores.topk(kk, dim=1)
            i = ids[j]
            if rows is None:
                cat_d, cat_i = torch.cat([best_d, d], 1), torch.cat([best_i, i], 1)
                best_d, pos = cat_d.topk(k, dim=1)
                best_i = cat_i.gather(1, pos)
            else:
                cat_d, cat_i = torch.cat([best_d[rows], d], 1), torch.cat([best_i[rows], i], 1)
                top, pos = cat_d.topk(k, dim=1)
                best_d[rows] = top
                best_i[rows] = cat_i.gather(1, pos)

        nlist = self.factory.nlist
        if nlist <= 1:
            step = max(1, (64 << 20) // max(nq, 1))  # bound the score tile to 64M entries
            for lo in range(0, self.ntotal, step):
                hi = min(lo + step, self.ntotal)
                merge(None, self._scores(q, lo, hi), self._ids(lo, hi))
        else:
            nprobe = max(1, min(self.nprobe, nlist))
            coarse = q @ self.centroids.T  # [nq, nlist]
            probed = coarse.topk(nprobe, dim=1).indices
            hit = torch.zeros(nq, nlist, dtype=torch.bool, device=self.device)
            hit.scatter_(1, probed, True)
            pq = self.factory.storage == "pq"
            dense = self.dense_scan if self.dense_scan is not None else nq * nprobe >= nlist
            if dense:
                # Most lists are probed by some query: one pass over all rows in large tiles, with the
                # (query, row) pairs whose list the query does not probe masked out -- the same
                # candidates as the per-list loop below without its many small launches.
                row_list = self._row_lists()
                step = max(1, (64 << 20) // max(nq, 1))
                for lo in range(0, self.ntotal, step):
                    hi = min(lo + step, self.ntotal)
                    lists = row_list[lo:hi]
                    s = self._scores(q, lo, hi)
                    if pq:
                        s = s + coarse[:, lists]
                    merge(None, s.masked_fill_(~hit[:, lists], float("-inf")), self._ids(lo, hi))
            else:
                for l in hit.any(0).nonzero().flatten().tolist():
                    lo, hi = int(self.offsets[l]), int(self.offsets[l + 1])
                    if hi == lo:
                        continue
                    rows = hit[:, l].nonzero().flatten()
                    s = self._scores(q[rows], lo, hi)
                    if pq:
                        s = s + coarse[rows, l][:, None]  # stored rows are residuals to the centroid
                    merge(rows, s, self._ids(lo, hi))
        best_i = best_i.masked_fill(torch.isneginf(best_d), -1)
        return best_d.cpu().numpy(), best_i.cpu().numpy()

    # ---------------------------------------------------------------- files
    def save(self, prefix: Path) -> None:
        prefix = Path(prefix)
        meta = {"dim": self.dim, "nlist": self.factory.nlist, "storage": self.factory.storage, "pq_m": self.factory.pq_m,
                "ntotal": self.ntotal}
        arrays = {"vectors": self.vectors, "ids": self.ids, "offsets": self.offsets, "centroids": self.centroids,
                  "codebooks": self.codebooks}
        for name, arr in arrays.items():
            if arr is None:
                continue
            a = arr.cpu().numpy() if isinstance(arr, Tensor) else np.asarray(arr)
            np.save(f"{prefix}.{name}.npy", a)
        with open(f"{prefix}.ann.json", "w") as f:
            json.dump(meta, f)

    @classmethod
    def load(cls, prefix: Path, device: str | torch.device = "cpu", mmap: bool = False) -> "NativeIndex":
        prefix = Path(prefix)
        with open(f"{prefix}.ann.json") as f:
            meta = json.load(f)
        self = cls(meta["dim"], Factory(meta["nlist"], meta["storage"], meta["pq_m"]), device)
        self.ntotal = meta["ntotal"]

        def read(name: str, keep_on_disk: bool):
            p = Path(f"{prefix}.{name}.npy")
            if not p.exists():
                return None
            if keep_on_disk:
                return np.load(p, mmap_mode="r")
            return torch.from_numpy(np.load(p)).to(self.device)

        self.vectors = read("vectors", mmap)
        self.ids = read("ids", mmap)
        self.offsets = np.load(f"{prefix}.offsets.npy")
        self.centroids = read("centroids", False)
        self.codebooks = read("codebooks", False)
        return self
