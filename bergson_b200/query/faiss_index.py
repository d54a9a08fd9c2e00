"""Sharded on-disk nearest-neighbour index over a gradient store
(reference ``bergson/query/faiss_index.py:56-409``).

With the optional ``faiss`` package installed the shards are FAISS indices built from
``index_factory`` (inner-product metric).  Without it the shards are the in-tree indices of
``native_ann.py`` (Flat, SQfp16, IVF<n>, PQ<m> and their combinations; searched with matrix
products on the store's device) behind the same directory layout and API; factory strings
that neither implements raise.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import numpy as np
import torch

from ..config import FaissConfig
from ..data import column_offsets, load_gradients
from ..utils.utils import numpy_to_tensor
from .native_ann import NativeIndex, parse_factory

try:
    import faiss  # type: ignore

    HAVE_FAISS = True
except ImportError:  # pragma: no cover - depends on the environment
    faiss = None
    HAVE_FAISS = False


def _prepare(block: np.ndarray, sizes: dict[str, int], device, unit_norm: bool, h_inv: dict) -> np.ndarray:
    x = numpy_to_tensor(np.ascontiguousarray(block)).to(device=device, dtype=torch.float32)
    if h_inv:
        for name, (lo, hi) in column_offsets(sizes).items():
            if name in h_inv:
                x[:, lo:hi] = x[:, lo:hi] @ h_inv[name].to(x.device, x.dtype)
    if unit_norm:
        x = torch.nan_to_num(x / x.norm(dim=1, keepdim=True), nan=0.0, posinf=0.0, neginf=0.0)
    return x.cpu().numpy()


class FaissIndex:
    """Shards ``0..k-1`` under ``path`` plus a ``config.yaml`` (JSON content)."""

    def __init__(self, path: Path, device: str = "cpu", mmap_index: bool = False):
        self.path = Path(path)
        with open(self.path / "config.yaml") as f:
            meta = json.load(f)
        self.ordered_modules = meta["ordered_modules"]
        self.backend = meta.get("backend", "faiss")
        self.nprobe = meta.get("nprobe", 10)
        self.shards = []
        self.sizes = []
        for i in range(meta["num_shards"]):
            if self.backend == "faiss":
                flags = faiss.IO_FLAG_MMAP | faiss.IO_FLAG_READ_ONLY if mmap_index else 0
                idx = faiss.read_index(str(self.path / f"{i}.faiss"), flags)
                if hasattr(idx, "nprobe"):
                    idx.nprobe = self.nprobe
                if device != "cpu" and not mmap_index and hasattr(faiss, "index_cpu_to_all_gpus"):
                    idx = faiss.index_cpu_to_all_gpus(idx)
                self.shards.append(idx)
                self.sizes.append(idx.ntotal)
            elif self.backend == "native":
                idx = NativeIndex.load(self.path / str(i), device="cpu" if mmap_index else device, mmap=mmap_index)
                idx.nprobe = self.nprobe
                self.shards.append(idx)
                self.sizes.append(idx.ntotal)
            else:  # exact fp32 rows written by earlier versions
                arr = np.load(self.path / f"{i}.npy", mmap_mode="r" if mmap_index else None)
                self.shards.append(arr)
                self.sizes.append(arr.shape[0])
        self.device = device

    @property
    def ntotal(self) -> int:
        return int(sum(self.sizes))

    @staticmethod
    def create_index(index_path: Path, faiss_path: Path, cfg: FaissConfig, device: str, unit_norm: bool, h_inv: dict):
        faiss_path.mkdir(parents=True, exist_ok=True)
        mm = load_gradients(index_path)
        with open(Path(index_path) / "info.json") as f:
            sizes = json.load(f)["grad_sizes"]
        n = mm.shape[0]
        per = math.ceil(n / cfg.num_shards)
        backend = "faiss" if HAVE_FAISS else "native"
        factory = None if HAVE_FAISS else parse_factory(cfg.index_factory)  # raises for unsupported strings
        for s in range(cfg.num_shards):
            lo, hi = s * per, min((s + 1) * per, n)
            parts = [_prepare(mm[a : min(a + cfg.batch_size, hi)], sizes, device, unit_norm, h_inv)
                     for a in range(lo, hi, cfg.batch_size)]
            x = np.concatenate(parts) if parts else np.zeros((0, mm.shape[1]), np.float32)
            if backend == "faiss":
                idx = faiss.index_factory(x.shape[1], cfg.index_factory, faiss.METRIC_INNER_PRODUCT)
                train = x if cfg.max_train_examples is None else x[: cfg.max_train_examples]
                idx.train(train)
                idx.add(x)
                faiss.write_index(idx, str(faiss_path / f"{s}.faiss"))
            else:
                idx = NativeIndex(x.shape[1], factory, device)
                if factory.needs_training:
                    idx.train(x if cfg.max_train_examples is None else x[: cfg.max_train_examples])
                idx.add(x)
                idx.save(faiss_path / str(s))
        with open(faiss_path / "config.yaml", "w") as f:
            json.dump({"ordered_modules": list(sizes), "num_shards": cfg.num_shards, "backend": backend,
                       "index_factory": cfg.index_factory, "nprobe": cfg.nprobe}, f)

    def search(self, q: np.ndarray, k: int | None, reverse: bool = False):
        """(scores, indices) of the ``k`` best (worst if ``reverse``) rows over all shards."""
        k = min(k or self.ntotal, self.ntotal)
        q = np.ascontiguousarray(q, dtype=np.float32)
        all_d, all_i, base = [], [], 0
        for shard, size in zip(self.shards, self.sizes):
            kk = min(k, size)
            if self.backend in ("faiss", "native"):
                d, i = shard.search(-q if reverse else q, kk)
                d = -d if reverse else d
            else:
                s = q @ np.asarray(shard).T
                order = np.argsort(s if reverse else -s, axis=1)[:, :kk]
                d, i = np.take_along_axis(s, order, 1), order
            all_d.append(d)
            all_i.append(np.where(i >= 0, i + base, -1))
            base += size
        d, i = np.concatenate(all_d, 1), np.concatenate(all_i, 1)
        order = np.argsort(d if reverse else -d, axis=1)[:, :k]
        return np.take_along_axis(d, order, 1), np.take_along_axis(i, order, 1)
