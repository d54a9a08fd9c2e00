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
from typing import Protocol

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


class Index(Protocol):
    """What a shard has to offer, whichever backend built it."""

    def search(self, x: np.ndarray, k: int) -> tuple[np.ndarray, np.ndarray]: ...

    @property
    def ntotal(self) -> int: ...

    def train(self, x: np.ndarray) -> None: ...

    def add(self, x: np.ndarray) -> None: ...


def validate_ram(batch: np.ndarray, max_shard_size: int) -> None:
    """Refuse to build when the largest shard (``max_shard_size`` rows of the width and type of
    ``batch``, widened to fp32 for the index) cannot fit into the memory that is free now."""
    import psutil

    free_gb = psutil.virtual_memory().available / 2**30
    per_row = max(batch.nbytes / max(batch.shape[0], 1), 4 * batch.shape[1])
    need_gb = max_shard_size * per_row / 2**30
    print(f"Largest index shard needs about {need_gb:.2f} GB of host memory; {free_gb:.2f} GB are free")
    assert need_gb <= free_gb, "Not enough RAM to build index."


def normalize_grads(grads: np.ndarray, device: str, batch_size: int) -> np.ndarray:
    """Rows scaled to unit norm (zero rows stay zero), ``batch_size`` rows at a time on ``device``."""
    out = np.empty(grads.shape, dtype=np.float32)
    for lo in range(0, grads.shape[0], batch_size):
        out[lo : lo + batch_size] = _prepare(grads[lo : lo + batch_size], {}, device, True, {})
    return out


def gradients_loader(root_dir: Path):
    """``(memory-mapped gradients, module names)`` for the store under ``root_dir``, or for each
    ``*shard*`` sub-directory (in name order) when the store was written in several parts."""
    root_dir = Path(root_dir)

    def one(d: Path):
        with open(d / "info.json") as f:
            return load_gradients(d), list(json.load(f)["grad_sizes"])

    if (root_dir / "info.json").exists():
        yield one(root_dir)
    else:
        for path in sorted(root_dir.iterdir()):
            if path.is_dir() and "shard" in path.name:
                yield one(path)


def index_to_device(index, device: str):
    """The shard on ``device``: an in-tree index moves its tensors, a FAISS index is cloned to the
    GPUs (``cuda`` = all visible ones, ``cuda:<i>`` = that one) or left alone for ``cpu``."""
    if isinstance(index, NativeIndex):
        dev = torch.device(device)
        if index.device != dev:
            for name in ("vectors", "ids", "centroids", "codebooks"):
                t = getattr(index, name)
                if isinstance(t, torch.Tensor):
                    setattr(index, name, t.to(dev))
            index._row_list = None
            index.device = dev
        return index
    if device == "cpu" or faiss is None or not hasattr(faiss, "index_cpu_to_all_gpus"):
        return index
    if ":" in device:
        return faiss.index_cpu_to_gpu(faiss.StandardGpuResources(), int(device.split(":")[1]), index)
    return faiss.index_cpu_to_all_gpus(index)


def _prepare(block: np.ndarray, sizes: dict[str, int], device, unit_norm: bool, h_inv: dict) -> np.ndarray:
    x = numpy_to_tensor(np.ascontiguousarray(block)).to(device=device, dtype=torch.float32)
    if h_inv:
        for name, (lo, hi) in column_offsets(sizes).items():
            if name in h_inv:
                x[:, lo:hi] = x[:, lo:hi] @ h_inv[name].to(x.device, x.dtype)
    if unit_norm:
        x = torch.nan_to_num(x / x.norm(dim=1, keepdim=True), nan=0.0, posinf=0.0, neginf=0.0)
    return x.cpu().numpy()


class _Concatenated:
    """Row-wise concatenation of several memory-mapped stores, sliced like one array."""

    def __init__(self, parts: list):
        self.parts = parts
        self.starts = np.cumsum([0] + [p.shape[0] for p in parts])
        self.shape = (int(self.starts[-1]), parts[0].shape[1])

    def __getitem__(self, key):
        assert isinstance(key, slice) and key.step in (None, 1)
        lo, hi, _ = key.indices(self.shape[0])
        out = []
        for p, s in zip(self.parts, self.starts[:-1]):
            a, b = max(lo - s, 0), min(hi - s, p.shape[0])
            if a < b:
                out.append(np.asarray(p[a:b]))
        return np.concatenate(out) if out else np.zeros((0, self.shape[1]), self.parts[0].dtype)


class FaissIndex:
    """Shards ``0..k-1`` under ``path`` plus a ``config.yaml`` (JSON content)."""

    def __init__(self, path: Path, device: str = "cpu", mmap_index: bool = False):
        self.path = Path(path)
        with open(self.path / "config.yaml") as f:
            meta = json.load(f)
        self.ordered_modules = meta["ordered_modules"]
        self.backend = meta.get("backend", "faiss")
        self._nprobe = meta.get("nprobe", 10)
        self.shards = []
        self.sizes = []
        for i in range(meta["num_shards"]):
            if self.backend == "faiss":
                flags = faiss.IO_FLAG_MMAP | faiss.IO_FLAG_READ_ONLY if mmap_index else 0
                idx = faiss.read_index(str(self.path / f"{i}.faiss"), flags)
                if hasattr(idx, "nprobe"):
                    idx.nprobe = self.nprobe
                if device != "cpu" and not mmap_index:
                    idx = index_to_device(idx, device)
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

    @property
    def nprobe(self) -> int:
        """Inverted lists probed per query; setting it reaches every shard that has lists."""
        return self._nprobe

    @nprobe.setter
    def nprobe(self, value: int) -> None:
        self._nprobe = int(value)
        for shard in self.shards:
            if hasattr(shard, "nprobe"):
                shard.nprobe = self._nprobe

    @staticmethod
    def create_index(gradients_path: Path, faiss_path: Path, faiss_cfg: FaissConfig, device: str, unit_norm: bool,
                     hessians: dict):
        """Build the shards of ``faiss_cfg`` under ``faiss_path`` from the store (or the ``*shard*`` parts)
        under ``gradients_path``; ``hessians`` maps module names to the matrices applied to their columns."""
        index_path, cfg, h_inv = Path(gradients_path), faiss_cfg, hessians
        faiss_path = Path(faiss_path)
        faiss_path.mkdir(parents=True, exist_ok=True)
        parts = list(gradients_loader(Path(index_path)))
        if not parts:
            raise FileNotFoundError(f"No gradient store under {index_path}")
        info_dir = Path(index_path) if (Path(index_path) / "info.json").exists() else \
            sorted(p for p in Path(index_path).iterdir() if p.is_dir() and "shard" in p.name)[0]
        with open(info_dir / "info.json") as f:
            sizes = json.load(f)["grad_sizes"]
        mm = parts[0][0] if len(parts) == 1 else _Concatenated([m for m, _ in parts])
        n = mm.shape[0]
        per = math.ceil(n / cfg.num_shards)
        validate_ram(np.asarray(mm[: min(n, 16)]), per)
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
