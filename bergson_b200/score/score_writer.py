"""Score stores.

``scores.bin`` is a 1-D structured array with, per score column i, a ``score_i`` value
and a ``written_i`` flag.  Each pair is padded to the next power of two of
``itemsize + 1`` bytes and the record size is rounded up to a multiple of 8
(reference ``bergson/score/score_writer.py:16-58``), so an interrupted run can tell
which cells are valid.
"""

from __future__ import annotations

import json
from abc import ABC, abstractmethod
from pathlib import Path
from typing import Any

import ml_dtypes  # noqa: F401
import numpy as np
import torch
import torch.distributed as dist

from ..data import compute_num_token_grads
from ..utils.utils import convert_dtype_to_np, numpy_to_tensor, tensor_to_numpy


def _score_struct_dtype(num_scores: int, np_dtype: np.dtype) -> tuple[dict, dict]:
    """(numpy dtype spec, JSON-safe copy of it)."""
    np_dtype = np.dtype(np_dtype)
    pair = np_dtype.itemsize + 1
    stride = 1 << (pair - 1).bit_length()
    names, formats, offsets = [], [], []
    for i in range(num_scores):
        names += [f"score_{i}", f"written_{i}"]
        formats += [np_dtype, "bool"]
        offsets += [i * stride, i * stride + np_dtype.itemsize]
    itemsize = (num_scores * stride + 7) // 8 * 8
    spec = {"names": names, "formats": formats, "offsets": offsets, "itemsize": itemsize}
    spec_json = dict(spec, formats=[str(f) if isinstance(f, np.dtype) else f for f in formats])
    return spec, spec_json


class ScoreWriter(ABC):
    scores: Any

    @abstractmethod
    def __call__(self, indices: list[int], scores: torch.Tensor, query_offset: int = 0): ...

    @abstractmethod
    def flush(self): ...


class InMemorySequenceScoreWriter(ScoreWriter):
    def __init__(self, num_items: int, num_scores: int, dtype: torch.dtype = torch.float32):
        self.scores = torch.zeros((num_items, num_scores), dtype=dtype)

    def __call__(self, indices, scores, query_offset: int = 0):
        w = scores.shape[1]
        self.scores[indices, query_offset : query_offset + w] = scores.to(self.scores.dtype).cpu()

    def flush(self):
        pass


class InMemoryTokenScoreWriter(ScoreWriter):
    def __init__(self, data, num_scores: int, dtype: torch.dtype = torch.float32):
        self.num_token_grads = compute_num_token_grads(data)
        self.offsets = np.zeros(len(self.num_token_grads) + 1, dtype=np.int64)
        np.cumsum(self.num_token_grads, out=self.offsets[1:])
        self.scores = [torch.zeros((int(n), num_scores), dtype=dtype) for n in self.num_token_grads]
        self.dtype = dtype

    def __call__(self, indices, scores, query_offset: int = 0):
        host = scores.to(self.dtype).cpu()
        row, w = 0, scores.shape[1]
        for idx in indices:
            n = int(self.num_token_grads[idx])
            self.scores[idx][:, query_offset : query_offset + w] = host[row : row + n]
            row += n

    def flush(self):
        pass


class _MemmapScoreWriter(ScoreWriter):
    """Shared creation / mapping logic of the two on-disk writers."""

    def _open(self, path: Path, num_rows: int, info: dict, num_scores: int, dtype, overwrite, distributed, extra=None):
        self.path = Path(path)
        self.num_scores = num_scores
        self.dtype = dtype
        self.path.mkdir(parents=True, exist_ok=True)
        file = self.path / "scores.bin"
        spec, spec_json = _score_struct_dtype(num_scores, convert_dtype_to_np(dtype))
        sync = distributed and dist.is_initialized()
        rank = dist.get_rank() if sync else 0
        if rank == 0 and (overwrite or not file.exists()):
            print(f"Creating new scores file: {file}")
            np.memmap(str(file), dtype=np.dtype(spec), mode="w+", shape=(num_rows,)).flush()
            with (self.path / "info.json").open("w") as f:
                json.dump(dict(info, num_rows=num_rows, num_scores=num_scores, dtype=spec_json), f, indent=2)
            if extra:
                extra()
        if sync:
            dist.barrier()
        self.scores = np.memmap(str(file), dtype=np.dtype(spec), mode="r+", shape=(num_rows,))
        self.num_batches_since_flush = 0

    def _tick(self):
        self.num_batches_since_flush += 1
        if self.num_batches_since_flush >= self.flush_interval:
            self.flush()

    def flush(self):
        self.scores.flush()
        self.num_batches_since_flush = 0


class MemmapSequenceScoreWriter(_MemmapScoreWriter):
    """One record per document.  An existing ``scores.bin`` is reused (resume) unless
    ``overwrite``."""

    def __init__(self, path, num_items: int, num_scores: int, *, dtype=torch.float32, flush_interval: int = 64,
                 overwrite: bool = False, distributed: bool = True):
        self.flush_interval = flush_interval
        self._open(path, num_items, {"attribute_tokens": False, "num_items": num_items}, num_scores, dtype,
                   overwrite, distributed)

    def __call__(self, indices, scores, query_offset: int = 0):
        host = tensor_to_numpy(scores.to(self.dtype).cpu())
        idx = np.asarray(indices)
        for i in range(host.shape[1]):
            self.scores[f"score_{query_offset + i}"][idx] = host[:, i]
            self.scores[f"written_{query_offset + i}"][idx] = True
        self._tick()


class MemmapTokenScoreWriter(_MemmapScoreWriter):
    """One record per gradient-carrying token; ``offsets.npy`` maps documents to rows."""

    def __init__(self, path, num_token_grads: np.ndarray, num_scores: int, *, dtype=torch.float32,
                 flush_interval: int = 64, overwrite: bool = False, distributed: bool = True):
        self.flush_interval = flush_interval
        self.num_token_grads = num_token_grads
        self.offsets = np.zeros(len(num_token_grads) + 1, dtype=np.int64)
        np.cumsum(num_token_grads, out=self.offsets[1:])
        path = Path(path)
        self._open(path, int(self.offsets[-1]), {"attribute_tokens": True, "num_items": len(num_token_grads)},
                   num_scores, dtype, overwrite, distributed,
                   extra=lambda: np.save(path / "offsets.npy", self.offsets))

    @classmethod
    def from_dataset(cls, path, data, num_scores: int, **kwargs):
        return cls(path, compute_num_token_grads(data), num_scores, **kwargs)

    def __call__(self, indices, scores, query_offset: int = 0):
        host = tensor_to_numpy(scores.to(self.dtype).cpu())
        row = 0
        for idx in indices:
            lo, hi = int(self.offsets[idx]), int(self.offsets[idx + 1])
            for i in range(host.shape[1]):
                self.scores[f"score_{query_offset + i}"][lo:hi] = host[row : row + hi - lo, i]
                self.scores[f"written_{query_offset + i}"][lo:hi] = True
            row += hi - lo
        self._tick()


def save_sequence_scores(path: Path, scores: np.ndarray, *, dtype: torch.dtype = torch.float32) -> None:
    """Write a complete ``[num_items, num_scores]`` matrix in one go."""
    scores = scores[:, None] if scores.ndim == 1 else scores
    w = MemmapSequenceScoreWriter(path, scores.shape[0], scores.shape[1], dtype=dtype, overwrite=True, distributed=False)
    w(list(range(scores.shape[0])), numpy_to_tensor(np.ascontiguousarray(scores)))
    w.flush()


def save_token_scores(path: Path, scores: np.ndarray, offsets: np.ndarray, *, dtype: torch.dtype = torch.float32) -> None:
    """Write a complete flat ``(total_tokens, num_scores)`` array in one go."""
    scores = scores[:, None] if scores.ndim == 1 else scores
    counts = np.diff(offsets).astype(np.int64)
    w = MemmapTokenScoreWriter(path, counts, scores.shape[1], dtype=dtype, overwrite=True, distributed=False)
    w(list(range(len(counts))), numpy_to_tensor(np.ascontiguousarray(scores)))
    w.flush()
