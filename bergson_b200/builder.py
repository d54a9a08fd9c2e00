"""Gradient-store writer.

``Builder`` receives per-module gradient blocks of a batch, optionally preconditions
and unit-normalises them, and either scatters the rows into the store (memmap on disk
or a numpy array in memory) or accumulates one aggregate row (reference
``bergson/builder.py:17-232``).

Rows leave the GPU without a device synchronisation: ``write_rows_async`` has the
row-finalisation kernel write the clamped / normalised / cast rows straight into a slot
of a page-locked staging ring (host memory mapped into the device address space),
records an event, and a writer thread copies the slot into the store once the event
has fired.
"""

from __future__ import annotations

import queue
import threading
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

from .config.config import PreprocessConfig
from .data import compute_num_token_grads, create_index, create_token_index
from .utils.utils import convert_dtype_to_np, current_device, tensor_to_numpy

_EPS_SQ = torch.finfo(torch.float32).eps ** 2


def _preprocess(mod_grads, grad_sizes, preconditioner, do_normalize: bool) -> torch.Tensor:
    """Precondition, concatenate in ``grad_sizes`` order, optionally unit-normalise
    (``row * rsqrt(max(sum(row^2), eps_fp32^2))``)."""
    if preconditioner is not None:
        mod_grads = preconditioner.apply(mod_grads)
    grads = torch.cat([mod_grads[m] for m in grad_sizes], dim=-1)
    if do_normalize:
        inv = grads.pow(2).sum(dim=-1).clamp_min_(_EPS_SQ).rsqrt().unsqueeze(1)
        grads = grads * inv
    return grads


class _StagedWriter:
    """Ring of pinned host buffers drained into the store by a background thread."""

    def __init__(self, store: np.ndarray, width: int, dtype: torch.dtype, slots: int = 3):
        self.store = store
        self.width = width
        self.dtype = dtype
        self.slots: list[torch.Tensor | None] = [None] * slots
        self.free: queue.Queue[int] = queue.Queue()
        for i in range(slots):
            self.free.put(i)
        self.work: queue.Queue = queue.Queue()
        self.error: BaseException | None = None
        self.thread = threading.Thread(target=self._drain, name="bergson-store-writer", daemon=True)
        self.thread.start()

    def acquire(self, n: int) -> tuple[int, torch.Tensor]:
        slot = self.free.get()
        buf = self.slots[slot]
        if buf is None or buf.shape[0] < n:
            buf = torch.empty(max(n, 1), self.width, dtype=self.dtype, pin_memory=True)
            self.slots[slot] = buf
        return slot, buf

    def submit(self, slot: int, n: int, indices, event: torch.cuda.Event) -> None:
        self.work.put((slot, n, np.asarray(indices, dtype=np.int64), event))

    def _drain(self) -> None:
        while True:
            item = self.work.get()
            if item is None:
                return
            slot, n, indices, event = item
            try:
                event.synchronize()
                self.store[indices] = tensor_to_numpy(self.slots[slot][:n])
            except BaseException as e:  # noqa: BLE001 - surfaced in close()
                self.error = e
            finally:
                self.free.put(slot)

    def close(self) -> None:
        self.work.put(None)
        self.thread.join()
        if self.error is not None:
            raise self.error


class Builder:
    """Writes gradient rows for every combination of disk / memory, per-sequence /
    per-token, with optional preconditioning and aggregation."""

    grad_buffer: np.ndarray

    def __init__(
        self,
        data,
        grad_sizes: dict[str, int],
        dtype: torch.dtype,
        preprocess_cfg: PreprocessConfig,
        *,
        attribute_tokens: bool = False,
        path: Path | None = None,
    ):
        from .hessians.preconditioner import load_preconditioner

        self.grad_sizes = grad_sizes
        self.num_items = len(data)
        self.preprocess_cfg = preprocess_cfg
        self.dtype = dtype
        total = sum(grad_sizes.values())
        device = current_device()
        self.preconditioner = load_preconditioner(
            preprocess_cfg.hessian_path,
            inversion_cfg=preprocess_cfg.inversion_cfg,
            power=-0.5 if preprocess_cfg.unit_normalize else -1.0,
            ev_correction=preprocess_cfg.ev_correction,
            device=device,
        )
        self._writer: _StagedWriter | None = None

        if preprocess_cfg.aggregation != "none":
            np_dtype, num_grads = np.dtype(np.float32), 1
            self.in_memory_grad_buffer: torch.Tensor | None = torch.zeros(
                (1, total), dtype=torch.float32, device=device
            )
        else:
            np_dtype, num_grads = convert_dtype_to_np(dtype), self.num_items
            self.in_memory_grad_buffer = None

        self.num_token_grads = None
        self.offsets = None
        if attribute_tokens:
            self.num_token_grads = compute_num_token_grads(data)
            if path is not None:
                self.grad_buffer, self.offsets = create_token_index(path, self.num_token_grads, grad_sizes, np_dtype)
            else:
                self.offsets = np.zeros(len(self.num_token_grads) + 1, dtype=np.int64)
                np.cumsum(self.num_token_grads, out=self.offsets[1:])
                self.grad_buffer = np.zeros((int(self.offsets[-1]), total), dtype=np_dtype)
        elif path is not None:
            self.grad_buffer = create_index(path, num_grads=num_grads, grad_sizes=grad_sizes, dtype=np_dtype)
        else:
            self.grad_buffer = np.zeros((num_grads, total), dtype=np_dtype)

    # -- synchronous path (any device) ---------------------------------------------------

    def __call__(self, indices: list[int], mod_grads: dict[str, torch.Tensor]) -> None:
        grads = _preprocess(mod_grads, self.grad_sizes, self.preconditioner, self.preprocess_cfg.unit_normalize)
        if self.in_memory_grad_buffer is not None:
            self.in_memory_grad_buffer[0] += grads.sum(dim=0).to(
                dtype=torch.float32, device=self.in_memory_grad_buffer.device
            )
            return
        host = tensor_to_numpy(grads.cpu())  # blocking copy orders after the producing kernels
        if self.offsets is None:
            self.grad_buffer[indices] = host
            return
        row = 0
        for idx in indices:
            lo, hi = int(self.offsets[idx]), int(self.offsets[idx + 1])
            self.grad_buffer[lo:hi] = host[row : row + (hi - lo)]
            row += hi - lo

    # -- asynchronous fused path (CUDA) -------------------------------------------------

    @property
    def supports_async_rows(self) -> bool:
        """Fused row emission handles per-sequence and per-token stores without a
        preconditioner or aggregation; everything else takes ``__call__``."""
        return self.in_memory_grad_buffer is None and self.preconditioner is None and torch.cuda.is_available()

    def write_rows_async(self, indices: list[int], acc: torch.Tensor, lo: float, hi: float) -> None:
        """``acc``: fp32 ``[n, total_dim]`` rows on the device.  Enqueues: finalise into a
        pinned slot -> event -> background copy into the store.  Never blocks on the GPU
        unless every slot is still in flight."""
        from .ops import native

        if self._writer is None:
            self._writer = _StagedWriter(self.grad_buffer, acc.shape[1], self.dtype)
        n = acc.shape[0]
        rows: list[int] | np.ndarray = indices
        if self.offsets is not None:
            # Per-token store: the accumulator holds the documents' collected tokens in order.
            rows = np.concatenate([np.arange(self.offsets[i], self.offsets[i + 1]) for i in indices]) if indices else \
                np.zeros(0, dtype=np.int64)
            assert len(rows) == n, f"token rows ({n}) do not match the store's offsets ({len(rows)})"
            if n == 0:
                return
        slot, buf = self._writer.acquire(n)
        native.finalize_rows(acc, buf[:n], None, lo, hi, self.preprocess_cfg.unit_normalize)
        ev = torch.cuda.Event()
        ev.record()
        self._writer.submit(slot, n, rows, ev)

    # -- lifecycle ----------------------------------------------------------------------

    def flush(self) -> None:
        if self._writer is not None:
            self._writer.close()
            self._writer = None
        if isinstance(self.grad_buffer, np.memmap):
            self.grad_buffer.flush()

    def teardown(self) -> None:
        self.flush()
        if self.in_memory_grad_buffer is None:
            # In-memory stores are filled disjointly by the ranks: a sum gathers them.
            if dist.is_initialized() and not isinstance(self.grad_buffer, np.memmap):
                buf = self.grad_buffer
                if buf.dtype == np.dtype("bfloat16"):
                    t = torch.from_numpy(buf.view(np.uint16)).view(torch.bfloat16)
                else:
                    t = torch.from_numpy(buf)
                dist.all_reduce(t, op=dist.ReduceOp.SUM)
            return
        agg = self.in_memory_grad_buffer
        if dist.is_initialized():
            dist.reduce(agg, dst=0, op=dist.ReduceOp.SUM)
        if self.preprocess_cfg.aggregation == "mean":
            agg /= self.num_items
        if self.preprocess_cfg.normalize_aggregated_grad:
            from .process_grads import normalize_flat_grad

            agg = normalize_flat_grad(agg, agg.device)
        self.in_memory_grad_buffer = agg = agg.cpu()
        if (dist.get_rank() if dist.is_initialized() else 0) == 0:
            self.grad_buffer[:] = tensor_to_numpy(agg).astype(self.grad_buffer.dtype)
