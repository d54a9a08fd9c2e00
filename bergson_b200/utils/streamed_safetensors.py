"""A safetensors file whose tensors are written one by one, from any thread, as they become
available.

``safetensors.torch.save_file`` needs every tensor on the host before it writes the first byte,
which puts the whole file write after the last producer.  Here the header (names, dtypes,
shapes and byte ranges, all known before any data exists) is written first and each tensor's
bytes go to their own range with ``os.pwrite`` -- the call releases the interpreter lock, so
writes overlap the device work of other threads.  The result is an ordinary safetensors file.
"""

from __future__ import annotations

import json
import os
import queue
import struct
import threading

import torch
from torch import Tensor

# Device tensors reach the file through a small pool of page-locked staging buffers: a copy
# into pageable memory runs at a few GB/s, a copy into pinned memory at the bus rate, and the
# file write of one chunk overlaps the device copy of the next.  The pool is created once per
# process (page-locking memory is slow) and shared by all writers and threads.
_CHUNK = 16 << 20
_MAX_SLOTS = 8
_free_slots: "queue.LifoQueue[Tensor]" = queue.LifoQueue()
_n_slots = 0
_slot_lock = threading.Lock()


def _acquire_slot(block: bool) -> Tensor | None:
    global _n_slots
    try:
        return _free_slots.get_nowait()
    except queue.Empty:
        pass
    with _slot_lock:
        if _n_slots < _MAX_SLOTS:
            _n_slots += 1
            try:
                return torch.empty(_CHUNK, dtype=torch.uint8, pin_memory=True)
            except RuntimeError:
                # No page-locked memory to be had (locked-memory limit): a pageable buffer is
                # slower but just as correct, the copy into it simply completes before it returns.
                return torch.empty(_CHUNK, dtype=torch.uint8)
    # Every holder of a slot writes it out and returns it without waiting for another one, so a
    # blocking wait always ends.
    return _free_slots.get() if block else None

_DTYPE_NAMES = {
    torch.float64: "F64", torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16",
    torch.int64: "I64", torch.int32: "I32", torch.int16: "I16", torch.int8: "I8", torch.uint8: "U8",
    torch.bool: "BOOL",
}


class StreamedSafetensors:
    """``layout`` maps tensor name -> (shape, dtype).  ``write`` may be called once per name from
    any thread; ``close`` checks that every tensor arrived and publishes the file under its
    final name (the data is written to ``<path>.partial`` until then)."""

    def __init__(self, path: str, layout: dict[str, tuple[tuple[int, ...], torch.dtype]]):
        self.path = str(path)
        self._tmp = self.path + ".partial"
        header: dict[str, dict] = {}
        self._ranges: dict[str, tuple[int, int]] = {}
        self._layout = {k: (tuple(int(s) for s in shape), dtype) for k, (shape, dtype) in layout.items()}
        offset = 0
        for name in sorted(self._layout):
            shape, dtype = self._layout[name]
            n = 1
            for s in shape:
                n *= s
            nbytes = n * torch.empty((), dtype=dtype).element_size()
            header[name] = {"dtype": _DTYPE_NAMES[dtype], "shape": list(shape), "data_offsets": [offset, offset + nbytes]}
            self._ranges[name] = (offset, nbytes)
            offset += nbytes
        blob = json.dumps(header, separators=(",", ":")).encode()
        blob += b" " * (-len(blob) % 8)  # data starts on an 8-byte boundary
        self._base = 8 + len(blob)
        self._fd = os.open(self._tmp, os.O_WRONLY | os.O_CREAT | os.O_TRUNC, 0o644)
        os.pwrite(self._fd, struct.pack("<Q", len(blob)) + blob, 0)
        if offset:
            os.ftruncate(self._fd, self._base + offset)
        self._pending = set(self._layout)
        self._lock = threading.Lock()

    def write(self, name: str, tensor: Tensor) -> None:
        shape, dtype = self._layout[name]
        if tuple(tensor.shape) != shape or tensor.dtype != dtype:
            raise ValueError(f"{name}: expected {shape} {dtype}, got {tuple(tensor.shape)} {tensor.dtype}")
        offset, nbytes = self._ranges[name]
        with self._lock:
            if name not in self._pending:
                raise ValueError(f"{name} was already written")
            self._pending.discard(name)
        if not nbytes:
            return
        if tensor.is_cuda:
            self._write_from_device(tensor.detach(), self._base + offset, nbytes)
            return
        host = tensor.detach().contiguous()
        self._pwrite(memoryview(host.reshape(-1).view(torch.uint8).numpy()), self._base + offset)

    def _pwrite(self, view: memoryview, at: int) -> None:
        done = 0
        while done < len(view):
            done += os.pwrite(self._fd, view[done:], at + done)

    def _write_from_device(self, tensor: Tensor, at: int, nbytes: int) -> None:
        """Chunks of the tensor's bytes: device -> pinned slot (asynchronous, on the calling thread's
        current stream, which also orders the copy after the kernels that produced the tensor) ->
        file.  Up to two chunks are in flight, so one is written while the next is copied."""
        flat = tensor.contiguous().reshape(-1).view(torch.uint8)
        with torch.cuda.device(tensor.device):
            stream = torch.cuda.current_stream()
            in_flight: list[tuple[Tensor, torch.cuda.Event, int, int]] = []
            pos = 0
            try:
                while pos < nbytes or in_flight:
                    while pos < nbytes and len(in_flight) < 2:
                        slot = _acquire_slot(block=not in_flight)
                        if slot is None:
                            break
                        m = min(_CHUNK, nbytes - pos)
                        slot[:m].copy_(flat[pos : pos + m], non_blocking=True)
                        ev = torch.cuda.Event()
                        ev.record(stream)
                        in_flight.append((slot, ev, m, pos))
                        pos += m
                    slot, ev, m, off = in_flight.pop(0)
                    ev.synchronize()
                    try:
                        self._pwrite(memoryview(slot.numpy())[:m], at + off)
                    finally:
                        _free_slots.put(slot)
            finally:
                for slot, ev, _, _ in in_flight:  # only after an error: wait before the slots are reused
                    ev.synchronize()
                    _free_slots.put(slot)

    def close(self) -> None:
        if self._fd is None:
            return
        os.close(self._fd)
        self._fd = None
        if self._pending:
            os.unlink(self._tmp)
            raise RuntimeError(f"{self.path}: tensors never written: {sorted(self._pending)[:4]}")
        os.replace(self._tmp, self.path)

    def abort(self) -> None:
        if self._fd is not None:
            os.close(self._fd)
            self._fd = None
            if os.path.exists(self._tmp):
                os.unlink(self._tmp)

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc, tb):
        if exc_type is None:
            self.close()
        else:
            self.abort()
        return False


def save_tensors(tensors: dict[str, Tensor], path: str, threads: int = 4) -> None:
    """``safetensors.torch.save_file`` for tensors that may live on a device: the file is written
    tensor by tensor from ``threads`` helper threads (device copies through pinned staging, file
    writes releasing the interpreter lock), without first assembling everything on the host."""
    layout = {k: (tuple(v.shape), v.dtype) for k, v in tensors.items()}
    with StreamedSafetensors(path, layout) as w:
        names = sorted(tensors, key=lambda k: -tensors[k].numel())
        if threads <= 1 or len(names) <= 1:
            for k in names:
                w.write(k, tensors[k])
            return
        from concurrent.futures import ThreadPoolExecutor

        cuda_dev = next((v.device for v in tensors.values() if v.is_cuda), None)
        ready = None
        if cuda_dev is not None:
            # The helper threads copy on their own streams: order them after the producers.
            ready = torch.cuda.Event()
            ready.record(torch.cuda.current_stream(cuda_dev))

        def one(k: str) -> None:
            if cuda_dev is not None:
                with torch.cuda.device(cuda_dev), torch.cuda.stream(_thread_stream(cuda_dev)):
                    torch.cuda.current_stream().wait_event(ready)
                    w.write(k, tensors[k])
            else:
                w.write(k, tensors[k])

        with ThreadPoolExecutor(max_workers=min(threads, len(names))) as pool:
            list(pool.map(one, names))


_thread_streams = threading.local()


def _thread_stream(device) -> "torch.cuda.Stream":
    key = f"s{torch.device(device).index}"
    if not hasattr(_thread_streams, key):
        setattr(_thread_streams, key, torch.cuda.Stream(device))
    return getattr(_thread_streams, key)
