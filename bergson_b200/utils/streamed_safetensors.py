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
import struct
import threading

import torch
from torch import Tensor

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
        host = tensor.detach().cpu().contiguous()  # waits for the producing stream of a device tensor
        offset, nbytes = self._ranges[name]
        with self._lock:
            if name not in self._pending:
                raise ValueError(f"{name} was already written")
            self._pending.discard(name)
        if nbytes:
            view = memoryview(host.reshape(-1).view(torch.uint8).numpy())
            done = 0
            while done < nbytes:
                done += os.pwrite(self._fd, view[done:], self._base + offset + done)

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
