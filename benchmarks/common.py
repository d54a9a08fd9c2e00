"""Shared helpers of the secondary benchmarks (EK-FAC fit, query throughput, MAGIC step)."""

from __future__ import annotations

import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def use_reference() -> bool:
    """Put the unmodified reference (baseline/_ref) and its import stand-ins on sys.path."""
    ref, shims = ROOT / "baseline" / "_ref", ROOT / "baseline" / "shims"
    if not (ref / "bergson").exists():
        return False
    sys.path[:0] = [str(shims), str(ref)]
    return True


def cuda_timed(fn, warmup: int = 1, iters: int = 3) -> float:
    """Mean seconds per call, CUDA events, synchronised on both sides."""
    import torch

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(iters):
        fn()
    t1.record()
    torch.cuda.synchronize()
    return t0.elapsed_time(t1) / 1e3 / iters


def wall(fn) -> float:
    import torch

    torch.cuda.synchronize()
    t = time.perf_counter()
    fn()
    torch.cuda.synchronize()
    return time.perf_counter() - t
