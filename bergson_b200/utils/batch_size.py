"""Automatic choice of ``token_batch_size``.

The reference searches exponentially and then by bisection for the largest batch that
does not raise an out-of-memory error (``bergson/utils/batch_size.py:21-309``).  Driving a
GPU out of memory on purpose is avoided here: peak memory of a worst-case forward/backward
under the real collector is *measured* at two small budgets, a linear model
``peak = base + per_token * tokens`` is fitted, and the largest budget whose predicted peak
stays below a safety fraction of the device memory is chosen and verified once.  Results
are cached in a JSONL file keyed by model / precision / GPU; rank 0 searches and the other
ranks read the cache after a barrier.
"""

from __future__ import annotations

import gc
import json
from pathlib import Path
from typing import Any, Optional

import torch
import torch.distributed as dist

from ..config.config import IndexConfig
from ..gradients import GradientProcessor

SAFETY_FRACTION = 0.85
CACHE_NAME = "batch_size_cache.jsonl"


def _clear() -> None:
    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.empty_cache()


def _shape_for(model, token_budget: int) -> tuple[int, int]:
    max_len = getattr(model.config, "max_position_embeddings", None) or token_budget
    seq = min(token_budget, max_len)
    return max(1, token_budget // seq), seq


def _fwd_bwd(model, token_budget: int, collector=None) -> None:
    from contextlib import nullcontext

    device = next(model.parameters()).device
    n, s = _shape_for(model, token_budget)
    x = torch.randint(0, 10, (n, s), device=device)
    y = torch.randint(0, 10, (n, s), device=device)
    if collector is not None and hasattr(collector, "begin_fused_batch"):
        collector.begin_fused_batch(n, device)
    with collector if collector is not None else nullcontext():
        logits = model(x).logits
        loss = torch.nn.functional.cross_entropy(logits[:, :-1].reshape(-1, logits.size(-1)).float(), y[:, 1:].reshape(-1))
        loss.backward()
    model.zero_grad(set_to_none=True)
    if collector is not None:
        collector.mod_grads.clear()


def test_fwd_bwd(model, token_batch_size: int) -> None:
    """One worst-case forward/backward at ``token_batch_size`` (CUDA only); raises a
    descriptive out-of-memory error if the configured size does not fit."""
    if next(model.parameters()).device.type != "cuda":
        return
    _clear()
    try:
        _fwd_bwd(model, token_batch_size)
    except torch.cuda.OutOfMemoryError as e:
        n, s = _shape_for(model, token_batch_size)
        raise torch.cuda.OutOfMemoryError(
            f"Pre-flight memory check failed for token_batch_size={token_batch_size} ({n} x {s}). "
            f"Lower --token_batch_size and retry. Underlying error: {e}") from e
    finally:
        model.zero_grad(set_to_none=True)
        _clear()


test_fwd_bwd.__test__ = False  # not a pytest test


def _get_system_metadata(cfg: IndexConfig) -> dict[str, Any]:
    name, mem = "cpu", 0.0
    if torch.cuda.is_available():
        name = torch.cuda.get_device_name(0)
        mem = torch.cuda.get_device_properties(0).total_memory / 1e9
    return {"model": cfg.model, "fsdp": cfg.fsdp, "precision": cfg.precision, "projection_dim": cfg.projection_dim,
            "reshape_to_square": cfg.reshape_to_square, "gpu_name": name, "gpu_memory_gb": round(mem, 1)}


def _check_cache(cache_file: Path, meta: dict[str, Any]) -> Optional[int]:
    if not cache_file.exists():
        return None
    try:
        for line in cache_file.read_text().splitlines():
            try:
                row = json.loads(line)
            except json.JSONDecodeError:
                continue
            if all(row.get(k) == v for k, v in meta.items()):
                return row.get("token_batch_size")
    except OSError:
        return None
    return None


def _append_to_cache(cache_file: Path, meta: dict[str, Any], batch_size: int) -> None:
    cache_file.parent.mkdir(parents=True, exist_ok=True)
    with open(cache_file, "a") as f:
        f.write(json.dumps({**meta, "token_batch_size": batch_size}) + "\n")
    print(f"Cached batch size {batch_size} to {cache_file}")


def _measure_peak(model, tokens: int, collector) -> int:
    _clear()
    dev = next(model.parameters()).device
    torch.cuda.reset_peak_memory_stats(dev)
    _fwd_bwd(model, tokens, collector)
    torch.cuda.synchronize(dev)
    peak = torch.cuda.max_memory_allocated(dev)
    _clear()
    return peak


def predict_batch_size(peak_a: int, tokens_a: int, peak_b: int, tokens_b: int, budget_bytes: float,
                       granularity: int = 256, max_tokens: int | None = None) -> int:
    """Largest multiple of ``granularity`` tokens whose predicted peak fits ``budget_bytes``
    under the line through the two measurements."""
    per_token = max((peak_b - peak_a) / max(tokens_b - tokens_a, 1), 1.0)
    base = peak_a - per_token * tokens_a
    tokens = int((budget_bytes - base) / per_token)
    if max_tokens is not None:
        tokens = min(tokens, max_tokens)
    return max(granularity, tokens // granularity * granularity)


def determine_batch_size(root: Path, cfg: IndexConfig, model, collector, starting_batch_size: int = 8192) -> int:
    cache = Path(root) / CACHE_NAME
    meta = _get_system_metadata(cfg)
    cached = _check_cache(cache, meta)
    if cached is not None:
        print(f"Loaded token_batch_size from cache: {cached}")
        return cached
    dev = next(model.parameters()).device
    if dev.type != "cuda":
        return starting_batch_size
    print("Determining token batch size from measured memory use...")
    small = max(256, min(starting_batch_size // 4, 2048))
    big = 2 * small
    pa, pb = _measure_peak(model, small, collector), _measure_peak(model, big, collector)
    total = torch.cuda.get_device_properties(dev).total_memory
    chosen = predict_batch_size(pa, small, pb, big, SAFETY_FRACTION * total, max_tokens=1 << 20)
    print(f"  peak {pa / 1e9:.2f} GB @ {small} tokens, {pb / 1e9:.2f} GB @ {big} tokens -> {chosen} tokens")
    _append_to_cache(cache, meta, chosen)
    return chosen


def maybe_auto_batch_size(cfg: IndexConfig, model, ds, processor: GradientProcessor, target_modules, rank: int = 0) -> None:
    """Sets ``cfg.token_batch_size`` in place when ``cfg.auto_batch_size``."""
    if not cfg.auto_batch_size:
        return
    from ..collector.gradient_collectors import GradientCollector

    group = dist.new_group(backend="gloo") if dist.is_initialized() else None
    if rank == 0:
        collector = GradientCollector(model=model.base_model, cfg=cfg, processor=processor,
                                      target_modules=target_modules, data=ds, skip_index=True)
        cfg.token_batch_size = determine_batch_size(Path(".cache"), cfg, model, collector, cfg.token_batch_size)
    if group is not None:
        dist.barrier(group=group)
        dist.destroy_process_group(group)
        if rank != 0:
            cached = _check_cache(Path(".cache") / CACHE_NAME, _get_system_metadata(cfg))
            assert cached is not None, "Cache missing after barrier"
            cfg.token_batch_size = cached
