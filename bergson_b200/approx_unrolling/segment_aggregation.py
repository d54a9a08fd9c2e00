"""Per-segment aggregation for SOURCE: covariances of a segment's checkpoints are summed
and eigendecomposed; per-checkpoint eigenvalue corrections are pooled into a per-document
average (reference ``bergson/approx_unrolling/segment_aggregation.py``)."""

from __future__ import annotations

from pathlib import Path

import torch
import torch.distributed as dist
from safetensors import safe_open

from ..config import DistributedConfig
from ..distributed import init_dist, launch_distributed_run
from ..hessians.eigenvectors import compute_eigendecomposition
from ..utils.logger import get_logger
from ..utils.step_state import partial_path, prepare_step, promote_step
from ..utils.streamed_safetensors import save_tensors
from ..utils.utils import get_device
from .precompute_checkpoints import DOCUMENTS_PROCESSED_FILENAME

_SHARD_KINDS = ("activation_sharded", "gradient_sharded")


def lambda_denominator(input_dirs: list[Path]) -> float:
    """Documents pooled over a segment's checkpoints."""
    total = 0
    for d in input_dirs:
        p = d / DOCUMENTS_PROCESSED_FILENAME
        if not p.exists():
            raise FileNotFoundError(f"Missing {p}; re-run the per-checkpoint lambda step.")
        total += int(torch.load(p, map_location="cpu", weights_only=False))
    return float(total)


def _sum_my_shard(in_paths: list[Path], out_path: Path, device: str, divisor: float = 1.0) -> None:
    acc: dict[str, torch.Tensor] = {}
    for p in in_paths:
        with safe_open(str(p), framework="pt", device=device) as f:
            for k in f.keys():
                t = f.get_tensor(k)
                acc[k] = t.clone() if k not in acc else acc[k].add_(t)
    if divisor != 1.0:
        for v in acc.values():
            v.div_(divisor)
    out_path.parent.mkdir(parents=True, exist_ok=True)
    save_tensors(acc, str(out_path))  # straight from the device when the sums live there


def _sum_dirs_worker(rank, local_rank, world_size, input_dirs: list[Path], output_dir: Path, divisor: float) -> None:
    init_dist(rank, local_rank, world_size)
    name = f"shard_{rank}.safetensors"
    _sum_my_shard([d / name for d in input_dirs], output_dir / name, get_device(local_rank), divisor)
    if world_size > 1:
        dist.barrier()


def sum_sharded_dirs(input_dirs: list[Path], output_dir: Path, distributed: DistributedConfig, divisor: float = 1.0):
    output_dir.mkdir(parents=True, exist_ok=True)
    launch_distributed_run("sum_sharded_dirs", _sum_dirs_worker, [input_dirs, output_dir, divisor], distributed)


def _aggregate_cov_worker(rank, local_rank, world_size, base_run: Path, method: str, per_segment: int,
                          segments: list[int]) -> None:
    init_dist(rank, local_rank, world_size)
    device, name = get_device(local_rank), f"shard_{rank}.safetensors"
    for seg in segments:
        seg_dir = base_run / f"segment_{seg}"
        out = seg_dir / method
        part = partial_path(out)
        srcs = [seg_dir / f"ckpt_{i}" / method for i in range(per_segment)]
        for kind in _SHARD_KINDS:
            _sum_my_shard([d / kind / name for d in srcs], part / kind / name, device)
        if rank == 0:
            total = sum(torch.load(d / "total_processed.pt", map_location="cpu", weights_only=False) for d in srcs)
            torch.save(total, part / "total_processed.pt")
        if world_size > 1:
            dist.barrier()
        total = torch.load(part / "total_processed.pt", map_location="cpu", weights_only=False)
        for kind in _SHARD_KINDS:
            compute_eigendecomposition(str(part / kind), total_processed=total)
        if world_size > 1:
            dist.barrier()
        if rank == 0:
            promote_step(out)
        if world_size > 1:
            dist.barrier()


def aggregate_segment_covariances(run_path, method: str, n_segments: int, per_segment: int,
                                  distributed: DistributedConfig, *, resume: bool = False) -> None:
    """``<run>/segment_l/<method>/{activation,gradient}_sharded`` = sum over the segment's
    checkpoints, plus their eigenvector shards and the summed ``total_processed.pt``."""
    log = get_logger("aggregate_segment_covariances")
    base = Path(run_path)
    todo = []
    for seg in range(n_segments):
        out = base / f"segment_{seg}" / method
        if not prepare_step(out, resume=resume):
            log.info(f"[seg {seg}] skip - already complete at {out}")
            continue
        for i in range(per_segment):
            d = base / f"segment_{seg}" / f"ckpt_{i}" / method
            if not d.exists():
                raise FileNotFoundError(f"Expected per-checkpoint covariance dir {d} not found.")
        todo.append(seg)
    if todo:
        launch_distributed_run("aggregate_segment_covariances", _aggregate_cov_worker,
                               [base, method, per_segment, todo], distributed)


def aggregate_segment_lambdas(run_path, method: str, n_segments: int, per_segment: int, distributed: DistributedConfig,
                              *, resume: bool = False, input_subdir: str = "averaged_ev_correct_sharded",
                              output_subdir: str = "eigenvalue_correction_sharded") -> None:
    """Per-document mean of the per-checkpoint corrections of each segment."""
    log = get_logger("aggregate_segment_lambdas")
    base = Path(run_path)
    for seg in range(n_segments):
        out = base / f"segment_{seg}" / method / output_subdir
        if not prepare_step(out, resume=resume):
            log.info(f"[seg {seg}] skip - already complete at {out}")
            continue
        srcs = [base / f"segment_{seg}" / f"ckpt_{i}" / method / input_subdir for i in range(per_segment)]
        for d in srcs:
            if not d.exists():
                raise FileNotFoundError(f"Missing per-ckpt lambda dir {d}; did the lambda step finish?")
        sum_sharded_dirs(srcs, partial_path(out), distributed, divisor=lambda_denominator(srcs))
        promote_step(out)
