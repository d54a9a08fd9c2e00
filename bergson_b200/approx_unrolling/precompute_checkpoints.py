"""Per-checkpoint passes of SOURCE: raw Kronecker covariances at every checkpoint and,
once the segment eigenbasis exists, eigenvalue corrections in that basis
(reference ``bergson/approx_unrolling/precompute_checkpoints.py``).  Checkpoint c of
segment l writes to ``<run>/segment_{l}/ckpt_{i}/<method>/``."""

from __future__ import annotations

import shutil
from copy import deepcopy
from pathlib import Path

import torch
from datasets import Dataset

from ..collector.collector import CollectorComputer, fwd_bwd_hessian_factory
from ..config import ApproxUnrollingConfig, HessianConfig, IndexConfig
from ..data import allocate_batches
from ..distributed import init_dist, launch_distributed_run
from ..hessians.eigenvectors import LambdaCollector
from ..hessians.hessian_approximations import approximate_hessians
from ..utils.logger import get_logger
from ..utils.utils import convert_precision_to_torch
from ..utils.worker_utils import setup_data_pipeline, setup_model_and_peft

DOCUMENTS_PROCESSED_FILENAME = "documents_processed.pt"


def _placement(c: int, per_segment: int) -> tuple[int, int]:
    return c // per_segment, c % per_segment


def precompute_checkpoint_hessians(index_cfg: IndexConfig, hessian_cfg: HessianConfig,
                                   approx_unrolling_cfg: ApproxUnrollingConfig, *, overwrite: bool = False) -> None:
    """One covariance pass (no eigendecomposition, no correction) per checkpoint."""
    log = get_logger("precompute_checkpoint_hessians")
    base, method = Path(index_cfg.run_path), hessian_cfg.method
    per = len(approx_unrolling_cfg.checkpoints) // approx_unrolling_cfg.segments
    for c, ckpt in enumerate(map(str, approx_unrolling_cfg.checkpoints)):
        seg, i = _placement(c, per)
        out = base / f"segment_{seg}" / f"ckpt_{i}" / method
        if out.exists():
            if not overwrite:
                log.info(f"[seg {seg} ckpt {i}] skip - exists at {out}")
                continue
            shutil.rmtree(out)
        log.info(f"[seg {seg} ckpt {i}] computing {method} at model={ckpt!r}")
        icfg = deepcopy(index_cfg)
        icfg.run_path, icfg.model = str(out), ckpt
        hcfg = deepcopy(hessian_cfg)
        hcfg.ev_correction = False
        approximate_hessians(icfg, hcfg, do_eigendecomposition=False)


def _lambda_worker(rank, local_rank, world_size, index_cfg: IndexConfig, hessian_cfg: HessianConfig, ds: Dataset,
                   output_dir: Path, eigen_path: Path, output_subdir: str) -> None:
    init_dist(rank, local_rank, world_size)
    model, targets = setup_model_and_peft(index_cfg)
    batches = allocate_batches(ds["length"][:], index_cfg.token_batch_size)
    output_dir.mkdir(parents=True, exist_ok=True)
    collector = LambdaCollector(
        model=model.base_model, target_modules=targets,
        attention_cfgs={m: index_cfg.attention for m in index_cfg.split_attention_modules}, path=str(output_dir),
        eigen_path=str(eigen_path), output_subdir=output_subdir, filter_modules=index_cfg.filter_modules,
        dtype=convert_precision_to_torch(hessian_cfg.hessian_dtype))
    computer = CollectorComputer(model=model, data=ds, collector=collector, batches=batches, cfg=index_cfg)
    computer.forward_backward = fwd_bwd_hessian_factory(index_cfg, hessian_cfg)
    computer.run_with_collector_hooks(desc=f"Lambda -> {output_dir}")


def precompute_checkpoint_averaged_lambdas(index_cfg: IndexConfig, hessian_cfg: HessianConfig,
                                           approx_unrolling_cfg: ApproxUnrollingConfig, *, resume: bool = False,
                                           output_subdir: str = "averaged_ev_correct_sharded") -> None:
    """Eigenvalue correction of every checkpoint in its segment's eigenbasis, plus the number
    of documents it covers (the divisor of the later segment average)."""
    log = get_logger("precompute_checkpoint_averaged_lambdas")
    base, method = Path(index_cfg.run_path), hessian_cfg.method
    per = len(approx_unrolling_cfg.checkpoints) // approx_unrolling_cfg.segments
    for c, ckpt in enumerate(map(str, approx_unrolling_cfg.checkpoints)):
        seg, i = _placement(c, per)
        ckpt_dir = base / f"segment_{seg}" / f"ckpt_{i}" / method
        eigen = base / f"segment_{seg}" / method
        out = ckpt_dir / output_subdir
        if out.exists():
            if resume:
                log.info(f"[seg {seg} ckpt {i}] skip - exists at {out}")
                continue
            shutil.rmtree(out)
        if not eigen.exists():
            raise FileNotFoundError(f"Missing segment eigvec dir {eigen}; did the aggregation step finish?")
        icfg = deepcopy(index_cfg)
        icfg.model, icfg.run_path = ckpt, str(ckpt_dir)
        icfg.partial_run_path.mkdir(parents=True, exist_ok=True)
        ds, _ = setup_data_pipeline(icfg)
        launch_distributed_run("checkpoint_averaged_lambda", _lambda_worker,
                               [icfg, hessian_cfg, ds, ckpt_dir, eigen, output_subdir], icfg.distributed)
        torch.save(torch.tensor(len(ds)), out / DOCUMENTS_PROCESSED_FILENAME)
        shutil.rmtree(icfg.partial_run_path, ignore_errors=True)
