"""SOURCE pipeline (reference ``bergson/approx_unrolling/pipeline.py:67-291``):

1. K-FAC covariances at every checkpoint.              -> segment_l/ckpt_i/<method>/
2. Per-segment covariance sums + eigendecomposition.   -> segment_l/<method>/
3. Per-checkpoint eigenvalue correction in the segment basis.
4. Per-segment averaged correction.                    -> .../eigenvalue_correction_sharded/
5. Query gradient at the last checkpoint.              -> query/
6. Backward walk of the query through the segments.    -> segment_l/query_grad_backward/
7. Segment responses.                                  -> segment_l/query_grad_segment/
8. Per-checkpoint scores, averaged per segment, summed -> scores/
"""

from __future__ import annotations

import gc
import shutil
from copy import deepcopy
from pathlib import Path

from ..build import build
from ..config import ApproxUnrollingConfig, HessianConfig, IndexConfig, PreprocessConfig
from ..config.config_io import save_run_config
from ..distributed import parent_barrier
from ..utils.logger import get_logger
from .adam_preconditioner import OPTIMIZER_STATE_FILE, build_segment_preconditioners
from .approx_unrolling_math import (
    compute_lr_times_steps_per_segment,
    score_per_segment_and_aggregate,
    walk_query_phase1,
    walk_query_phase2,
)
from .precompute_checkpoints import precompute_checkpoint_averaged_lambdas, precompute_checkpoint_hessians
from .segment_aggregation import aggregate_segment_covariances, aggregate_segment_lambdas
from .train_cfg_io import resolve


def approx_unrolling_pipeline(index_cfg: IndexConfig, hessian_cfg: HessianConfig, cfg: ApproxUnrollingConfig):
    from ..cli.commands import Build

    log = get_logger("approx_unrolling_pipeline")
    cfg = resolve(cfg)
    n, L = len(cfg.checkpoints), cfg.segments
    if n == 0:
        raise ValueError("approx_unrolling_cfg.checkpoints is empty.")
    if L < 1:
        raise ValueError(f"approx_unrolling_cfg.segments must be >= 1, got {L}.")
    if n % L != 0:
        raise ValueError(f"checkpoints ({n}) must be divisible by segments ({L}).")
    assert hessian_cfg.ev_correction, "The approximate unrolling pipeline needs ev_correction=True."
    if cfg.use_adam_preconditioner:
        for c in cfg.checkpoints:
            if not (Path(c) / OPTIMIZER_STATE_FILE).exists():
                raise FileNotFoundError(f"use_adam_preconditioner requires {Path(c) / OPTIMIZER_STATE_FILE}; write it "
                                        "during training with TrainingConfig.save_optimizer_state.")
    lr_k = compute_lr_times_steps_per_segment(cfg)
    per, run, method = n // L, index_cfg.run_path, hessian_cfg.method
    resume = not index_cfg.overwrite
    log.info(f"SOURCE pipeline -> {run}: {n} checkpoints, {L} segments, method {method}, eta*K {lr_k}")

    log.info("Step 1/8: covariances at each checkpoint")
    precompute_checkpoint_hessians(index_cfg, hessian_cfg, cfg, overwrite=index_cfg.overwrite)
    gc.collect()
    log.info("Step 2/8: segment covariance sums and eigendecomposition")
    aggregate_segment_covariances(run, method, L, per, index_cfg.distributed, resume=resume)
    log.info("Step 3/8: per-checkpoint eigenvalue corrections in the segment basis")
    precompute_checkpoint_averaged_lambdas(index_cfg, hessian_cfg, cfg, resume=resume)
    log.info("Step 4/8: segment eigenvalue corrections")
    aggregate_segment_lambdas(run, method, L, per, index_cfg.distributed, resume=resume)

    log.info("Step 5/8: query gradient at the final checkpoint")
    query_path = Path(run) / "query"
    if resume and query_path.exists():
        log.info(f"  skip - exists at {query_path}")
    else:
        if query_path.exists():
            shutil.rmtree(query_path)
        qcfg = deepcopy(index_cfg)
        qcfg.model, qcfg.data, qcfg.run_path, qcfg.projection_dim = str(cfg.checkpoints[-1]), cfg.query, str(query_path), 0
        qpre = PreprocessConfig(aggregation=cfg.query_aggregation)
        qcfg.partial_run_path.mkdir(parents=True, exist_ok=True)
        save_run_config(Build(qcfg, qpre), qcfg.partial_run_path)
        build(qcfg, qpre)

    pre_paths: list[Path] = []
    if cfg.use_adam_preconditioner:
        if index_cfg.distributed._node_rank == 0:
            pre_paths = build_segment_preconditioners(run, method, [str(c) for c in cfg.checkpoints], L)
        else:
            pre_paths = [Path(run) / f"segment_{l}" / "preconditioner.safetensors" for l in range(L)]
        parent_barrier(index_cfg.distributed)
    pre = [str(p) for p in pre_paths] or None

    log.info("Step 6/8: backward walk of the query")
    q_paths = walk_query_phase1(run, method, lr_k, index_cfg.distributed, pre, cfg.inversion_cfg)
    log.info("Step 7/8: segment responses")
    r_paths = walk_query_phase2(run, method, lr_k, q_paths, index_cfg.distributed, pre, cfg.inversion_cfg)
    log.info("Step 8/8: scoring and aggregation")
    out = score_per_segment_and_aggregate(
        index_cfg, r_paths, [[str(c) for c in cfg.checkpoints[l * per : (l + 1) * per]] for l in range(L)],
        cfg.query_batch_size)
    log.info(f"SOURCE pipeline done. Final scores at {out}")
    return out
