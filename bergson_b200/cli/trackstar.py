"""TrackStar pipeline: value Hessian -> query Hessian -> mix -> query build -> score
(reference ``bergson/cli/trackstar.py:43-176``)."""

from __future__ import annotations

from copy import deepcopy
from pathlib import Path

from ..build import build
from ..config.config import HessianConfig, IndexConfig, TrackstarConfig
from ..config.config_io import save_run_config
from ..distributed import parent_barrier
from ..hessians.hessian_approximations import approximate_hessians
from ..process_grads import mix_autocorrelation_matrices
from ..score.score import score_dataset
from ..utils.worker_utils import validate_run_path


def _limit_split_for_hess(cfg: IndexConfig, n: int | None) -> None:
    """Restrict the split to its first ``n`` rows for Hessian fitting."""
    if n is not None:
        cfg.data.split = f"{cfg.data.split.split('[')[0]}[:{n}]"


def _step_complete(path: str, resume: bool) -> bool:
    if resume and Path(path).exists():
        print(f"  Skipping (output exists at {path})")
        return True
    return False


def trackstar(index_cfg: IndexConfig, trackstar_cfg: TrackstarConfig):
    from .commands import Build, Hessian, Mix, Score

    if index_cfg.projection_dim == 0:
        raise ValueError("Trackstar scores via compressed random-projected gradients and requires a nonzero "
                         "index_cfg.projection_dim; got 0.")
    run = index_cfg.run_path
    value_h, query_h, mixed_h = f"{run}/value_hessian", f"{run}/query_hessian", f"{run}/mixed_hessian"
    query_path, scores_path = f"{run}/query", f"{run}/scores"
    resume = trackstar_cfg.resume
    hess_cfg = HessianConfig(method="autocorrelation")

    def validate(cfg: IndexConfig):
        if not (resume and cfg.partial_run_path.exists()):
            validate_run_path(cfg)

    print("Step 1/5: Computing hessians on value dataset...")
    if not _step_complete(value_h, resume):
        c = deepcopy(index_cfg)
        c.run_path = value_h
        _limit_split_for_hess(c, trackstar_cfg.stats_sample_size)
        validate(c)
        save_run_config(Hessian(hessian_cfg=hess_cfg, index_cfg=c), c.partial_run_path)
        approximate_hessians(c, hess_cfg)

    if not trackstar_cfg.mix_hessians:
        print("Steps 2-3/5: Skipped (mix_hessians=false); using the value hessian.")
        pre_path = value_h
    else:
        print("Step 2/5: Computing hessians on query dataset...")
        if not _step_complete(query_h, resume):
            c = deepcopy(index_cfg)
            c.run_path, c.data = query_h, deepcopy(trackstar_cfg.query)
            _limit_split_for_hess(c, trackstar_cfg.stats_sample_size)
            validate(c)
            save_run_config(Hessian(hessian_cfg=hess_cfg, index_cfg=c), c.partial_run_path)
            approximate_hessians(c, hess_cfg)
        print("Step 3/5: Mixing hessians...")
        if not _step_complete(mixed_h, resume) and index_cfg.distributed._node_rank == 0:
            k = trackstar_cfg.target_downweight_components
            save_run_config(Mix(query_path=query_h, index_path=value_h, output_path=mixed_h,
                                target_downweight_components=k), mixed_h)
            mix_autocorrelation_matrices(query_h, value_h, mixed_h, k)
        pre_path = mixed_h
    parent_barrier(index_cfg.distributed)
    trackstar_cfg.preprocess_cfg.hessian_path = pre_path

    print("Step 4/5: Building query gradient index...")
    if not _step_complete(query_path, resume):
        c = deepcopy(index_cfg)
        c.run_path, c.data = query_path, deepcopy(trackstar_cfg.query)
        if trackstar_cfg.preprocess_cfg.aggregation != "none" and c.attribute_tokens:
            print("Query aggregation is not compatible with query-side token attribution; "
                  "query gradients are collected per sequence.")
            c.attribute_tokens = False
        validate(c)
        save_run_config(Build(c, trackstar_cfg.preprocess_cfg), c.partial_run_path)
        build(c, trackstar_cfg.preprocess_cfg)

    print("Step 5/5: Scoring value dataset...")
    if not _step_complete(scores_path, resume):
        c = deepcopy(index_cfg)
        c.run_path = scores_path
        trackstar_cfg.score_cfg.query_path = query_path
        trackstar_cfg.score_cfg.higher_is_better = True
        validate(c)
        save_run_config(Score(trackstar_cfg.score_cfg, c, trackstar_cfg.preprocess_cfg), c.partial_run_path)
        score_dataset(c, trackstar_cfg.score_cfg, trackstar_cfg.preprocess_cfg)
