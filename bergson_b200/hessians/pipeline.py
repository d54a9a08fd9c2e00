"""EK-FAC influence pipeline: query build -> factor fit -> inverse-Hessian apply -> score
(reference ``bergson/hessians/pipeline.py:46-150``)."""

from __future__ import annotations

import time
from contextlib import contextmanager
from copy import deepcopy

from ..build import build
from ..config.config import HessianConfig, HessianPipelineConfig, IndexConfig, PreprocessConfig, ScoreConfig
from ..config.config_io import save_run_config
from ..distributed import launch_distributed_run
from ..score.score import score_dataset
from ..utils.step_state import prepare_step
from ..utils.worker_utils import validate_run_path
from .apply_hessian import EkfacConfig, apply_worker
from .hessian_approximations import approximate_hessians


def _step_complete(path: str, resume: bool) -> bool:
    if prepare_step(path, resume=resume):
        return False
    print(f"  Skipping (already complete at {path})")
    return True


@contextmanager
def _timed(label: str, durations: dict[str, float]):
    t0 = time.perf_counter()
    try:
        yield
    finally:
        durations[label] = time.perf_counter() - t0
        print(f"  [{label}] took {durations[label]:.1f}s")


def hessian_pipeline(index_cfg: IndexConfig, hessian_cfg: HessianConfig, score_cfg: ScoreConfig,
                     preprocess_cfg: PreprocessConfig, hessian_pipeline_cfg: HessianPipelineConfig):
    from ..cli.commands import Build, Score

    if preprocess_cfg.unit_normalize:
        raise ValueError("preprocess_cfg.unit_normalize (cosine similarity) is not supported with "
                         "Kronecker-factored Hessians.")
    run, method = index_cfg.run_path, hessian_cfg.method
    query_path, hessian_path = f"{run}/query", f"{run}/hessian"
    transformed, scores_path = f"{run}/{method}_query", f"{run}/scores"
    resume = hessian_pipeline_cfg.resume
    durations: dict[str, float] = {}

    def validate(cfg: IndexConfig):
        if not (resume and cfg.partial_run_path.exists()):
            validate_run_path(cfg)

    agg = hessian_pipeline_cfg.query_aggregation
    print(f"Step 1/4: Building query gradient(s) (aggregation={agg})...")
    if not _step_complete(query_path, resume):
        with _timed("step1_build_query", durations):
            qcfg = deepcopy(index_cfg)
            qcfg.run_path, qcfg.data, qcfg.projection_dim = query_path, hessian_pipeline_cfg.query, 0
            validate(qcfg)
            qpre = PreprocessConfig(aggregation=agg)
            save_run_config(Build(qcfg, qpre), qcfg.partial_run_path)
            build(qcfg, qpre)

    print(f"Step 2/4: Fitting {method} factors on training data...")
    if not _step_complete(hessian_path, resume):
        with _timed("step2_fit_hessian", durations):
            hcfg = deepcopy(index_cfg)
            hcfg.run_path = f"{hessian_path}/{method}"
            validate(hcfg)
            approximate_hessians(hcfg, hessian_cfg)

    print(f"Step 3/4: Applying {method} inverse Hessian to the query gradient(s)...")
    if not _step_complete(transformed, resume):
        with _timed("step3_apply", durations):
            ecfg = EkfacConfig(
                hessian_method_path=f"{hessian_path}/{method}", gradient_path=query_path, run_path=transformed,
                ev_correction=hessian_cfg.ev_correction, projection_dim=index_cfg.projection_dim,
                projection_type=index_cfg.projection_type,
            )
            launch_distributed_run("apply_hessian", apply_worker, [ecfg, hessian_pipeline_cfg.inversion_cfg],
                                   index_cfg.distributed)

    print("Step 4/4: Scoring training data against transformed query...")
    if not _step_complete(scores_path, resume):
        with _timed("step4_score", durations):
            scfg = deepcopy(index_cfg)
            scfg.run_path = scores_path
            score_cfg.query_path = transformed
            score_cfg.higher_is_better = True
            validate(scfg)
            save_run_config(Score(score_cfg, scfg, preprocess_cfg), scfg.partial_run_path)
            score_dataset(scfg, score_cfg, preprocess_cfg)
    print(f"Done! Scores saved to: {scores_path}")
    if durations:
        print(f"Step timings (s): {durations} | total {sum(durations.values()):.1f}s")
    return durations
