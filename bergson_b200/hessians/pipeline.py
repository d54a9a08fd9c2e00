"""EK-FAC influence pipeline.

Four steps under one run directory, each restartable (``.part`` / promote protocol):

====================  ===================================================================
``query/``            gradient(s) of the query set at full resolution (projection 0),
                      aggregated as ``query_aggregation`` says
``hessian/<method>``  Kronecker factors of the training set, their eigendecomposition and
                      (EK-FAC) the corrected eigenvalues
``<method>_query/``   the query gradient(s) multiplied by the inverse of that Hessian
``scores/``           inner products of every training example's gradient with them
====================  ===================================================================
"""

from __future__ import annotations

from ..build import build
from ..cli.steps import Step, StepRunner, derive
from ..config.config import HessianConfig, HessianPipelineConfig, IndexConfig, PreprocessConfig, ScoreConfig
from ..config.config_io import save_run_config
from ..distributed import launch_distributed_run
from ..score.score import score_dataset
from .apply_hessian import EkfacConfig, apply_worker
from .hessian_approximations import approximate_hessians


def hessian_pipeline(index_cfg: IndexConfig, hessian_cfg: HessianConfig, score_cfg: ScoreConfig,
                     preprocess_cfg: PreprocessConfig, hessian_pipeline_cfg: HessianPipelineConfig):
    from ..cli.commands import Build, Score

    if preprocess_cfg.unit_normalize:
        raise ValueError("preprocess_cfg.unit_normalize (cosine similarity) is not supported with "
                         "Kronecker-factored Hessians.")
    root, method = index_cfg.run_path, hessian_cfg.method
    out = {"query": f"{root}/query", "hessian": f"{root}/hessian", "ivhp": f"{root}/{method}_query",
           "scores": f"{root}/scores"}
    factors = f"{out['hessian']}/{method}"
    runner = StepRunner(resume=hessian_pipeline_cfg.resume, protocol="promote")

    def build_query():
        cfg = derive(index_cfg, run_path=out["query"], data=hessian_pipeline_cfg.query, projection_dim=0)
        runner.check_run_path(cfg)
        pre = PreprocessConfig(aggregation=hessian_pipeline_cfg.query_aggregation)
        save_run_config(Build(cfg, pre), cfg.partial_run_path)
        build(cfg, pre)

    def fit_factors():
        cfg = derive(index_cfg, run_path=factors)
        runner.check_run_path(cfg)
        approximate_hessians(cfg, hessian_cfg)

    def apply_inverse():
        ecfg = EkfacConfig(hessian_method_path=factors, gradient_path=out["query"], run_path=out["ivhp"],
                           ev_correction=hessian_cfg.ev_correction, projection_dim=index_cfg.projection_dim,
                           projection_type=index_cfg.projection_type)
        launch_distributed_run("apply_hessian", apply_worker, [ecfg, hessian_pipeline_cfg.inversion_cfg],
                               index_cfg.distributed)

    def score():
        cfg = derive(index_cfg, run_path=out["scores"])
        score_cfg.query_path, score_cfg.higher_is_better = out["ivhp"], True
        runner.check_run_path(cfg)
        save_run_config(Score(score_cfg, cfg, preprocess_cfg), cfg.partial_run_path)
        score_dataset(cfg, score_cfg, preprocess_cfg)

    timings = runner.run([
        Step(f"query gradient(s), aggregation={hessian_pipeline_cfg.query_aggregation}", out["query"], build_query,
             key="step1_build_query"),
        Step(f"{method} factors of the training data", out["hessian"], fit_factors, key="step2_fit_hessian"),
        Step(f"inverse {method} Hessian applied to the query gradient(s)", out["ivhp"], apply_inverse, key="step3_apply"),
        Step("training data scored against the transformed query", out["scores"], score, key="step4_score"),
    ])
    print(f"EK-FAC pipeline finished; scores at {out['scores']}")
    if timings:
        print(f"seconds per step: {timings} (total {sum(timings.values()):.1f})")
    return timings
