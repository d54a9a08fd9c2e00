"""TrackStar pipeline: gradient-similarity attribution with the gradients of both sides
whitened by a mixture of the training ("value") and query autocorrelation Hessians.

Outputs under the run directory: ``value_hessian/``, ``query_hessian/``, ``mixed_hessian/``
(the latter two only when ``mix_hessians``), ``query/`` (preconditioned query gradients) and
``scores/``.  With ``resume`` a step whose output directory exists is not repeated.
"""

from __future__ import annotations

from ..build import build
from ..config.config import HessianConfig, IndexConfig, TrackstarConfig
from ..config.config_io import save_run_config
from ..distributed import parent_barrier
from ..hessians.hessian_approximations import approximate_hessians
from ..process_grads import mix_autocorrelation_matrices
from ..score.score import score_dataset
from .steps import Step, StepRunner, derive


def _head_of_split(split: str, n: int | None) -> str:
    """``split`` restricted to its first ``n`` rows (any earlier slice is replaced)."""
    return split if n is None else f"{split.partition('[')[0]}[:{n}]"


def trackstar(index_cfg: IndexConfig, trackstar_cfg: TrackstarConfig):
    from .commands import Build, Hessian, Mix, Score

    if index_cfg.projection_dim == 0:
        raise ValueError("Trackstar scores via compressed random-projected gradients and requires a nonzero "
                         "index_cfg.projection_dim; got 0.")
    root = index_cfg.run_path
    out = {k: f"{root}/{k}" for k in ("value_hessian", "query_hessian", "mixed_hessian", "query", "scores")}
    tc = trackstar_cfg
    runner = StepRunner(resume=tc.resume, protocol="exists")
    autocorr = HessianConfig(method="autocorrelation")
    mixing = tc.mix_hessians
    # Every later step whitens with the mixed Hessian, or with the value Hessian alone.
    tc.preprocess_cfg.hessian_path = out["mixed_hessian"] if mixing else out["value_hessian"]

    def fit_autocorrelation(where: str, data):
        def action():
            cfg = derive(index_cfg, run_path=where, data=data)
            cfg.data.split = _head_of_split(cfg.data.split, tc.stats_sample_size)
            runner.check_run_path(cfg)
            save_run_config(Hessian(hessian_cfg=autocorr, index_cfg=cfg), cfg.partial_run_path)
            approximate_hessians(cfg, autocorr)
        return action

    def mix():
        if index_cfg.distributed._node_rank == 0:
            k = tc.target_downweight_components
            save_run_config(Mix(query_path=out["query_hessian"], index_path=out["value_hessian"],
                                output_path=out["mixed_hessian"], target_downweight_components=k), out["mixed_hessian"])
            mix_autocorrelation_matrices(out["query_hessian"], out["value_hessian"], out["mixed_hessian"], k)
        parent_barrier(index_cfg.distributed)

    def build_query():
        cfg = derive(index_cfg, run_path=out["query"], data=tc.query)
        if tc.preprocess_cfg.aggregation != "none" and cfg.attribute_tokens:
            print("  aggregated queries are per sequence: token attribution is switched off on the query side")
            cfg.attribute_tokens = False
        runner.check_run_path(cfg)
        save_run_config(Build(cfg, tc.preprocess_cfg), cfg.partial_run_path)
        build(cfg, tc.preprocess_cfg)

    def score():
        cfg = derive(index_cfg, run_path=out["scores"])
        tc.score_cfg.query_path, tc.score_cfg.higher_is_better = out["query"], True
        runner.check_run_path(cfg)
        save_run_config(Score(tc.score_cfg, cfg, tc.preprocess_cfg), cfg.partial_run_path)
        score_dataset(cfg, tc.score_cfg, tc.preprocess_cfg)

    note = "mix_hessians=false: the value Hessian is used alone"
    return runner.run([
        Step("autocorrelation Hessian of the value data", out["value_hessian"],
             fit_autocorrelation(out["value_hessian"], index_cfg.data)),
        Step("autocorrelation Hessian of the query data", out["query_hessian"],
             fit_autocorrelation(out["query_hessian"], tc.query), enabled=mixing, skip_note=note),
        Step("mixture of the two Hessians", out["mixed_hessian"], mix, enabled=mixing, skip_note=note),
        Step("query gradient index", out["query"], build_query),
        Step("value data scored against the queries", out["scores"], score),
    ])
