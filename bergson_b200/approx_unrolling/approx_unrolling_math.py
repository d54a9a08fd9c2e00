"""Math of SOURCE (approximate unrolled differentiation).

Training is cut into L segments.  With ``eta K_l`` the summed learning rate of segment l
(scaled by ``1/(1 - beta)`` under heavy-ball momentum) and ``H_l = Q Lambda_l Q^T`` the
segment's EK-FAC Hessian (reference ``bergson/approx_unrolling/approx_unrolling_math.py``):

* backward walk   ``q_{l-1} = Q f_b(Lambda_l) Q^T q_l``,  ``f_b(s) = exp(-eta K_l s)``
* segment response ``r_l = Q f_s(Lambda_l) Q^T q_l``,      ``f_s(s) = (1 - exp(-eta K_l s)) / s``
  (``eta K_l`` at ``s = 0``; evaluated with ``expm1``)
* score            ``sum_l mean_{c in l} <r_l, grad loss(z; theta_c)>``

Scores are written loss-signed (``higher_is_better = False``).
"""

from __future__ import annotations

import json
import re
import shutil
from copy import deepcopy
from pathlib import Path
from typing import Callable

import numpy as np
import torch
from torch import Tensor

from ..config.config import (
    ApproxUnrollingConfig,
    DistributedConfig,
    IndexConfig,
    InversionConfig,
    PreprocessConfig,
    ScoreConfig,
)
from ..config.config_io import load_subconfig, save_run_config
from ..data import load_scores
from ..distributed import init_dist, launch_distributed_run
from ..hessians.apply_hessian import EkfacApplicator, EkfacConfig
from ..score.score import score_dataset
from ..score.score_writer import save_sequence_scores, save_token_scores

LR_HISTORY_FILENAME = "log_history.json"


def _checkpoint_step(p: str) -> int:
    """Step index from ``checkpoint-<N>``, ``step_<N>[.ckpt]`` or a bare ``<N>`` directory."""
    name = Path(p).name
    for pat in (r"checkpoint-(\d+)$", r"step_(\d+)(?:\.ckpt)?$", r"(\d+)$"):
        if m := re.match(pat, name):
            return int(m.group(1))
    raise ValueError(
        f"Cannot infer a training step from checkpoint {p!r}: expected 'checkpoint-<N>', 'step_<N>[.ckpt]' or "
        "'<N>'. Set `lr_list` and `step_size_list` on ApproxUnrollingConfig instead.")


def compute_lr_times_steps_per_segment(cfg: ApproxUnrollingConfig) -> list[float]:
    """``eta K_l`` per segment: ``lr_list * step_size_list`` when given, else the sum of
    logged per-step learning rates between segment boundaries; times ``1/(1 - momentum)``."""
    from .train_cfg_io import lr_history_path

    momentum = cfg.momentum if cfg.momentum is not None else 0.0
    if not 0.0 <= momentum < 1.0:
        raise ValueError(f"momentum must be in [0, 1), got {momentum}.")
    scale = 1.0 / (1.0 - momentum)
    if cfg.lr_list and cfg.step_size_list:
        return [lr * k * scale for lr, k in zip(cfg.lr_list, cfg.step_size_list)]
    L = cfg.segments
    per = len(cfg.checkpoints) // L
    steps = [_checkpoint_step(p) for p in cfg.checkpoints]
    bounds = [0] + [steps[(l + 1) * per - 1] for l in range(L)]
    log = lr_history_path(cfg.checkpoints) or Path(str(cfg.checkpoints[0])).parent / LR_HISTORY_FILENAME
    if log.exists():
        history = json.loads(log.read_text())
    else:
        history = json.loads((Path(str(cfg.checkpoints[-1])) / "trainer_state.json").read_text())["log_history"]
    lr_at = {e["step"]: e["learning_rate"] for e in history if "learning_rate" in e}
    return [scale * sum(lr_at.get(s, 0.0) for s in range(bounds[l] + 1, bounds[l + 1] + 1)) for l in range(L)]


def f_backward(lr_times_steps: float) -> Callable[[Tensor], Tensor]:
    return lambda sigma: torch.exp(-lr_times_steps * sigma)


def f_segment(lr_times_steps: float) -> Callable[[Tensor], Tensor]:
    def fn(sigma: Tensor) -> Tensor:
        x = lr_times_steps * sigma
        zero = x == 0
        xs = x.masked_fill(zero, 1.0)
        return lr_times_steps * (-torch.expm1(-xs) / xs).masked_fill(zero, 1.0)

    return fn


def f_one_minus_exp(lr_times_steps: float) -> Callable[[Tensor], Tensor]:
    """Numerator of ``f_segment``; the ``1/s`` is then supplied by an EK-FAC inverse."""
    return lambda sigma: -torch.expm1(-lr_times_steps * sigma)


def _apply_eigfn_worker(rank, local_rank, world_size, cfg: EkfacConfig, lr_times_steps: float, fn_kind: str,
                        inversion_cfg: InversionConfig | None) -> None:
    init_dist(rank, local_rank, world_size)
    # The EK-FAC inverse only takes part in the optimizer-preconditioned hybrid, where it
    # supplies the 1/sigma of f_segment after the diagonal multiplier; without a
    # preconditioner grid the eigenvalue function carries the 1/sigma itself.
    if not cfg.preconditioner_path:
        inversion_cfg = None
    if inversion_cfg is not None:
        fn = f_one_minus_exp(lr_times_steps)
    else:
        fn = {"f_segment": f_segment, "f_backward": f_backward}[fn_kind](lr_times_steps)
    EkfacApplicator(cfg, inversion_cfg=inversion_cfg, apply_fn=fn).compute_ivhp_sharded()


def apply_eigfn_to_query(src_grad_path: Path, dst_grad_path: Path, segment_dir: Path, lr_times_steps: float,
                         fn_kind: str, distributed: DistributedConfig, preconditioner_path: str = "",
                         inversion_cfg: InversionConfig | None = None) -> None:
    """Apply one segment's ``f_backward`` / ``f_segment`` to a stored query gradient."""
    cfg = EkfacConfig(hessian_method_path=str(segment_dir), gradient_path=str(src_grad_path),
                      run_path=str(dst_grad_path), ev_correction=True, preconditioner_path=preconditioner_path)
    launch_distributed_run("apply_eigfn_to_query", _apply_eigfn_worker,
                           [cfg, lr_times_steps, fn_kind, inversion_cfg if fn_kind == "f_segment" else None],
                           distributed)


def walk_query_phase1(run_path, method: str, lr_times_steps_per_segment: list[float], distributed,
                      preconditioner_paths: list[str] | None = None, inversion_cfg=None) -> list[Path]:
    """``q_{L-1}`` is ``<run>/query``; ``q_{k-1} = F_backward(segment k) q_k`` lands in
    ``segment_{k-1}/query_grad_backward``.  Returns ``[q_0, ..., q_{L-1}]`` paths."""
    base, L = Path(run_path), len(lr_times_steps_per_segment)
    paths: list[Path] = [Path("")] * L
    paths[L - 1] = base / "query"
    for k in range(L - 1, 0, -1):
        dst = base / f"segment_{k - 1}" / "query_grad_backward"
        apply_eigfn_to_query(paths[k], dst, base / f"segment_{k}" / method, lr_times_steps_per_segment[k],
                             "f_backward", distributed, preconditioner_paths[k] if preconditioner_paths else "")
        paths[k - 1] = dst
    return paths


def walk_query_phase2(run_path, method: str, lr_times_steps_per_segment: list[float], query_grad_paths: list[Path],
                      distributed, preconditioner_paths: list[str] | None = None, inversion_cfg=None) -> list[Path]:
    """``r_l = F_segment(segment l) q_l`` into ``segment_l/query_grad_segment``."""
    base = Path(run_path)
    out = []
    for l, k in enumerate(lr_times_steps_per_segment):
        dst = base / f"segment_{l}" / "query_grad_segment"
        apply_eigfn_to_query(query_grad_paths[l], dst, base / f"segment_{l}" / method, k, "f_segment", distributed,
                             preconditioner_paths[l] if preconditioner_paths else "", inversion_cfg)
        out.append(dst)
    return out


def score_per_segment_and_aggregate(index_cfg: IndexConfig, query_grad_segment_paths: list[Path],
                                    segment_checkpoints: list[list[str]], query_batch_size: int | None = None) -> Path:
    """Score every checkpoint of every segment against the segment's response, average
    within segments, sum over segments, write ``<run>/scores`` (loss-signed)."""
    from ..cli.commands import Score

    base = Path(index_cfg.run_path)
    dirs: list[Path] = []

    def oriented(d: Path):
        s = load_scores(d)[:]
        cfg = load_subconfig(d, "score_cfg", ScoreConfig)
        if cfg is None:
            raise FileNotFoundError(f"No score_cfg found at {d}; cannot determine the scores' orientation.")
        return -s if cfg.higher_is_better else s

    total = None
    for l, ckpts in enumerate(segment_checkpoints):
        seg = None
        for c, ckpt in enumerate(ckpts):
            d = base / f"segment_{l}" / f"scores_ckpt_{c}"
            if index_cfg.distributed._node_rank == 0 and d.exists():
                shutil.rmtree(d)
            icfg = deepcopy(index_cfg)
            icfg.model, icfg.run_path, icfg.projection_dim = ckpt, str(d), 0
            scfg = ScoreConfig(query_path=str(query_grad_segment_paths[l]), higher_is_better=True,
                               query_batch_size=query_batch_size)
            pcfg = PreprocessConfig()
            save_run_config(Score(scfg, icfg, pcfg), icfg.partial_run_path)
            score_dataset(icfg, scfg, pcfg)
            dirs.append(d)
            s = oriented(d)
            seg = s if seg is None else seg + s
        assert seg is not None, "each segment has >= 1 checkpoint"
        total = seg / len(ckpts) if total is None else total + seg / len(ckpts)
    assert total is not None
    out = base / "scores"
    if index_cfg.attribute_tokens:
        save_token_scores(out, total, np.load(dirs[0] / "offsets.npy"))
    else:
        save_sequence_scores(out, total)
    ocfg = deepcopy(index_cfg)
    ocfg.run_path = str(out)
    save_run_config(Score(ScoreConfig(higher_is_better=False), ocfg, PreprocessConfig()), out)
    return out
