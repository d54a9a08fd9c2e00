"""Fill unset SOURCE options from the training run the checkpoints came from
(reference ``bergson/approx_unrolling/train_cfg_io.py``)."""

from __future__ import annotations

from pathlib import Path

from ..config.config import ApproxUnrollingConfig, TrainingConfig
from ..config.config_io import CONFIG_FILENAME, read_config
from ..utils.logger import get_logger

LR_HISTORY_FILENAME = "log_history.json"
logger = get_logger(__name__)


def load_training_config(trainer_run) -> TrainingConfig:
    """The ``TrainingConfig`` recorded in ``<trainer_run>/config.yaml`` (first step)."""
    path = Path(trainer_run) / CONFIG_FILENAME
    if not path.is_file():
        raise FileNotFoundError(f"{path} not found; trainer_run must be a run directory with config.yaml.")
    steps = read_config(path)["steps"]
    if not steps or not isinstance(steps[0], dict):
        raise ValueError(f"{path} is not a run config")
    body = next(iter(steps[0].values()))
    if not isinstance(body, dict):
        raise ValueError(f"{path} is not a run config")
    try:
        return TrainingConfig.from_dict(body, drop_extra_fields=True)
    except Exception as e:  # noqa: BLE001
        raise ValueError(f"{path} is not a training config: {e}") from e


def derive_momentum(cfg: TrainingConfig) -> float:
    """SGD trains with heavy-ball ``adam_beta1``; AdamW's first moment is handled by the
    preconditioned variant, so 0."""
    if cfg.optimizer == "sgd":
        return float(cfg.adam_beta1)
    if cfg.optimizer != "adamw":
        logger.warning("Cannot derive a SOURCE momentum for optimizer %r; using 0.0.", cfg.optimizer)
    return 0.0


def infer_trainer_run(checkpoints: list[str]) -> str:
    """``<run>`` for checkpoints at ``<run>/exported/checkpoint-N`` or ``<run>/checkpoint-N``."""
    if not checkpoints:
        return ""
    first = Path(checkpoints[0])
    for cand in (first.parent.parent, first.parent):
        if (cand / CONFIG_FILENAME).is_file():
            return str(cand)
    return ""


def resolve(cfg: ApproxUnrollingConfig) -> ApproxUnrollingConfig:
    from ..utils.trainer_export import ensure_exported

    # Raw trainer checkpoints (step_<n>.ckpt) are exported to model directories on demand.
    cfg.checkpoints = ensure_exported([str(c) for c in cfg.checkpoints])
    run = infer_trainer_run([str(c) for c in cfg.checkpoints])
    tcfg = None
    if run:
        try:
            tcfg = load_training_config(run)
        except ValueError as e:
            logger.warning("Ignoring %s as a trainer run: %s", run, e)
    if tcfg is None:
        if cfg.momentum is None:
            cfg.momentum = 0.0
        return cfg
    if tcfg.optimizer == "adamw" and not cfg.use_adam_preconditioner:
        logger.warning("%s trained with adamw but use_adam_preconditioner is not set; using the SGD variant.", run)
    if cfg.model_path is None:
        cfg.model_path = tcfg.model
    if cfg.momentum is None:
        cfg.momentum = derive_momentum(tcfg)
    return cfg


def lr_history_path(checkpoints: list[str]) -> Path | None:
    run = infer_trainer_run([str(c) for c in checkpoints])
    if not run:
        return None
    for cand in (Path(run) / LR_HISTORY_FILENAME, Path(run) / "checkpoints" / LR_HISTORY_FILENAME):
        if cand.is_file():
            return cand
    return None
