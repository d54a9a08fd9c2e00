"""MAGIC: attribution by differentiating through training."""

from ..config.config import MagicConfig

_LAZY = {
    "run_magic": ".cli",
    "DataStream": ".data_stream",
    "muon": ".optim",
    "adamw": ".optim",
    "sgd": ".optim",
    "BackwardState": ".trainer",
    "Trainer": ".trainer",
    "TrainerState": ".trainer",
    "prepare_trainer": ".trainer",
    "apply_dtensor_patch": ".dtensor_patch",
}

__all__ = ["MagicConfig", *sorted(_LAZY)]


def __getattr__(name: str):
    if name in _LAZY:
        import importlib

        value = getattr(importlib.import_module(_LAZY[name], __name__), name)
        globals()[name] = value
        return value
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
