"""Optional Weights & Biases loss logging.  Logging must never break or stall a training run,
so every way wandb can be unavailable (disabled by ``WANDB_MODE``, not installed, ``init``
raising) yields a callable that does nothing (reference ``bergson/utils/logging.py:9-53``)."""

from __future__ import annotations

import os
import warnings
from typing import Callable

LogFn = Callable[[int, float], None]


def _no_log(step: int, loss: float) -> None:
    return None


def wandb_log_fn(project: str, config: dict | None = None) -> LogFn:
    """``log(step, loss)`` writing ``train/loss`` to the active wandb run; a run that already
    exists is reused, otherwise one is started in ``project`` with ``config``."""
    if os.environ.get("WANDB_MODE") == "disabled":
        return _no_log  # decided before the import: the package may not even be installed
    try:
        import wandb
    except ImportError:
        warnings.warn("wandb is not installed; the training loss will not be logged", UserWarning, stacklevel=2)
        return _no_log
    if wandb.run is None:
        try:
            wandb.init(project=project, config=config) if config is not None else wandb.init(project=project)
        except Exception as e:  # noqa: BLE001 - a dead service or bad credentials on one rank must not stall the others
            warnings.warn(f"wandb.init failed ({type(e).__name__}: {e}); the training loss will not be logged",
                          UserWarning, stacklevel=2)
            return _no_log

    def log(step: int, loss: float) -> None:
        wandb.log({"train/loss": loss}, step=step)

    return log
