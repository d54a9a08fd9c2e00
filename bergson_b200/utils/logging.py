"""Optional Weights & Biases loss logging; degrades to a no-op when wandb is missing or
disabled (reference ``bergson/utils/logging.py:9-53``)."""

from __future__ import annotations

import os
from typing import Callable


def wandb_log_fn(project: str, config: dict | None = None) -> Callable[[int, float], None]:
    if os.environ.get("WANDB_MODE") == "disabled":
        return lambda step, loss: None
    try:
        import wandb

        run = wandb.init(project=project, config=config or {})
    except Exception as e:  # noqa: BLE001 - logging must never break training
        print(f"wandb unavailable ({e}); training loss will not be logged")
        return lambda step, loss: None

    def log(step: int, loss: float) -> None:
        run.log({"train/loss": loss}, step=step)

    return log
