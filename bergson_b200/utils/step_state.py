"""``.part`` / promote protocol for restartable pipeline steps.

A step writes into ``<out>.part`` and renames it to ``<out>`` when finished, so
``<out>`` existing means "finished", only ``<out>.part`` means "interrupted"
(reference ``bergson/utils/step_state.py:21-88``).
"""

from __future__ import annotations

import shutil
from pathlib import Path
from typing import Literal

StepState = Literal["complete", "partial", "missing"]


def partial_path(path: Path | str) -> Path:
    path = Path(path)
    return path.with_name(path.name + ".part")


def _parked(path: Path) -> Path:
    return path.with_name(path.name + ".superseded")


def step_state(path: Path | str) -> StepState:
    path = Path(path)
    if path.exists():
        return "complete"
    return "partial" if partial_path(path).exists() else "missing"


def prepare_step(path: Path | str, *, resume: bool) -> bool:
    """True if the step must run. Clears an interrupted ``.part`` (and a parked
    ``.superseded``) but never the finished output: a rerun replaces that only
    when it is promoted."""
    path = Path(path)
    if resume and step_state(path) == "complete":
        return False
    for stale in (partial_path(path), _parked(path)):
        if stale.exists():
            shutil.rmtree(stale)
    return True


def promote_step(path: Path | str) -> None:
    """Rename ``<path>.part`` to ``<path>``; an older output is parked under
    ``.superseded`` until the new one is in place, then removed."""
    path = Path(path)
    part = partial_path(path)
    if not part.exists():
        raise FileNotFoundError(f"No partial output to promote at {part}")
    if path.exists():
        parked = _parked(path)
        if parked.exists():
            shutil.rmtree(parked)
        path.rename(parked)
        part.rename(path)
        shutil.rmtree(parked)
    else:
        part.rename(path)
