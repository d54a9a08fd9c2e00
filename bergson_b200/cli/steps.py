"""A small runner for multi-step pipelines whose steps leave a directory behind.

A pipeline is a list of ``Step`` records; the runner announces each one, skips those whose
output already marks them complete (when resuming), times the rest and returns the timings.
Two completion protocols exist among the commands: ``"promote"`` (a step writes
``<out>.part`` and renames it when done, so an interrupted ``.part`` is cleared before a
rerun; see ``utils.step_state``) and ``"exists"`` (the output directory appearing is the
mark).  ``derive`` builds the per-step variations of an index configuration.
"""

from __future__ import annotations

import time
from copy import deepcopy
from dataclasses import dataclass
from pathlib import Path
from typing import Callable, Literal

from ..config.config import IndexConfig
from ..utils.step_state import prepare_step
from ..utils.worker_utils import validate_run_path


@dataclass
class Step:
    title: str                       # what the step does, for the progress line
    output: str | None               # directory that marks the step complete (None: always run)
    action: Callable[[], None]
    key: str = ""                    # name in the timing table (defaults to the title)
    enabled: bool = True             # a disabled step is announced as skipped and never runs
    skip_note: str = ""


def derive(cfg: IndexConfig, **changes) -> IndexConfig:
    """A deep copy of ``cfg`` with attributes replaced (values are deep-copied too)."""
    out = deepcopy(cfg)
    for name, value in changes.items():
        setattr(out, name, deepcopy(value))
    return out


class StepRunner:
    def __init__(self, *, resume: bool, protocol: Literal["promote", "exists"] = "exists"):
        self.resume, self.protocol = resume, protocol
        self.timings: dict[str, float] = {}

    def check_run_path(self, cfg: IndexConfig) -> None:
        """Refuse to clobber an existing run unless this is a resume that left a partial one."""
        if not (self.resume and cfg.partial_run_path.exists()):
            validate_run_path(cfg)

    def _done(self, output: str | None) -> bool:
        if output is None:
            return False
        if self.protocol == "promote":
            return not prepare_step(output, resume=self.resume)
        return self.resume and Path(output).exists()

    def run(self, steps: list[Step]) -> dict[str, float]:
        n = len(steps)
        for k, step in enumerate(steps, 1):
            head = f"[{k}/{n}] {step.title}"
            if not step.enabled:
                print(f"{head}: not needed{' (' + step.skip_note + ')' if step.skip_note else ''}")
                continue
            if self._done(step.output):
                print(f"{head}: already complete at {step.output}")
                continue
            print(f"{head} ...")
            t0 = time.perf_counter()
            step.action()
            self.timings[step.key or step.title] = dt = time.perf_counter() - t0
            print(f"{head}: {dt:.1f}s")
        return self.timings
