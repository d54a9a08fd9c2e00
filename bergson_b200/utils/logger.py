"""Rank-aware logging (reference ``bergson/utils/logger.py:17-69``)."""

from __future__ import annotations

import inspect
import logging
import sys

import torch.distributed as dist

logging.basicConfig(
    level=logging.INFO,
    format="%(filename)s:%(funcName)s:%(lineno)d:%(levelname)s:  %(message)s",
    stream=sys.stdout,
    force=True,
)


class RankFilter(logging.Filter):
    """Pass records on rank 0 only."""

    def filter(self, record):
        return (dist.get_rank() if dist.is_initialized() else 0) == 0


def get_logger(name: str | None = None, level: str | None = None, disable_filter: bool = False):
    if name is None:
        frame = inspect.currentframe()
        caller = frame.f_back if frame else None
        name = caller.f_globals.get("__name__", "unknown") if caller else "unknown"
    logger = logging.getLogger(name)
    if not disable_filter and not any(isinstance(f, RankFilter) for f in logger.filters):
        logger.addFilter(RankFilter())
    if level is not None:
        logger.setLevel(getattr(logging, level.upper(), logging.INFO))
    return logger
