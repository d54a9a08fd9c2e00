"""Type names the reference imports from ``torchopt.typing``."""

from __future__ import annotations

from typing import Any, Callable, NamedTuple, Union

import torch

Params = Any
Updates = Any
OptState = Any
Schedule = Callable[[Any], Any]
ScalarOrSchedule = Union[float, int, torch.Tensor, Schedule]


class GradientTransformation(NamedTuple):
    init: Callable
    update: Callable
