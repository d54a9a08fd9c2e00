"""Compatibility entry point.

The reference makes DTensor's redistribute differentiable to any order by patching torch
internals (``bergson/magic/dtensor_patch.py:15-214``).  Parameter sharding here does not
use DTensor: the all-gather / reduce-scatter pair in ``magic.collectives`` is
differentiable by construction, so there is nothing to patch.  The function is kept so
that code calling it keeps working.
"""


def apply_dtensor_patch() -> None:
    return None
