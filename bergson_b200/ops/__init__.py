"""Operators: model-side ops (``functional``), attribution kernels (``attribution``)
and the loader of the in-tree sm_100a extension (``native``)."""

from .linear import Linear, linear
from .functional import (
    causal_attention,
    composable,
    gelu,
    layer_norm,
    rms_norm,
    rotary,
    rotary_tables,
    swiglu,
    token_cross_entropy,
    use_fused,
)

__all__ = [
    "Linear",
    "linear",
    "causal_attention",
    "composable",
    "gelu",
    "layer_norm",
    "rms_norm",
    "rotary",
    "rotary_tables",
    "swiglu",
    "token_cross_entropy",
    "use_fused",
]
