"""Options of the ``test_model_configuration`` diagnostic (kept apart from the
diagnostic itself so that the CLI can describe its flags without importing models)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Literal

from .config.parsing import Serializable, field
from .utils.utils import get_device


@dataclass
class DiagnoseConfig(Serializable):
    model: str = "EleutherAI/pythia-160m"
    """Model to test."""

    dataset: str = "NeelNanda/pile-10k"
    """Dataset to draw document pairs from."""

    split: str = "train"
    """Dataset split."""

    n_trials: int = 100
    """Random document pairs per configuration."""

    seed: int = 42
    """Random seed."""

    precision: Literal["bf16", "fp16", "fp32"] = "bf16"
    """Base parameter precision."""

    device: str = field(default_factory=get_device)
    """Device to run on."""

    max_len: int = 512
    """Truncate longer documents."""

    min_len: int = 4
    """Skip shorter documents."""

    threshold: float = 0.99
    """Cosine similarity below this is flagged."""

    model_kwargs: str = ""
    """Extra ``from_pretrained`` kwargs as ``a=b,c=d``."""
