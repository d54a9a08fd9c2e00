"""Shampoo second-moment factors (see ``kfac.py`` for the shared machinery)."""

from dataclasses import dataclass

from .kfac import _FactorCollector


@dataclass(kw_only=True)
class ShampooCollector(_FactorCollector):
    """Batch gradient ``M = g^T a``; ``A += M^T M``, ``S += M M^T``; ``A /= tr(A)``."""

    method: str = "shampoo"
