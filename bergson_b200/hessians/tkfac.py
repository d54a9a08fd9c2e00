"""Trace-weighted K-FAC factors (see ``kfac.py`` for the shared machinery)."""

from dataclasses import dataclass

from .kfac import _FactorCollector


@dataclass(kw_only=True)
class TraceCovarianceCollector(_FactorCollector):
    """``A += tr(g^T g) a^T a``, ``S += tr(a^T a) g^T g`` per batch."""

    method: str = "tkfac"
