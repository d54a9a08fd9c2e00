"""Gradient processing state: optimizer normalisers, Hessians, projection settings.

Formats match the reference (``bergson/gradients.py:77-239``):
``processor_config.yaml``, ``normalizers.pth``, ``hessians.pth``,
``hessians_eigen.pth`` (legacy ``preconditioners*.pth`` names are still read).
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Literal, Mapping

import torch
import torch.nn as nn
import yaml
from torch import Tensor

from .models.common import Conv1D

try:  # HF's GPT-2 layer, when transformers is importable
    from transformers.pytorch_utils import Conv1D as HFConv1D
except Exception:  # pragma: no cover
    HFConv1D = Conv1D  # type: ignore[misc,assignment]

NORMALIZER_TYPES: dict[str, type["Normalizer"]] = {}


class Normalizer(ABC):
    """Scales gradients by optimizer second-moment statistics."""

    def __init_subclass__(cls, **kwargs):
        super().__init_subclass__(**kwargs)
        NORMALIZER_TYPES[cls.__name__] = cls

    @staticmethod
    def from_state_dict(state: dict) -> "Normalizer":
        state = dict(state)
        name = state.pop("__class__")
        cls = NORMALIZER_TYPES.get(name)
        if cls is None:
            raise ValueError(f"Unknown normalizer class: '{name}'")
        if "avg_sq" in state:  # old key name
            state["weight_avg_sq"] = state.pop("avg_sq")
        return cls(**state)

    @abstractmethod
    def normalize_weight(self, grad: Tensor, eps: float = 1e-8) -> Tensor: ...

    @abstractmethod
    def normalize_bias(self, grad: Tensor, eps: float = 1e-8) -> Tensor: ...

    def state_dict(self) -> dict:
        return {
            "__class__": type(self).__name__,
            **{k: v for k, v in self.__dict__.items() if isinstance(v, Tensor)},
        }


@dataclass
class AdafactorNormalizer(Normalizer):
    """Factored second moments: ``row`` [O], ``col`` [I], optional bias moments [O].

    ``V_ij = row_i col_j / mean(row)``; gradients are multiplied by ``V^-1/2`` which
    factorises into a row scale ``sqrt(mean(row+eps)) / sqrt(row+eps)`` and a column
    scale ``1/sqrt(col+eps)`` — so it can be applied to ``g`` and ``a`` separately
    and the full gradient never has to be formed.
    """

    row: Tensor
    col: Tensor
    bias_avg_sq: Tensor | None = None

    def __post_init__(self):
        assert self.row.ndim == 1 and self.col.ndim == 1
        assert self.bias_avg_sq is None or self.bias_avg_sq.ndim == 1

    def row_scale(self, eps: float = 1e-30) -> Tensor:
        r = self.row.add(eps)
        return r.mean().sqrt() * r.rsqrt()

    def col_scale(self, eps: float = 1e-30) -> Tensor:
        return self.col.add(eps).rsqrt()

    def normalize_weight(self, grad: Tensor, eps: float = 1e-30) -> Tensor:
        grad *= self.row_scale(eps)[:, None]
        grad *= self.col_scale(eps)[None, :]
        return grad

    def normalize_bias(self, grad: Tensor, eps: float = 1e-8) -> Tensor:
        assert self.bias_avg_sq is not None
        return grad * self.bias_avg_sq.add(eps).rsqrt()

    def to_adam(self) -> "AdamNormalizer":
        return AdamNormalizer(torch.outer(self.row, self.col) / self.row.mean(), self.bias_avg_sq)


@dataclass
class AdamNormalizer(Normalizer):
    """Full second moments ``weight_avg_sq`` [O, I]; ``g / (sqrt(v) + eps)``."""

    weight_avg_sq: Tensor
    bias_avg_sq: Tensor | None = None

    def normalize_weight(self, grad: Tensor, eps: float = 1e-8) -> Tensor:
        return grad.div_(self.weight_avg_sq.sqrt().add_(eps))

    def normalize_bias(self, grad: Tensor, eps: float = 1e-8) -> Tensor:
        assert self.bias_avg_sq is not None
        return grad / self.bias_avg_sq.sqrt().add_(eps)

    def to_adafactor(self) -> AdafactorNormalizer:
        assert self.weight_avg_sq.ndim == 2
        return AdafactorNormalizer(
            self.weight_avg_sq.mean(1), self.weight_avg_sq.mean(0), self.bias_avg_sq
        )


@dataclass
class GradientProcessor:
    """Everything needed to turn raw per-example gradients into store rows."""

    normalizers: Mapping[str, Normalizer] = field(default_factory=dict)
    hessians: dict[str, Tensor] = field(default_factory=dict)
    hessians_eigen: Mapping[str, tuple[Tensor, Tensor]] = field(default_factory=dict)
    projection_dim: int | None = None
    reshape_to_square: bool = False
    projection_type: Literal["normal", "rademacher"] = "rademacher"
    projection_target: Literal["per_module", "global"] = "per_module"
    projection_scale: Literal["jl", "row_norm"] = "jl"
    include_bias: bool = False

    def __post_init__(self):
        self._projection_matrices: dict = {}

    @classmethod
    def load(cls, path, *, map_location=None, skip_hessians: bool = False):
        path = Path(path)

        def pick(new: str, old: str) -> Path:
            return path / new if (path / new).exists() else path / old

        with (path / "processor_config.yaml").open() as f:
            cfg = yaml.safe_load(f) or {}
        # Defaults of stores written before these keys existed.
        cfg.setdefault("projection_type", "normal")
        cfg.setdefault("include_bias", False)
        cfg.setdefault("projection_scale", "row_norm")
        for key in list(cfg):
            if "precond" in key:
                new = (
                    key.replace("preconditioners", "hessians")
                    .replace("preconditioner", "hessian")
                    .replace("precond", "hess")
                )
                cfg[new] = cfg.pop(key)
        allowed = {f for f in cls.__dataclass_fields__}
        cfg = {k: v for k, v in cfg.items() if k in allowed}

        norm_state = torch.load(path / "normalizers.pth", map_location=map_location, weights_only=True)
        normalizers = {k: Normalizer.from_state_dict(v) for k, v in norm_state.items()}
        hessians, eigen = {}, {}
        if not skip_hessians:
            hp = pick("hessians.pth", "preconditioners.pth")
            ep = pick("hessians_eigen.pth", "preconditioners_eigen.pth")
            if hp.exists():
                hessians = torch.load(hp, map_location=map_location, weights_only=True)
            if ep.exists():
                eigen = torch.load(ep, map_location=map_location, weights_only=True)
        return cls(normalizers=normalizers, hessians=hessians, hessians_eigen=eigen, **cfg)

    def save(self, path) -> None:
        path = Path(path)
        path.mkdir(parents=True, exist_ok=True)
        cfg = asdict(self)
        for k in ("normalizers", "hessians", "hessians_eigen"):
            cfg.pop(k)
        with (path / "processor_config.yaml").open("w") as f:
            yaml.safe_dump(cfg, f, sort_keys=False)
        torch.save({k: n.state_dict() for k, n in self.normalizers.items()}, path / "normalizers.pth")
        torch.save(self.hessians, path / "hessians.pth")
        torch.save(self.hessians_eigen, path / "hessians_eigen.pth")


class LayerAdapter:
    """Uniform view of the layer types whose weight gradient is ``g^T a``."""

    supported_modules = tuple(
        dict.fromkeys((nn.Linear, Conv1D, HFConv1D, nn.Conv1d, nn.Conv2d, nn.Conv3d))
    )
    _conv1d_like = tuple(dict.fromkeys((Conv1D, HFConv1D)))

    @classmethod
    def in_attr(cls, layer: nn.Module) -> str:
        if isinstance(layer, nn.Linear):
            return "in_features"
        if isinstance(layer, cls._conv1d_like):
            return "nx"
        if isinstance(layer, (nn.Conv1d, nn.Conv2d, nn.Conv3d)):
            return "in_channels"
        raise ValueError(f"Unsupported layer type: {type(layer)}")

    @classmethod
    def out_attr(cls, layer: nn.Module) -> str:
        if isinstance(layer, nn.Linear):
            return "out_features"
        if isinstance(layer, cls._conv1d_like):
            return "nf"
        if isinstance(layer, (nn.Conv1d, nn.Conv2d, nn.Conv3d)):
            return "out_channels"
        raise ValueError(f"Unsupported layer type: {type(layer)}")

    @classmethod
    def weight_transposed(cls, layer: nn.Module) -> bool:
        """True when the weight is stored ``[in, out]`` (Conv1D)."""
        return isinstance(layer, cls._conv1d_like)
