"""Preconditioners: ``apply({module: [n, d]}) -> {module: [n, d]}``.

* ``DensePreconditioner``: per-module ``[d, d]`` matrix ``H^p`` of an autocorrelation
  Hessian; ``g @ H^p``.
* ``FactoredPreconditioner``: Kronecker-factored (K-FAC / EK-FAC / TKFAC / Shampoo):
  ``Q_G [(Q_G^T G Q_A) * m(Lambda)] Q_A^T`` on ``G`` viewed ``[n, O, I]``.
* ``DiagonalFactoredPreconditioner``: elementwise ``f(p * diag(H))`` with
  ``diag(H) = (Q_G*Q_G) Lambda (Q_A*Q_A)^T`` (optimizer-preconditioned SOURCE).

``load_preconditioner`` picks dense vs factored by the presence of
``eigen_activation_sharded/`` (reference ``bergson/hessians/preconditioner.py``).
The sharded factors of a module are assembled once with a single all-gather and cached,
so repeated applications cost local GEMMs only.
"""

from __future__ import annotations

import os
from glob import glob
from pathlib import Path
from typing import Protocol, runtime_checkable

import torch
from safetensors.torch import load_file
from torch import Tensor

from ..config import InversionConfig
from ..gradients import GradientProcessor
from ..utils.logger import get_logger
from .inversion import eigenvalue_multiplier, invert_psd_matrix
from .sharded_computation import ShardedMul


@runtime_checkable
class Preconditioner(Protocol):
    def apply(self, grads: dict[str, Tensor]) -> dict[str, Tensor]: ...


class DensePreconditioner:
    def __init__(self, h_inv: dict[str, Tensor]):
        self.h_inv = h_inv

    @classmethod
    def from_processor(cls, processor: GradientProcessor, *, inversion_cfg: InversionConfig | None = None,
                       power: float = -1.0, device="cpu") -> "DensePreconditioner":
        cfg = inversion_cfg or InversionConfig()
        return cls({
            name: invert_psd_matrix(H.to(device=device, dtype=torch.float32), inversion=cfg.inversion,
                                    damping_factor=cfg.damping_factor, power=power)
            for name, H in processor.hessians.items()
        })

    def apply(self, grads: dict[str, Tensor]) -> dict[str, Tensor]:
        if not self.h_inv:
            return grads
        out = {}
        for name, g in grads.items():
            h = self.h_inv.get(name)
            out[name] = g if h is None else (g.to(device=h.device, dtype=h.dtype) @ h).to(g.device)
        return out


def _shard_files(hessian_path, subdir: str) -> list[str]:
    d = Path(hessian_path) / subdir
    files = sorted(glob(os.path.join(d, "shard_*.safetensors")), key=lambda p: int(Path(p).stem.split("_")[1]))
    if not files:
        raise FileNotFoundError(f"No shard_*.safetensors found in {d}")
    return files


def _load_full(hessian_path, subdir: str, device) -> dict[str, Tensor]:
    """Concatenate every shard along dim 0 (exact for any writer world size), fp32."""
    loaded = [load_file(f, device=str(device)) for f in _shard_files(hessian_path, subdir)]
    return {k: torch.cat([s[k] for s in loaded], dim=0).float() for k in loaded[0]}


def _load_shard(hessian_path, subdir: str, rank: int, device) -> dict[str, Tensor]:
    f = os.path.join(str(hessian_path), subdir, f"shard_{rank}.safetensors")
    return {k: v.float() for k, v in load_file(f, device=str(device)).items()}


class FactoredPreconditioner:
    """Pass either ``inversion_cfg`` (standard inversions) or ``apply_fn`` (a custom
    eigenvalue function, e.g. the learning-rate maps of approximate unrolling)."""

    def __init__(self, eigen_a, eigen_g, lambdas, *, inversion_cfg: InversionConfig | None = None, apply_fn=None,
                 power: float = -1.0, factor_eig_a=None, factor_eig_g=None):
        if inversion_cfg is not None and apply_fn is not None:
            raise ValueError("Pass either inversion_cfg or apply_fn, not both.")
        self.eigen_a, self.eigen_g, self.lambdas = eigen_a, eigen_g, lambdas
        self.factor_eig_a = factor_eig_a or {}
        self.factor_eig_g = factor_eig_g or {}
        self.inversion_cfg = inversion_cfg or InversionConfig()
        self.apply_fn = apply_fn
        self.power = power
        self.shard_computer = ShardedMul()
        self.logger = get_logger("FactoredPreconditioner")
        self._full: dict[str, tuple[Tensor, Tensor, Tensor]] = {}

    @classmethod
    def from_path(cls, hessian_path, *, inversion_cfg=None, apply_fn=None, power: float = -1.0,
                  ev_correction: bool = False, device="cpu"):
        """Single process: whole factors (shards concatenated).  ``factor_eig_a`` is
        replicated in every shard, so only shard 0 of it is read."""
        return cls._build(
            lambda sub: _load_full(hessian_path, sub, device),
            lambda sub: _load_shard(hessian_path, sub, 0, device),
            inversion_cfg, apply_fn, power, ev_correction,
        )

    @classmethod
    def from_shards(cls, hessian_path, *, rank: int, device, inversion_cfg=None, apply_fn=None, power: float = -1.0,
                    ev_correction: bool = False):
        """Distributed: this rank's shard files."""
        load = lambda sub: _load_shard(hessian_path, sub, rank, device)  # noqa: E731
        return cls._build(load, load, inversion_cfg, apply_fn, power, ev_correction)

    @classmethod
    def _build(cls, load, load_replicated, inversion_cfg, apply_fn, power, ev_correction):
        ft = inversion_cfg is not None and inversion_cfg.inversion == "factored_tikhonov"
        if ft and ev_correction:
            raise ValueError(
                "factored_tikhonov inversion is incompatible with ev_correction: the corrected eigenvalues "
                "do not factorize as l_G (x) l_A. Use a different inversion or set ev_correction=False."
            )
        lam_dir = "eigenvalue_correction_sharded" if ev_correction else "eigenvalue_sharded"
        return cls(
            load("eigen_activation_sharded"), load("eigen_gradient_sharded"), load(lam_dir),
            inversion_cfg=inversion_cfg, apply_fn=apply_fn, power=power,
            factor_eig_a=load_replicated("factor_eig_a") if ft else None,
            factor_eig_g=load("factor_eig_g") if ft else None,
        )

    def _multiplier_shard(self, name: str, o: int, i: int) -> Tensor:
        lam = self.lambdas[name]
        if self.apply_fn is not None:
            return self.apply_fn(lam)
        sc = self.shard_computer
        mean = sc.global_mean(lam, o * i)
        cfg = self.inversion_cfg
        if cfg.inversion == "factored_tikhonov":
            fa, fg = self.factor_eig_a[name], self.factor_eig_g[name]
            return eigenvalue_multiplier(
                cfg.inversion, lam, mean, cfg.damping_factor, factor_a=fa, factor_g=fg,
                mean_a=fa.clamp_min(0).mean(), mean_g=sc.global_mean(fg.clamp_min(0), o), power=self.power,
            )
        return eigenvalue_multiplier(cfg.inversion, lam, mean, cfg.damping_factor, power=self.power)

    def _assembled(self, name: str) -> tuple[Tensor, Tensor, Tensor]:
        """(Q_A [I, I], Q_G [O, O], m(Lambda) [O, I]) in local memory, gathered once."""
        if name not in self._full:
            sc = self.shard_computer
            q_a, q_g = self.eigen_a[name], self.eigen_g[name]
            o, i = q_g.shape[1], q_a.shape[1]
            self._full[name] = (
                sc.gather_rows(q_a, i), sc.gather_rows(q_g, o), sc.gather_rows(self._multiplier_shard(name, o, i), o)
            )
        return self._full[name]

    def apply(self, grads: dict[str, Tensor]) -> dict[str, Tensor]:
        out: dict[str, Tensor] = {}
        for name, flat in grads.items():
            if name not in self.eigen_a:
                out[name] = flat
                continue
            q_a, q_g, mult = self._assembled(name)
            o, i = q_g.shape[0], q_a.shape[0]
            g = flat.to(q_a.device, torch.float32).view(-1, o, i)
            g = _left(q_g.T, _right(g, q_a))   # into the eigenbasis
            g = g * mult
            g = _left(q_g, _right(g, q_a.T))   # and back
            out[name] = g.reshape(flat.shape[0], -1).to(flat.dtype)
        return out


def _right(g: Tensor, m: Tensor) -> Tensor:
    """``g [n, O, I] @ m [I, J]``: one GEMM over all ``n * O`` rows (fp32-accurate tensor-core
    product on CUDA, see ``ops.attribution.split_matmul``)."""
    from ..ops.attribution import split_matmul

    n, o, i = g.shape
    return split_matmul(g.reshape(n * o, i), m.contiguous()).view(n, o, m.shape[1])


def _left(m: Tensor, g: Tensor) -> Tensor:
    """``m [P, O] @ g [n, O, I]`` for every n, as ``(g^T m^T)^T`` so that it is one GEMM too."""
    from ..ops.attribution import split_matmul

    n, o, i = g.shape
    gt = g.transpose(1, 2).reshape(n * i, o)
    return split_matmul(gt, m.T.contiguous()).view(n, i, m.shape[0]).transpose(1, 2)


class DiagonalFactoredPreconditioner:
    """Gradients are multiplied elementwise, in parameter space, by
    ``apply_fn(p * diag(H))`` (no rotation)."""

    def __init__(self, eigen_a, eigen_g, lambdas, preconditioner, *, apply_fn):
        self.eigen_a, self.eigen_g, self.lambdas = eigen_a, eigen_g, lambdas
        self.preconditioner = preconditioner
        self.apply_fn = apply_fn
        self.shard_computer = ShardedMul()
        self.logger = get_logger("DiagonalFactoredPreconditioner")
        self._multipliers: dict[str, Tensor] = {}

    @classmethod
    def from_shards(cls, hessian_path, preconditioner_path, *, rank: int, device, apply_fn, ev_correction: bool = False):
        lam_dir = "eigenvalue_correction_sharded" if ev_correction else "eigenvalue_sharded"
        eigen_a = _load_shard(hessian_path, "eigen_activation_sharded", rank, device)
        eigen_g = _load_shard(hessian_path, "eigen_gradient_sharded", rank, device)
        lambdas = _load_shard(hessian_path, lam_dir, rank, device)
        grids = load_file(str(preconditioner_path), device=str(device))
        sc = ShardedMul()
        pre = {}
        for name, q_g in eigen_g.items():
            if name not in grids:
                raise KeyError(
                    f"Module {name!r} has EKFAC factors but no preconditioner grid in {preconditioner_path}; "
                    f"available: {sorted(grids)}"
                )
            p = grids[name].float()
            o, i = q_g.shape[1], eigen_a[name].shape[1]
            if p.shape != (o, i):
                raise ValueError(f"Preconditioner grid for {name!r} has shape {tuple(p.shape)}, expected ({o}, {i}).")
            lo, hi = sc.shard_bounds(o)
            pre[name] = p[lo:hi]
        return cls(eigen_a, eigen_g, lambdas, pre, apply_fn=apply_fn)

    def _diag_hessian_shard(self, name: str) -> Tensor:
        """This rank's ``[c_o, I]`` rows of ``(Q_G*Q_G) Lambda (Q_A*Q_A)^T``."""
        sc = self.shard_computer
        q_a, q_g, lam = self.eigen_a[name], self.eigen_g[name], self.lambdas[name]
        if not sc.dist:
            return (q_g**2) @ lam @ (q_a**2).T
        q_a_full = sc.gather_rows(q_a, q_a.shape[1])
        lam_full = sc.gather_rows(lam, q_g.shape[1])
        return (q_g**2) @ (lam_full @ (q_a_full**2).T)

    def _multiplier(self, name: str) -> Tensor:
        if name not in self._multipliers:
            self._multipliers[name] = self.apply_fn(self.preconditioner[name] * self._diag_hessian_shard(name))
        return self._multipliers[name]

    def apply(self, grads: dict[str, Tensor]) -> dict[str, Tensor]:
        out: dict[str, Tensor] = {}
        for name, flat in grads.items():
            if name not in self.eigen_a:
                out[name] = flat
                continue
            o, i = self.eigen_g[name].shape[1], self.eigen_a[name].shape[1]
            # copy: the input may alias a read-only memmap
            g = flat.to(self.lambdas[name].device, torch.float32, copy=True).view(-1, o, i)
            self.shard_computer.scale_rows_in_place(g, self._multiplier(name))
            out[name] = g.reshape(flat.shape[0], -1).to(flat.dtype)
        return out


def is_factored_hessian(hessian_path) -> bool:
    return (Path(hessian_path) / "eigen_activation_sharded").is_dir()


def load_preconditioner(hessian_path, *, inversion_cfg: InversionConfig | None = None, power: float | None = -1.0,
                        ev_correction: bool = False, device="cpu") -> Preconditioner | None:
    """fp32 preconditioner for the Hessian stored at ``hessian_path`` (None if unset)."""
    if power is None or hessian_path is None:
        return None
    if is_factored_hessian(hessian_path):
        return FactoredPreconditioner.from_path(
            hessian_path, inversion_cfg=inversion_cfg, power=power, ev_correction=ev_correction, device=device
        )
    processor = GradientProcessor.load(Path(hessian_path), map_location="cpu")
    return DensePreconditioner.from_processor(processor, inversion_cfg=inversion_cfg, power=power, device=device)
