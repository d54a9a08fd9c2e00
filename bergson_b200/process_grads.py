"""Query-gradient preprocessing and autocorrelation-Hessian mixing
(reference ``bergson/process_grads.py:13-182``)."""

from __future__ import annotations

import warnings
from pathlib import Path
from typing import Literal

import torch

from .config.config import HessianConfig
from .config.config_io import load_subconfig
from .gradients import GradientProcessor
from .utils.math import compute_lambda


def normalize_flat_grad(grad: torch.Tensor, device: torch.device) -> torch.Tensor:
    """Unit-normalise one gradient tensor (computed in fp32, returned in its dtype)."""
    out_dtype = grad.dtype
    g = grad.to(device=device, dtype=torch.float32)
    n = g.norm()
    if n > 0:
        g = g / n
    else:
        warnings.warn("Gradient norm is zero, skipping normalization")
    return g.to(out_dtype)


def assert_autocorrelation_hessian(path: Path) -> None:
    cfg = load_subconfig(path, "hessian_cfg", HessianConfig)
    assert cfg is not None, f"No hessian_cfg recorded at '{path}'."
    assert cfg.method == "autocorrelation", (
        f"Hessian at '{path}' was computed with method '{cfg.method}'; "
        "mix_autocorrelation_matrices only supports autocorrelation."
    )


def mix_autocorrelation_matrices(query_path, index_path, output_path, target_downweight_components: int = 1000) -> Path:
    """``H = lam * H_query + (1 - lam) * H_index`` per module, ``lam`` from the pooled
    eigenvalue crossing; saved as a new processor at ``output_path``."""
    query_path, index_path, output_path = Path(query_path), Path(index_path), Path(output_path)
    assert_autocorrelation_hessian(query_path)
    assert_autocorrelation_hessian(index_path)
    q = GradientProcessor.load(query_path)
    i = GradientProcessor.load(index_path)
    lam = compute_lambda(q.hessians_eigen, i.hessians_eigen, target_downweight_components)
    mixed = {k: q.hessians[k] * lam + i.hessians[k] * (1 - lam) for k in q.hessians}
    GradientProcessor(
        normalizers=q.normalizers,
        hessians=mixed,
        hessians_eigen={},
        projection_dim=q.projection_dim,
        reshape_to_square=q.reshape_to_square,
        projection_type=q.projection_type,
        projection_target=q.projection_target,
        projection_scale=q.projection_scale,
        include_bias=q.include_bias,
    ).save(output_path)
    return output_path


def precondition_flat_grads(grads: torch.Tensor, h_inv: dict[str, torch.Tensor], ordered_modules: list[str],
                            batch_size: int = 8192) -> torch.Tensor:
    """In-place ``grads[:, cols_m] @= h_inv[m]`` over row blocks."""
    if not h_inv:
        return grads
    for lo in range(0, grads.shape[0], batch_size):
        hi = min(lo + batch_size, grads.shape[0])
        col = 0
        for name in ordered_modules:
            h = h_inv[name]
            d = h.shape[0]
            blk = grads[lo:hi, col : col + d].to(device=h.device, dtype=h.dtype) @ h
            grads[lo:hi, col : col + d] = blk.to(device=grads.device, dtype=grads.dtype)
            col += d
    return grads


def normalize_and_aggregate_grads(
    grad_dict: dict[str, torch.Tensor],
    grad_column_names: list[str],
    unit_normalize: bool,
    device: torch.device,
    aggregate_grads: Literal["mean", "sum", "none"] = "none",
    normalize_aggregated_grad: bool = False,
) -> dict[str, torch.Tensor]:
    """Per-item unit-norm over the concatenated modules, then mean/sum over items, then
    optional unit-norm of the aggregate.  Output ``[N, d_m]`` or ``[1, d_m]`` per module."""
    if aggregate_grads == "none" and not unit_normalize:
        return {n: grad_dict[n].to(device=device) for n in grad_column_names}
    grads = {n: grad_dict[n].to(device=device, dtype=torch.float32) for n in grad_column_names}
    if unit_normalize:
        norms = torch.cat(list(grads.values()), dim=1).norm(dim=1, keepdim=True)
        grads = {k: v / norms for k, v in grads.items()}
    if aggregate_grads == "mean":
        grads = {n: g.mean(0, keepdim=True) for n, g in grads.items()}
    elif aggregate_grads == "sum":
        grads = {n: g.sum(0, keepdim=True) for n, g in grads.items()}
    elif aggregate_grads != "none":
        raise ValueError(f"Invalid aggregate_grads: {aggregate_grads}")
    if normalize_aggregated_grad:
        total = torch.cat([g.flatten() for g in grads.values()]).norm()
        grads = {n: g / total for n, g in grads.items()}
    return grads
