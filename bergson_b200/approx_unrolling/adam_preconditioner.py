"""Per-segment diagonal Adam preconditioners for the optimizer-preconditioned SOURCE
variant: read every checkpoint's ``optimizer.pt``, bias-correct the second moments,
average them within the segment and write ``P = 1 / (sqrt(v_bar + eps_root) + eps)``
oriented ``[out, in]`` to ``<run>/segment_<l>/preconditioner.safetensors``
(reference ``bergson/approx_unrolling/adam_preconditioner.py:32-187``)."""

from __future__ import annotations

from glob import glob
from pathlib import Path

import torch
from safetensors import safe_open
from safetensors.torch import save_file

from ..models import load_model
from ..utils.load_from_optimizer import (
    _second_moment,
    load_optimizer,
    optimizer_param_index_to_name,
    orient_second_moment,
)

OPTIMIZER_STATE_FILE = "optimizer.pt"


def _module_grids(hessian_dir) -> dict[str, tuple[int, int]]:
    """Module -> full ``(out, in)`` from the eigenvector shards' column counts."""
    a_dir, g_dir = Path(hessian_dir) / "eigen_activation_sharded", Path(hessian_dir) / "eigen_gradient_sharded"
    if not a_dir.is_dir() or not glob(str(g_dir / "shard_*.safetensors")):
        raise FileNotFoundError(f"No EKFAC factor shards under {hessian_dir}")
    grids = {}
    with safe_open(str(a_dir / "shard_0.safetensors"), framework="pt") as fa, \
            safe_open(str(g_dir / "shard_0.safetensors"), framework="pt") as fg:
        for name in fa.keys():
            grids[name] = (fg.get_slice(name).get_shape()[1], fa.get_slice(name).get_shape()[1])
    return grids


def _match_params(grids: dict, param_names: list[str]) -> dict[str, str]:
    """Factor module names are suffixes of parameter names (``h.0.attn.c_attn`` ->
    ``transformer.h.0.attn.c_attn.weight``); exactly one parameter must match."""
    out = {}
    for module in grids:
        suffix = f"{module}.weight"
        hits = [n for n in param_names if n == suffix or n.endswith(f".{suffix}")]
        if len(hits) != 1:
            raise KeyError(f"Module {module!r} matched {len(hits)} params ({hits}); expected exactly one *.{suffix}.")
        out[module] = hits[0]
    return out


def _adam_hparams(opt: dict) -> tuple[float, float, float]:
    groups = opt.get("param_groups", [])
    betas = groups[0].get("betas") if groups else None
    eps = groups[0].get("eps") if groups else None
    if betas is None or eps is None:
        raise ValueError("optimizer.pt has no param_groups betas/eps; regenerate it with "
                         "TrainingConfig.save_optimizer_state.")
    return float(betas[1]), float(eps), float(groups[0].get("eps_root", 0.0))


def _extract_v_hat(opt: dict, index_to_name: dict[int, str], beta2: float) -> dict[str, torch.Tensor]:
    out = {}
    for idx, entry in opt["state"].items():
        name = entry.get("param_name") or index_to_name.get(int(idx))
        if name is None:
            continue
        if "step" not in entry:
            raise ValueError(f"optimizer.pt state entry {idx} has no step; regenerate it with save_optimizer_state.")
        step = int(entry["step"])
        sm = _second_moment(entry)
        if sm is None or sm[0] != "adam":
            continue
        nu = sm[1].float()
        out[name] = nu / (1.0 - beta2**step) if step > 0 else torch.zeros_like(nu)
    return out


def build_segment_preconditioners(run_path, method: str, checkpoints: list[str], segments: int) -> list[Path]:
    base = Path(run_path)
    per = len(checkpoints) // segments
    reference = load_model(checkpoints[0], dtype=torch.float32, device="cpu")
    paths = []
    for seg in range(segments):
        ckpts = checkpoints[seg * per : (seg + 1) * per]
        v_sum: dict[str, torch.Tensor] = {}
        eps = eps_root = 0.0
        for ckpt in ckpts:
            if not (Path(ckpt) / OPTIMIZER_STATE_FILE).exists():
                raise FileNotFoundError(f"use_adam_preconditioner requires {Path(ckpt) / OPTIMIZER_STATE_FILE}.")
            opt = load_optimizer(str(ckpt))
            beta2, eps, eps_root = _adam_hparams(opt)
            for name, v in _extract_v_hat(opt, optimizer_param_index_to_name(opt, reference), beta2).items():
                v_sum[name] = v_sum[name] + v if name in v_sum else v
        grids = _module_grids(base / f"segment_{seg}" / method)
        pre = {}
        for module, pname in _match_params(grids, list(v_sum)).items():
            try:
                layer = reference.get_submodule(pname.removesuffix(".weight"))
            except AttributeError:
                layer = None
            p = 1.0 / ((v_sum[pname] / len(ckpts) + eps_root).sqrt() + eps)
            oriented = orient_second_moment(p, *grids[module], layer=layer)
            if oriented is None:
                raise ValueError(f"Second moments for {module!r} have shape {tuple(p.shape)}; expected {grids[module]}.")
            pre[module] = oriented
        out = base / f"segment_{seg}" / "preconditioner.safetensors"
        save_file(pre, str(out))
        paths.append(out)
    return paths
