"""Optimizer second moments <-> gradient normalisers.

Reads ``optimizer.pt`` files written by HF ``Trainer`` (Adam/AdamW ``exp_avg_sq``,
Adafactor ``exp_avg_sq_row/col``, bitsandbytes 8-bit Adam ``state2``) or by this
package's trainer, and turns the weight (and optionally bias) moments of every Linear
into ``AdamNormalizer`` / ``AdafactorNormalizer`` keyed by the module name relative to
``model.base_model``.  ``save_second_moments_as_optimizer_pt`` writes the trainer's AdamW
moments in the same layout (reference ``bergson/utils/load_from_optimizer.py``).
"""

from __future__ import annotations

import re
from enum import Enum
from pathlib import Path

import torch
import torch.distributed as dist
from torch import nn

from ..gradients import AdafactorNormalizer, AdamNormalizer, LayerAdapter, Normalizer


def load_optimizer(optimizer_state: str) -> dict:
    """Local file, local directory containing ``optimizer.pt``, or
    ``hf://<repo>[@<revision>][/<path>]``."""
    if optimizer_state.startswith("hf://"):
        from huggingface_hub import hf_hub_download

        rest = optimizer_state[len("hf://"):]
        parts = rest.split("/")
        repo = "/".join(parts[:2])
        sub = "/".join(parts[2:])
        revision = None
        if "@" in repo:
            repo, revision = repo.split("@", 1)
        if sub.endswith((".pt", ".pth")):
            filename = sub
        else:
            filename = f"{sub.rstrip('/')}/optimizer.pt" if sub else "optimizer.pt"
        path = Path(hf_hub_download(repo_id=repo, filename=filename, revision=revision))
    else:
        local = Path(optimizer_state)
        if not local.exists():
            raise FileNotFoundError(
                f"Optimizer state '{optimizer_state}' is not a local path and does not start with 'hf://'.")
        path = local / "optimizer.pt" if local.is_dir() else local
    return torch.load(path, map_location="cpu", weights_only=False)


def _second_moment(entry) -> tuple[str, object] | None:
    """("adam", v) | ("adafactor", (row, col)) | None for one optimizer-state entry."""
    if not isinstance(entry, dict):
        return None
    if "exp_avg_sq" in entry:
        return "adam", entry["exp_avg_sq"]
    if "exp_avg_sq_row" in entry:
        return "adafactor", (entry["exp_avg_sq_row"], entry.get("exp_avg_sq_col"))
    bnb = entry.get("__bnb_optimizer_quant_state__")
    if isinstance(bnb, dict) and "state2" in bnb:
        return "adam", bnb["state2"]
    return None


class OptimizerStateFormat(Enum):
    """How one parameter's second moment is stored: a full tensor (Adam, 8-bit Adam, Adafactor's 1-D
    parameters) or Adafactor's row / column factors."""

    UNFACTORED = 1
    FACTORED = 2


def get_optimizer_state_format(param_state) -> OptimizerStateFormat | None:
    """Format of one optimizer-state entry, None when it carries no second moment."""
    sm = _second_moment(param_state)
    if sm is None:
        return None
    return OptimizerStateFormat.UNFACTORED if sm[0] == "adam" else OptimizerStateFormat.FACTORED


def get_unfactored_second_moment(state: dict) -> torch.Tensor:
    """The full second-moment tensor of an UNFACTORED entry."""
    sm = _second_moment(state)
    if sm is None or sm[0] != "adam":
        raise KeyError("entry has no unfactored second moment (exp_avg_sq / 8-bit state2)")
    return sm[1]  # type: ignore[return-value]


def _base_model_prefix(model) -> str:
    base = getattr(model, "base_model", model)
    if base is model:
        return ""
    for name, module in model.named_modules():
        if module is base:
            return f"{name}." if name else ""
    return ""


def orient_second_moment(t: torch.Tensor, out_dim: int, in_dim: int, layer=None) -> torch.Tensor | None:
    """``t`` as ``[out, in]``.  The layer type decides for square weights (Conv1D stores
    ``[in, out]``); without a layer the shape decides.  None if nothing fits."""
    if layer is not None and isinstance(layer, LayerAdapter.supported_modules):
        o = t.T if LayerAdapter.weight_transposed(layer) else t
        return o.contiguous() if tuple(o.shape) == (out_dim, in_dim) else None
    if tuple(t.shape) == (out_dim, in_dim):
        return t.contiguous()
    if tuple(t.shape) == (in_dim, out_dim):
        return t.T.contiguous()
    return None


def optimizer_param_index_to_name(optimizer_pt: dict, model) -> dict[int, str]:
    """State index -> parameter name.  One param group: ``named_parameters()`` order.  Two
    groups: HF Trainer's decay / no-decay split (norm layers and biases do not decay)."""
    groups = optimizer_pt.get("param_groups", [])
    named = [(n, p) for n, p in model.named_parameters()]
    if len(groups) <= 1:
        mapping = {i: n for i, (n, _) in enumerate(named)}
    else:
        norm_types = (nn.LayerNorm,)
        norm_params = set()
        for mname, mod in model.named_modules():
            if isinstance(mod, norm_types) or "norm" in type(mod).__name__.lower():
                norm_params.update(f"{mname}.{p}" if mname else p for p, _ in mod.named_parameters(recurse=False))
        trainable = [(n, p) for n, p in named if p.requires_grad]
        decay = [n for n, _ in trainable if n not in norm_params and "bias" not in n]
        no_decay = [n for n, _ in trainable if n not in set(decay)]
        sizes = [len(g.get("params", [])) for g in groups]
        if len(groups) != 2 or sizes != [len(decay), len(no_decay)]:
            raise ValueError(
                f"Cannot map optimizer.pt state indices to params: {len(groups)} param groups of sizes {sizes} "
                f"do not match the decay/no-decay split {[len(decay), len(no_decay)]} for this model.")
        mapping = dict(zip([i for g in groups for i in g["params"]], decay + no_decay))
    shapes = {n: tuple(p.shape) for n, p in named}
    for idx, entry in optimizer_pt.get("state", {}).items():
        if not isinstance(entry, dict) or "param_name" in entry or "exp_avg_sq" not in entry:
            continue
        name = mapping.get(int(idx))
        if name is not None and tuple(entry["exp_avg_sq"].shape) != shapes.get(name):
            raise ValueError(
                f"optimizer.pt state entry {idx} has second-moment shape {tuple(entry['exp_avg_sq'].shape)} but "
                f"maps to {name!r} of shape {shapes.get(name)}; the index layout is not the expected one.")
    return mapping


def _bias_moment(layer_name: str, index_to_name: dict[int, str], state: dict, include_bias: bool):
    if not include_bias:
        return None
    bias_name = layer_name + ".bias"
    for entry in state.values():
        if isinstance(entry, dict) and entry.get("param_name") == bias_name:
            sm = _second_moment(entry)
            return sm[1] if sm and sm[0] == "adam" else None
    for idx, name in index_to_name.items():
        if name == bias_name:
            sm = _second_moment(state.get(idx))
            return sm[1] if sm and sm[0] == "adam" else None
    return None


def get_normalizers(optimizer_state: dict, target_param_index_to_name: dict[int, str], target_modules: set[str] | None,
                    adapter_suffix: str, include_bias: bool, device, base_prefix: str = "", model=None) -> dict[str, Normalizer]:
    """Normalisers of every ``<layer>.weight`` entry of ``optimizer_state["state"]``, keyed by the
    module name relative to the base model (+ ``adapter_suffix``).  An entry's recorded
    ``param_name`` wins over its positional index; ``model`` (optional) tells which layers store
    their weight transposed."""
    index_to_name = target_param_index_to_name
    out: dict[str, Normalizer] = {}
    for idx, entry in optimizer_state["state"].items():
        name = (entry.get("param_name") if isinstance(entry, dict) else None) or index_to_name.get(int(idx))
        if name is None or not name.endswith(".weight"):
            continue
        layer = name.removesuffix(".weight")
        module_name = layer.removeprefix("base_model.").removeprefix(base_prefix) + adapter_suffix
        if target_modules is not None and module_name not in target_modules:
            continue
        sm = _second_moment(entry)
        if sm is None:
            print("Unrecognized format, skipping normalizer for param_idx", idx)
            continue
        bias = _bias_moment(layer, index_to_name, optimizer_state["state"], include_bias)
        bias = bias.to(device) if bias is not None else None
        try:
            module = model.get_submodule(layer) if model is not None else None
        except AttributeError:
            module = None
        transposed = module is not None and isinstance(module, LayerAdapter.supported_modules) and \
            LayerAdapter.weight_transposed(module)
        if sm[0] == "adam":
            v = sm[1]
            if v.ndim != 2:
                continue
            out[module_name] = AdamNormalizer((v.T.contiguous() if transposed else v).to(device), bias)
        else:
            row, col = sm[1]
            if row.ndim != 1 or col is None:
                continue
            if transposed:  # factored over the stored [in, out] layout
                row, col = col, row
            out[module_name] = AdafactorNormalizer(row.to(device), col.to(device), bias)
    return out


def load_from_optimizer(model, optimizer_state: str, include_bias: bool = False,
                        target_modules: set[str] | None = None) -> dict[str, Normalizer]:
    """Normalisers for every Linear whose weight has second moments in the checkpoint."""
    opt = load_optimizer(optimizer_state)
    adapter_suffix = ""
    is_peft = type(model).__name__.startswith("Peft") and hasattr(model, "peft_config")
    if is_peft:
        from peft import get_peft_model_state_dict

        index_to_name = {i: n for i, n in enumerate(get_peft_model_state_dict(model))}
        adapters = list(model.peft_config)
        if len(adapters) == 1:
            adapter_suffix = "." + adapters[0]
        base_prefix = ""
    else:
        index_to_name = optimizer_param_index_to_name(opt, model)
        base_prefix = _base_model_prefix(model)
    device = next(model.parameters()).device
    out = get_normalizers(opt, index_to_name, target_modules, adapter_suffix, include_bias, device,
                          base_prefix=base_prefix, model=model)
    assert out, (f"No optimizer second moments found in '{optimizer_state}'. Ensure the checkpoint was saved from "
                 "an Adam-family or Adafactor optimizer.")
    kinds = ", ".join(sorted({type(n).__name__ for n in out.values()}))
    print(f"Loaded {len(out)} normalizers ({kinds}) from '{optimizer_state}'")
    return out


def _canonical_param_name(name: str) -> str:
    return re.sub(r"\.parametrizations\.([^.]+)\.original$", r".\1", name)


def save_second_moments_as_optimizer_pt(model: nn.Module, opt_state, path, step: int | None = None,
                                        betas: tuple[float, float] | None = None, eps: float | None = None,
                                        eps_root: float | None = None, full_shapes: dict | None = None) -> int:
    """Write ``{"state": {idx: {"exp_avg_sq", "param_name", "step"?}}, "param_groups":
    [{"params", "betas"?, "eps"?, "eps_root"?}]}`` with ``idx`` the position in
    ``model.named_parameters()``.  ``opt_state`` is the trainer's AdamW state (``{"nu":
    {name: tensor}}``); row-sharded moments are gathered (every rank must call; rank 0
    writes).  Returns the number of entries."""
    if not isinstance(opt_state, dict) or "nu" not in opt_state:
        raise ValueError("opt_state has no second-moment (`nu`) field; save_optimizer_state supports AdamW only.")
    main = not dist.is_initialized() or dist.get_rank() == 0
    shapes = {n: tuple(p.shape) for n, p in model.named_parameters()}
    moments = {}
    for name, nu in opt_state["nu"].items():
        if nu is None:
            continue
        t = nu.detach()
        want = tuple(full_shapes[name]) if full_shapes and name in full_shapes else shapes.get(name)
        if want is not None and tuple(t.shape) != want and dist.is_initialized():
            parts = [torch.empty_like(t) for _ in range(dist.get_world_size())]
            dist.all_gather(parts, t.contiguous())
            t = torch.cat(parts)[: want[0]]
        if main:
            moments[name] = t.cpu()
    state, ids = {}, []
    for idx, (name, _) in enumerate(model.named_parameters()):
        if name in moments:
            state[idx] = {"exp_avg_sq": moments[name], "param_name": _canonical_param_name(name)}
            if step is not None:
                state[idx]["step"] = torch.tensor(step)
            ids.append(idx)
    if not main:
        return len(ids)
    group: dict = {"params": ids}
    if betas is not None:
        group["betas"] = tuple(betas)
    if eps is not None:
        group["eps"] = eps
    if eps_root is not None:
        group["eps_root"] = eps_root
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    torch.save({"state": state, "param_groups": [group]}, path)
    print(f"Saved {len(state)} optimizer second moments to '{path}'")
    return len(state)
