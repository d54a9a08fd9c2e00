"""Run a module with externally held parameter / buffer tensors.

The trainer keeps parameters in a ``TrainerState`` and calls the model functionally;
``swap_parameters`` is the context-manager form of that (reference
``bergson/magic/swap.py``): inside the block the module's named parameters and buffers
are the given tensors (graph-preserving), afterwards the originals are restored.
"""

from __future__ import annotations

from contextlib import contextmanager

import torch.nn as nn
from torch import Tensor


def _owner(model: nn.Module, name: str) -> tuple[nn.Module, str]:
    mod_name, _, leaf = name.rpartition(".")
    return (model.get_submodule(mod_name) if mod_name else model), leaf


@contextmanager
def swap_parameters(model: nn.Module, params: dict[str, Tensor], buffers: dict[str, Tensor] | None = None, *,
                    strict: bool = False, preserve_graph: bool = True):
    """Yields the dict of tensors now acting as the module's parameters.  With
    ``preserve_graph=False`` they are detached leaves that require grad."""
    if strict:
        missing = {k for k, p in model.named_parameters() if p.requires_grad} - set(params)
        if missing:
            raise KeyError(f"swap_parameters(strict=True): no tensor given for {sorted(missing)[:5]}")
    active = {k: (v if preserve_graph else v.detach().requires_grad_(True)) for k, v in params.items()}
    saved_p, saved_b = {}, {}
    try:
        for name, t in active.items():
            mod, leaf = _owner(model, name)
            saved_p[name] = mod._parameters.pop(leaf)
            setattr(mod, leaf, t)  # plain attribute: keeps t's autograd history
        for name, t in (buffers or {}).items():
            mod, leaf = _owner(model, name)
            saved_b[name] = mod._buffers[leaf]
            mod._buffers[leaf] = t
        yield active
    finally:
        for name, orig in saved_p.items():
            mod, leaf = _owner(model, name)
            if leaf in mod.__dict__:
                del mod.__dict__[leaf]
            mod._parameters[leaf] = orig
        for name, orig in saved_b.items():
            mod, leaf = _owner(model, name)
            mod._buffers[leaf] = orig
