"""Parameter sharding for the twice-differentiable trainer.

Every trainable parameter is stored as this rank's block of rows (dim 0 padded to a
multiple of the world size).  ``gather_params`` rebuilds the full tensors with the
differentiable all-gather of ``collectives``; its backward is a reduce-scatter, so
parameter gradients come back sharded (summed over ranks), and the backward of that is
again an all-gather: the whole step stays differentiable to any order.  The reference
reaches the same behaviour with DTensor ``Shard(0)`` parametrisations and a patched
redistribute backward (``bergson/magic/fsdp.py:20-87``, ``dtensor_patch.py``).
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist
from torch import Tensor

from .collectives import all_gather_rows, finish_all_gather_rows, start_all_gather_rows


def shallow_copy(tensors: dict[str, Tensor]) -> dict[str, Tensor]:
    """New tensor objects sharing storage (so in-place state edits do not alias the module)."""
    return {k: v.detach().clone() if v.device.type == "meta" else v.detach().view_as(v) for k, v in tensors.items()}


def _world() -> tuple[int, int]:
    if dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


def shard_param(full: Tensor) -> Tensor:
    """This rank's rows of ``full`` (zero-padded so that dim 0 divides evenly)."""
    rank, world = _world()
    if world == 1 or full.ndim == 0:
        return full
    rows = -(-full.shape[0] // world)
    pad = rows * world - full.shape[0]
    if pad:
        full = torch.cat([full, full.new_zeros(pad, *full.shape[1:])])
    return full[rank * rows : (rank + 1) * rows].clone()


def gather_param(shard: Tensor, full_shape: torch.Size) -> Tensor:
    """Differentiable inverse of ``shard_param``.  Its adjoint is a *summing* reduce-scatter;
    the trainer averages over ranks by scaling each rank's loss with ``1 / world`` instead,
    which keeps second-order terms correctly scaled as well."""
    _, world = _world()
    if world == 1 or len(full_shape) == 0:
        return shard
    return all_gather_rows(shard)[: full_shape[0]]


def simple_fsdp(params: dict[str, Tensor]) -> tuple[dict[str, Tensor], dict[str, torch.Size]]:
    """Shard a parameter dict; returns ``(shards, full_shapes)``."""
    shapes = {k: p.shape for k, p in params.items()}
    return {k: shard_param(p) for k, p in params.items()}, shapes


def gather_params(shards: dict[str, Tensor], shapes: dict[str, torch.Size]) -> dict[str, Tensor]:
    return {k: gather_param(s, shapes[k]) for k, s in shards.items()}


# --------------------------------------------------------------------------- #
# Per-module gathering
# --------------------------------------------------------------------------- #


class _Regather:
    """What autograd keeps instead of a gathered parameter: enough to gather it again."""

    __slots__ = ("key",)

    def __init__(self, key: str):
        self.key = key


class LazyGather:
    """Run a module whose trainable parameters live as row shards, gathering each
    parameter only around the forward of the module that owns it.

    * A forward pre-hook on every parameter-owning module gathers that module's parameters
      (differentiable all-gather), the forward hook drops them again: at any moment only the
      running module's full parameters exist, instead of the whole model's.
    * Operations save their weight for the backward pass; ``saved_tensors_hooks`` replaces
      each saved gathered parameter by a marker, and unpacking gathers it again from the
      shard, *with* autograd history, so the backward of the backward still reaches the
      shard (what a metagradient needs).  Peak memory is shards + one module's parameters +
      activations, at the price of a second all-gather per parameter in the backward pass.

    * With ``prefetch`` (``BERGSON_B200_FSDP_PREFETCH=1``), while a module runs, the all-gather
      of the module that ran after it in the previous forward pass is already under way; its
      pre-hook then only waits for the data.  The call order is learnt during the first pass
      and kept on the model.  Re-gathers of the backward pass are not prefetched.

    The reference gets the same effect from DTensor parametrisations
    (``bergson/magic/fsdp.py``); its full parameters are likewise gathered per module call.
    """

    def __init__(self, model: torch.nn.Module, shards: dict[str, Tensor], shapes: dict[str, torch.Size],
                 prefetch: bool | None = None):
        self.model, self.shards, self.shapes = model, shards, shapes
        self.prefetch = os.environ.get("BERGSON_B200_FSDP_PREFETCH") == "1" if prefetch is None else prefetch
        self.prefetch_hits = 0  # gathers whose data had been requested ahead of time
        self._started: dict[str, tuple] = {}
        self._seen: list[torch.nn.Module] = []
        self.gathers = 0  # forward gathers + re-gathers (read by the tests)
        self.packed = 0   # saved gathered parameters that were replaced by a marker
        key_of = {}
        for name, p in model.named_parameters(remove_duplicate=False):
            key_of.setdefault(id(p), name)
        # (module, attribute, state key) for every trainable parameter slot, tied slots included
        self.slots: dict[torch.nn.Module, list[tuple[str, str]]] = {}
        for mod in model.modules():
            for leaf, p in mod._parameters.items():
                if p is not None and key_of.get(id(p)) in shards:
                    self.slots.setdefault(mod, []).append((leaf, key_of[id(p)]))
        self._live: dict[int, str] = {}
        self._handles: list = []
        self._originals: dict[tuple[int, str], torch.nn.Parameter] = {}

    def _gather(self, key: str) -> Tensor:
        self.gathers += 1
        return gather_param(self.shards[key], self.shapes[key])

    def _gather_now_or_finish(self, key: str) -> Tensor:
        handle = self._started.pop(key, None)
        if handle is None:
            return self._gather(key)
        self.gathers += 1
        self.prefetch_hits += 1
        return finish_all_gather_rows(self.shards[key], handle)[: self.shapes[key][0]]

    def _start_next(self, mod) -> None:
        """Request the parameters of the module that followed ``mod`` in the last pass."""
        order = getattr(self.model, "_lazy_gather_order", None)
        if not order or not dist.is_initialized() or dist.get_world_size() == 1:
            return
        try:
            nxt = order[order.index(mod) + 1]
        except (ValueError, IndexError):
            return
        for _, key in self.slots.get(nxt, ()):
            if key not in self._started and len(self.shapes[key]) > 0:
                self._started[key] = start_all_gather_rows(self.shards[key])

    def _pre(self, mod, args):
        if self.prefetch:
            if mod not in self._seen:
                self._seen.append(mod)
        for leaf, key in self.slots[mod]:
            full = self._gather_now_or_finish(key) if self.prefetch else self._gather(key)
            self._live[id(full)] = key
            self._originals[(id(mod), leaf)] = mod._parameters.pop(leaf)
            setattr(mod, leaf, full)  # plain attribute: keeps the autograd history of the gather
        if self.prefetch:
            self._start_next(mod)

    def _post(self, mod, args, output):
        for leaf, _ in self.slots[mod]:
            full = mod.__dict__.pop(leaf, None)
            if full is not None:
                self._live.pop(id(full), None)
            mod._parameters[leaf] = self._originals.pop((id(mod), leaf))

    def _pack(self, t: Tensor):
        key = self._live.get(id(t))
        if key is None:
            return t
        self.packed += 1
        return _Regather(key)

    def _unpack(self, obj):
        return self._gather(obj.key) if isinstance(obj, _Regather) else obj

    def __enter__(self):
        for mod in self.slots:
            self._handles.append(mod.register_forward_pre_hook(self._pre))
            self._handles.append(mod.register_forward_hook(self._post, always_call=True))
        self._saved = torch.autograd.graph.saved_tensors_hooks(self._pack, self._unpack)
        self._saved.__enter__()
        return self

    def __exit__(self, *exc):
        for handle in self._started.values():  # requested but never used (the call order changed)
            handle[0].wait()
        self._started.clear()
        if self.prefetch and self._seen:
            self.model._lazy_gather_order = list(self._seen)
        self._saved.__exit__(*exc)
        for h in self._handles:
            h.remove()
        self._handles.clear()
        return False
