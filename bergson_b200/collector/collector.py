"""Hook-based collection engine.

``HookCollectorBase`` attaches a forward hook to every supported layer and, from
inside it, a tensor hook on the layer's output, so that the subclass sees the layer
input ``a`` [N, S, I] and the output gradient ``g`` [N, S, O].  The per-example weight
gradient is ``g^T a``; with projection the stored value is ``P_out g^T a P_in^T``
computed as ``(g P_out^T)^T (a P_in^T)`` (reference
``bergson/collector/collector.py:518-743``).

Two execution paths produce the same numbers:

* the **torch path** (any device, every option), and
* the **fused path** (CUDA, 16-bit activations, ``projection_dim`` 8..64, no Adam
  normaliser): in-tree layers emit ``a P_in^T`` and ``g P_out^T`` as side outputs of their
  own forward and input-gradient GEMMs (``ops.linear`` taps); a contraction kernel turns both
  into the example's ``p x p`` block (or per-token rows) in the fp32 row accumulator of the
  batch at the module's column offset.  Adafactor row and column scales are folded into the
  projection matrices once; without a normaliser a bias column is the constant vector
  ``P_in[:, I]`` added to the projected activations.  Layers that are not in-tree take the hook form of the same path
  (``projection_dim == 16``): a skinny projection kernel in the forward hook, and one kernel
  in the backward hook that projects ``g`` and contracts.
"""

from __future__ import annotations

import functools
import hashlib
import math
import os
from abc import ABC, abstractmethod
from contextlib import ContextDecorator, nullcontext
from dataclasses import astuple, dataclass, field
from fnmatch import fnmatchcase
from typing import Callable, Literal, Mapping, Optional

import numpy as np
import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor
from tqdm.auto import tqdm

from .. import ops
from ..config import AttentionConfig, HessianConfig, IndexConfig
from ..data import compute_num_token_grads, pad_and_tensor
from ..gradients import AdafactorNormalizer, AdamNormalizer, GradientProcessor, LayerAdapter
from ..models.common import NativeCausalLM
from ..utils.logger import get_logger
from ..utils.utils import assert_type

FUSED_PROJECTION_DIM = 16


def create_projection_matrix(
    identifier: str,
    m: int,
    n: int,
    dtype: torch.dtype,
    device: torch.device,
    projection_type: Literal["normal", "rademacher"] = "normal",
    projection_scale: Literal["jl", "row_norm"] = "jl",
) -> Tensor:
    """Deterministic ``[m, n]`` projection seeded by ``md5(identifier) mod (2^63 - 1)``.

    ``rademacher`` unpacks bits of a numpy PCG64 byte stream (portable across devices);
    ``normal`` draws from a ``torch.Generator`` of ``device`` (the stream is
    device-type specific).  ``jl`` scales by ``1/sqrt(m)``; ``row_norm`` normalises rows.
    """
    seed = int.from_bytes(hashlib.md5(identifier.encode("utf-8")).digest(), "big") % (2**63 - 1)
    if projection_type == "normal":
        gen = torch.Generator(device).manual_seed(seed)
        A = torch.randn(m, n, device=device, dtype=dtype, generator=gen)
    elif projection_type == "rademacher":
        raw = np.random.Generator(np.random.PCG64(seed)).bytes((m * n + 7) // 8)
        bits = np.unpackbits(np.frombuffer(raw, dtype=np.uint8))[: m * n].reshape(m, n)
        A = torch.from_numpy(bits).to(device, dtype=dtype).add_(-0.5).mul_(2)
    else:
        raise ValueError(f"Unknown projection type: {projection_type}")
    if projection_scale == "row_norm":
        A /= A.norm(dim=1, keepdim=True)
    else:
        A /= math.sqrt(m)
    return A


TAP_PROJECTION_DIMS = (8, 16, 32, 64)


def _tap_module_types() -> tuple[type, ...]:
    from ..models.common import Conv1D
    from ..ops.linear import Linear

    return (Linear, Conv1D)


class _FusedTap:
    """Collector side of ``ops.linear``'s tap: hands the layer its two projection operands and
    turns the projected activations / output gradients that come back into the module's block
    of the batch's row accumulator."""

    def __init__(self, collector: "HookCollectorBase", name: str):
        self.collector, self.name = collector, name

    def operands(self, module: nn.Module, x: Tensor):
        c = self.collector
        if not c._tap_accepts(module, x):
            return None
        module._tapped = True  # the forward hook that follows skips this call
        i = getattr(module, LayerAdapter.in_attr(module))
        o = getattr(module, LayerAdapter.out_attr(module))
        return c._tap_matrices(self.name, o, i, x.device, x.dtype, bool(module._collect_bias))

    def collect(self, module: nn.Module, a_proj: Tensor, g_proj: Tensor, lead_shape) -> None:
        from ..ops import native

        c = self.collector
        p = c.per_module_projection_dim
        acc = c._row_acc[: c._fused_rows]
        off = c._col_offsets[self.name]
        bias_col = c._tap_bias.get(self.name)
        if bias_col is not None:
            # The bias gradient is the gradient for a constant input of one: its projection adds
            # the same vector (the bias column of P_in) to every token's projected activation.
            a_proj = a_proj + bias_col
        if c.attribute_tokens:
            native.proj_token_rows(g_proj, a_proj, c._token_index, acc, p, off)
        else:
            n, s = int(lead_shape[0]), int(lead_shape[1])
            native.proj_contract(g_proj, a_proj, acc, n, s, p, off)
        c._fused_written.add(self.name)
        c._tap_calls += 1


@dataclass
class HookCollectorBase(ContextDecorator, ABC):
    """Base class of every collector.

    Subclasses implement ``setup``, ``teardown``, ``backward_hook`` and
    ``process_batch``; ``forward_hook`` may be overridden too.  Use as a context
    manager around forward/backward passes; ``with_batch(mask)`` passes the batch's
    collection mask to the hooks.
    """

    model: nn.Module
    filter_modules: str | None = None
    target_modules: set[str] | None = None
    processor: GradientProcessor = field(default_factory=GradientProcessor)
    attention_cfgs: dict[str, AttentionConfig] = field(default_factory=dict)
    attribute_tokens: bool = False
    lo: float = float("-inf")
    hi: float = float("inf")
    mod_grads: dict = field(default_factory=dict)
    save_dtype: torch.dtype = torch.float32

    logger = get_logger("HookCollectorBase", level="INFO")

    def __post_init__(self):
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.world_size = dist.get_world_size() if dist.is_initialized() else 1
        self._fwd_hooks: list = []
        self._current_collection_mask: Tensor | None = None
        # fused-path state (enabled by subclasses through ``enable_fused``)
        self._fused_enabled = False
        self._tap_dim_ok = False
        self._hook_fused_ok = False
        self._tap_calls = 0  # modules x batches collected through GEMM taps (diagnostic)
        self._row_acc: Tensor | None = None
        self._col_offsets: dict[str, int] = {}
        self._fused_mats: dict = {}
        self._tap_bias: dict[str, Tensor] = {}  # name -> bias column of the input projection
        self._fused_written: set[str] = set()

        self.target_info = self.discover_targets(
            self.model, self.target_modules, self.processor.include_bias, self.filter_modules
        )
        # Tensor-parallel shards: name -> ("out" | "in", lo, hi, full size of the split dim).
        self._tp_shards = {
            n: m._tp_shard for n, m in self.model.named_modules() if n in self.target_info and hasattr(m, "_tp_shard")
        }
        if unknown := set(self.attention_cfgs) - set(self.target_info):
            raise ValueError(
                f"attention_cfgs contains module names not found in the model: {unknown}. "
                f"Available modules: {set(self.target_info)}"
            )
        self.setup()

    # ------------------------------------------------------------------ discovery

    @staticmethod
    def discover_targets(
        model: nn.Module,
        target_modules: set[str] | None = None,
        include_bias: bool = False,
        filter_modules: str | None = None,
    ) -> dict[str, tuple[torch.device, torch.Size, bool]]:
        """``{name: (device, [O, I], collect_bias)}`` in ``named_modules()`` order."""
        pats = [p.strip() for p in filter_modules.split(",")] if filter_modules else []
        out = {}
        for name, layer in model.named_modules():
            if not isinstance(layer, LayerAdapter.supported_modules):
                continue
            if target_modules is not None and name not in target_modules:
                continue
            if any(fnmatchcase(name, p) for p in pats):
                continue
            o = getattr(layer, LayerAdapter.out_attr(layer))
            i = getattr(layer, LayerAdapter.in_attr(layer))
            has_bias = getattr(layer, "bias", None) is not None and include_bias
            out[name] = (layer.weight.device, torch.Size([o, i]), has_bias)
        return out

    @staticmethod
    def get_head_name(name: str, head_idx: int) -> str:
        return f"{name}.head_{head_idx}"

    @staticmethod
    def split_head_name(name: str) -> tuple[str, int] | None:
        base, sep, idx = name.rpartition(".head_")
        return (base, int(idx)) if sep and idx.isdigit() else None

    @staticmethod
    def split_attention_heads(fn):
        """Decorator for ``backward_hook``: call it once per head for modules listed in
        ``attention_cfgs``, with the module renamed ``<name>.head_<h>`` and its output
        size narrowed to the head size."""

        @functools.wraps(fn)
        def wrapper(self, module, g):
            name = module._name
            cfg = self.attention_cfgs.get(name)
            if cfg is None:
                return fn(self, module, g)
            num_heads, head_size, head_dim = astuple(cfg)
            attr = LayerAdapter.out_attr(module)
            full = getattr(module, attr)
            assert num_heads * head_size == full, (
                f"{name}: num_heads * head_size = {num_heads * head_size} does not cover the "
                f"module's {full} output features"
            )
            setattr(module, attr, head_size)
            try:
                for h in range(num_heads):
                    module._name = self.get_head_name(name, h)
                    fn(self, module, torch.narrow(g, head_dim, h * head_size, head_size))
            finally:
                module._name = name
                setattr(module, attr, full)

        return wrapper

    def normalizer_for(self, name: str):
        """Normaliser of ``name``; a ``.head_<h>`` module gets its parent's, sliced."""
        norm = self.processor.normalizers.get(name)
        if norm is not None:
            return norm
        split = self.split_head_name(name)
        if split is None:
            return None
        base, h = split
        norm = self.processor.normalizers.get(base)
        if norm is None or base not in self.attention_cfgs:
            return norm
        size = self.attention_cfgs[base].head_size
        sl = slice(h * size, (h + 1) * size)
        bias = norm.bias_avg_sq[sl] if norm.bias_avg_sq is not None else None
        if isinstance(norm, AdamNormalizer):
            return AdamNormalizer(norm.weight_avg_sq[sl], bias)
        if isinstance(norm, AdafactorNormalizer):
            return AdafactorNormalizer(norm.row[sl], norm.col, bias)
        return norm

    @property
    def per_module_projection_dim(self) -> int | None:
        if self.processor.projection_target == "global":
            return None
        return self.processor.projection_dim or None

    def shapes(self) -> Mapping[str, torch.Size]:
        """Shape of each stored gradient block, in store column order."""
        if self.processor.projection_target == "global":
            assert self.processor.projection_dim is not None
            return {"gradients": torch.Size((self.processor.projection_dim,))}
        p = self.per_module_projection_dim
        out: dict[str, torch.Size] = {}
        for name, (_, (o, i), bias) in self.target_info.items():
            cfg = self.attention_cfgs.get(name)
            if p is not None:
                block = torch.Size((p, p))
            else:
                dims = [o, i]
                if cfg is not None:
                    dims[cfg.head_dim - 2] = cfg.head_size
                if bias:
                    dims[-1] += 1
                block = torch.Size(dims)
            if cfg is not None:
                for h in range(cfg.num_heads):
                    out[self.get_head_name(name, h)] = block
            else:
                out[name] = block
        return out

    def projection(self, name: str, m: int, n: int, role: Literal["left", "right", "single"], device, dtype) -> Tensor:
        """Cached ``role`` projection for parameter ``name``."""
        key = (name, role, device)
        cache = self.processor._projection_matrices
        if key not in cache:
            shard = self._tp_shards.get(name)
            split = shard is not None and ((role == "left" and shard[0] == "out") or (role == "right" and shard[0] == "in"))
            full_n = shard[3] if split else n
            mat = create_projection_matrix(
                f"{name}/{role}", m, full_n, dtype, device,
                self.processor.projection_type, self.processor.projection_scale,
            )
            # A rank that holds a slice of the split dimension projects with the matching
            # columns of the full matrix; the partial results are summed over the group.
            cache[key] = mat[:, shard[1] : shard[2]].contiguous() if split else mat
        return cache[key]

    def adafactor_scales(self, name: str, norm: AdafactorNormalizer) -> tuple[Tensor, Tensor]:
        """(row scale [O_local], column scale [I_local]); statistics are those of the whole
        layer, sliced to this rank's shard under tensor parallelism."""
        row, col = norm.row_scale(), norm.col_scale()
        shard = self._tp_shards.get(name)
        if shard is not None:
            dim, lo, hi, full = shard
            if dim == "out" and row.shape[0] == full:
                row = row[lo:hi]
            if dim == "in" and col.shape[0] == full:
                col = col[lo:hi]
        return row, col

    def accumulate_global_projection(self, name: str, P: Tensor) -> bool:
        """``projection_target == "global"``: add ``P @ R_name^T`` into the single
        ``"gradients"`` entry and return True; otherwise return False."""
        if self.processor.projection_target != "global":
            return False
        assert self.processor.projection_dim is not None
        R = self.projection(name, self.processor.projection_dim, P.shape[1], "single", P.device, P.dtype)
        proj = P @ R.T
        if "gradients" in self.mod_grads:
            self.mod_grads["gradients"].add_(proj)
        else:
            self.mod_grads["gradients"] = proj
        return True

    def finalize_global_projection(self) -> None:
        if self.processor.projection_target == "global" and "gradients" in self.mod_grads:
            self.mod_grads["gradients"] = self.mod_grads["gradients"].to(
                device="cpu", dtype=self.save_dtype, non_blocking=True
            )

    def num_rows(self, data) -> int:
        """Rows that enter an autocorrelation Gram: tokens or documents."""
        if self.attribute_tokens:
            return int(compute_num_token_grads(data).sum())
        return len(data)

    # ------------------------------------------------------------------ hooks

    def with_batch(self, collection_mask: Tensor | None = None) -> "HookCollectorBase":
        self._current_collection_mask = collection_mask
        return self

    def __enter__(self):
        # Re-entrant: the collection loop holds the hooks for the whole run while each
        # batch enters again through ``with_batch``.
        self._depth = getattr(self, "_depth", 0) + 1
        if self._depth > 1:
            return self
        for name in self.target_info:
            layer = self.model.get_submodule(name)
            layer._name = name  # type: ignore[attr-defined]
            layer._collect_bias = self.target_info[name][2]  # type: ignore[attr-defined]
            self._fwd_hooks.append(layer.register_forward_hook(self._on_forward))
            if self._fused_enabled and self._tap_dim_ok and isinstance(layer, _tap_module_types()):
                # In-tree layers compute the projections inside their own GEMM passes.
                layer._tap = _FusedTap(self, name)  # type: ignore[attr-defined]
        return self

    def _on_forward(self, module: nn.Module, inp: tuple, out):
        if module.__dict__.pop("_tapped", False):
            return  # this call was collected through the module's tap
        x = inp[0].detach()
        assert x.ndim == 3, f"Expected input of shape [N, S, I], got {x.shape}"
        self.forward_hook(module, x)
        if isinstance(out, Tensor) and out.requires_grad:
            # A tensor hook on the output delivers dL/d(out) without wrapping the module
            # in an extra autograd node the way a full backward hook would.
            out.register_hook(functools.partial(self._on_backward, module))

    def _on_backward(self, module: nn.Module, grad_out: Tensor):
        assert isinstance(module, LayerAdapter.supported_modules)
        self.backward_hook(module, grad_out.detach())
        if hasattr(module, "_inputs"):
            del module._inputs
        return None

    def __exit__(self, exc_type, exc, tb):
        self._depth -= 1
        if self._depth > 0:
            return False
        for layer in self.model.modules():
            for attr in ("_inputs", "_name", "_collect_bias", "_fused", "_tap", "_tapped"):
                if hasattr(layer, attr):
                    delattr(layer, attr)
        for h in self._fwd_hooks:
            h.remove()
        self._fwd_hooks.clear()
        return False

    def on_batch_start(self, step: int, num_steps: int) -> None:
        """Called by the collection loop before batch ``step`` of ``num_steps`` (no-op by default)."""

    @abstractmethod
    def setup(self) -> None: ...

    @abstractmethod
    def teardown(self) -> None: ...

    @abstractmethod
    def backward_hook(self, module: nn.Module, g: Tensor) -> None: ...

    @abstractmethod
    def process_batch(self, indices: list[int], **kwargs) -> None: ...

    # ------------------------------------------------------------------ fused path

    def enable_fused(self, col_offsets: dict[str, int], total_dim: int, token_rows: bool = False) -> bool:
        """Switch on the tcgen05 projection paths if the configuration allows it.
        ``col_offsets`` maps (head-expanded) module names to their first column.

        Two paths feed the fp32 row accumulator: *taps* on in-tree layers (projections as
        side outputs of the layers' own GEMMs; projection dims 8 / 16 / 32 / 64, per-sequence
        or, with ``token_rows``, per-token rows) and, for any other ``nn.Linear``, the
        stand-alone projection kernels behind the hooks (dim 16, per-sequence rows).  Modules
        that neither path covers (bias columns, Adam normalisers, split heads) take the torch
        expressions and are merged into the accumulator afterwards."""
        self._fused_enabled = False
        p = self.per_module_projection_dim
        self._tap_dim_ok = p in TAP_PROJECTION_DIMS
        self._hook_fused_ok = p == FUSED_PROJECTION_DIM and not self.attribute_tokens
        if not (self._tap_dim_ok or self._hook_fused_ok):
            return False
        if self.attribute_tokens and not (token_rows and self._tap_dim_ok):
            return False
        dev = next(self.model.parameters()).device
        if dev.type != "cuda":
            return False
        from ..ops import native

        if not native.available():
            return False
        self._col_offsets = dict(col_offsets)
        self._total_dim = total_dim
        self._fused_enabled = True
        return True

    def _fused_eligible(self, module: nn.Module, x: Tensor) -> bool:
        if not self._fused_enabled or not self._hook_fused_ok or module._collect_bias:
            return False
        if x.dtype not in (torch.bfloat16, torch.float16):
            return False
        name = module._name
        if name not in self._col_offsets:
            return False
        if isinstance(self.processor.normalizers.get(name), AdamNormalizer):
            return False
        i = getattr(module, LayerAdapter.in_attr(module))
        o = getattr(module, LayerAdapter.out_attr(module))
        return i % 8 == 0 and o % 8 == 0

    def _fused_matrices(self, name: str, o: int, i: int, device, dtype) -> tuple[Tensor, Tensor]:
        """(P_in [16, I], P_out [16, O]) in the activation dtype with the Adafactor
        column / row scales folded in."""
        key = (name, device, dtype)
        if key not in self._fused_mats:
            p = FUSED_PROJECTION_DIM
            p_in = self.projection(name, p, i, "right", device, dtype).float()
            p_out = self.projection(name, p, o, "left", device, dtype).float()
            norm = self.processor.normalizers.get(name)
            if isinstance(norm, AdafactorNormalizer):
                row, col = self.adafactor_scales(name, norm)
                p_in = p_in * col.to(device).float()[None, :]
                p_out = p_out * row.to(device).float()[None, :]
            self._fused_mats[key] = (p_in.to(dtype).contiguous(), p_out.to(dtype).contiguous())
        return self._fused_mats[key]

    def _tap_matrices(self, name: str, o: int, i: int, device, dtype, bias: bool = False) -> tuple[Tensor, Tensor]:
        """(P_in [p16, I], P_out [p16, O]) for the GEMM side outputs: the projection matrices
        with the Adafactor column / row scales folded in, rows zero-padded to a multiple of 16.
        With ``bias`` the input projection has one more column (the bias acts as an input that
        is always one); that column is kept aside in ``_tap_bias`` and added to the projected
        activations when the tap collects."""
        key = ("tap", name, device, dtype)
        if key not in self._fused_mats:
            p = self.per_module_projection_dim
            assert p is not None
            p16 = (p + 15) // 16 * 16
            p_in = self.projection(name, p, i + 1 if bias else i, "right", device, dtype).float()
            p_out = self.projection(name, p, o, "left", device, dtype).float()
            norm = self.processor.normalizers.get(name)
            if isinstance(norm, AdafactorNormalizer):
                row, col = self.adafactor_scales(name, norm)
                p_in = p_in * col.to(device).float()[None, :]
                p_out = p_out * row.to(device).float()[None, :]
            pad = lambda m: torch.cat([m, m.new_zeros(p16 - p, m.shape[1])]) if p16 > p else m  # noqa: E731
            p_in = pad(p_in).to(dtype)
            if bias:
                self._tap_bias[name] = p_in[:, i].float().contiguous()  # [p16], rounded like the matrix
                p_in = p_in[:, :i]
            self._fused_mats[key] = (p_in.contiguous(), pad(p_out).to(dtype).contiguous())
        return self._fused_mats[key]

    def _tap_accepts(self, module: nn.Module, x: Tensor) -> bool:
        if not self._fused_enabled:
            return False
        if x.dtype not in (torch.bfloat16, torch.float16) or x.ndim != 3 or x.shape[0] != getattr(self, "_fused_n", -1):
            return False
        name = module._name
        if name not in self._col_offsets or name in self.attention_cfgs:
            return False
        norm = self.processor.normalizers.get(name)
        if module._collect_bias and norm is not None:
            # A normaliser scales the bias gradient by its own second moments, i.e. with another
            # left projection than the weight block's: that case stays on the hook path.
            return False
        return not isinstance(norm, AdamNormalizer)

    def begin_fused_batch(self, n: int, device, collection_mask: Tensor | None = None) -> None:
        """Zero the fp32 row accumulator of the coming batch (one row per document, or per
        collected token when rows are per token)."""
        if not self._fused_enabled:
            return
        self._fused_n = n
        rows = n
        if self.attribute_tokens:
            assert collection_mask is not None, "per-token rows need the batch's collection mask"
            self._token_index = collection_mask.reshape(-1).nonzero(as_tuple=True)[0]
            rows = int(self._token_index.numel())
        if self._row_acc is None or self._row_acc.shape[0] < rows or self._row_acc.device != device:
            self._row_acc = torch.zeros(max(rows, 1), self._total_dim, device=device, dtype=torch.float32)
        else:
            self._row_acc[:rows].zero_()
        self._fused_written.clear()
        self._fused_rows = rows

    def fused_rows(self) -> Tensor:
        """fp32 ``[n, total_dim]`` accumulator of the current batch; blocks of modules
        that took the torch path are copied in from ``mod_grads`` first."""
        assert self._row_acc is not None
        acc = self._row_acc[: self._fused_rows]
        for name, P in self.mod_grads.items():
            if name in self._fused_written or name not in self._col_offsets:
                continue
            off = self._col_offsets[name]
            acc[:, off : off + P.shape[1]] = P.to(acc.device, torch.float32)
        return acc

    # ------------------------------------------------------------------ gradient math

    def forward_hook(self, module: nn.Module, a: Tensor) -> None:
        """Cache the (scaled, right-projected) activations in ``module._inputs``."""
        name = assert_type(str, module._name)
        if self._fused_eligible(module, a) and a.shape[0] == getattr(self, "_fused_n", -1):
            from ..ops import native

            i = a.shape[-1]
            o = getattr(module, LayerAdapter.out_attr(module))
            p_in, _ = self._fused_matrices(name, o, i, a.device, a.dtype)
            module._inputs = native.proj_right(a.reshape(-1, i).contiguous(), p_in)
            module._fused = True
            return
        module._fused = False
        p = self.per_module_projection_dim
        i = getattr(module, LayerAdapter.in_attr(module))
        norm = self.normalizer_for(name)
        if isinstance(norm, AdamNormalizer):
            module._inputs = a
            return
        if isinstance(norm, AdafactorNormalizer):
            a = a * self.adafactor_scales(name, norm)[1].type_as(a)
        # With a bias column the un-projected activations are needed in backward.
        if p is not None and not module._collect_bias:
            a = a @ self.projection(name, p, i, "right", a.device, a.dtype).T
        module._inputs = a

    def double_sided_projection(self, name: str, P: Tensor, g: Tensor, p: int, o: int, i: int) -> Tensor:
        L = self.projection(name, p, o, "left", g.device, g.dtype)
        R = self.projection(name, p, i, "right", g.device, g.dtype)
        return L @ P @ R.T

    def double_sided_projection_with_bias(self, name, g, a, bias_grad, p: int, o: int, i: int) -> Tensor:
        """``L [g^T a | b] R^T = (g L^T)^T (a R[:, :i]^T) + (b L^T) (x) R[:, i]`` without
        forming the ``[O, I+1]`` gradient."""
        L = self.projection(name, p, o, "left", g.device, g.dtype)
        R = self.projection(name, p, i + 1, "right", g.device, g.dtype)
        gp = g @ L.T
        ap = a @ R[:, :i].T
        bp = bias_grad @ L.T
        P = gp.unsqueeze(-1) * ap.unsqueeze(-2) if self.attribute_tokens else gp.mT @ ap
        return P + bp.unsqueeze(-1) * R[:, i]

    def _compute_gradient(self, module: nn.Module, g: Tensor) -> Tensor:
        """Flattened, clamped per-example (or per-token) gradient block of ``module``:
        ``[N, d]`` or ``[valid_tokens, d]``."""
        a = module._inputs
        assert isinstance(a, Tensor), "Activation cache missing for module"
        name = assert_type(str, module._name)
        p = self.per_module_projection_dim
        i = getattr(module, LayerAdapter.in_attr(module))
        o = getattr(module, LayerAdapter.out_attr(module))
        norm = self.normalizer_for(name)
        tokens = self.attribute_tokens
        with_bias = bool(module._collect_bias)

        def outer(gg: Tensor, aa: Tensor) -> Tensor:
            return gg.unsqueeze(-1) * aa.unsqueeze(-2) if tokens else gg.mT @ aa

        def bias_of(gg: Tensor) -> Tensor:
            return gg if tokens else gg.sum(dim=1)

        if isinstance(norm, AdamNormalizer):
            # Elementwise normalisation does not commute with projection: materialise.
            P = norm.normalize_weight(outer(g, a))
            if with_bias:
                P = torch.cat([P, bias_of(norm.normalize_bias(g)).unsqueeze(-1)], dim=-1)
                i += 1
            if p is not None:
                P = self.double_sided_projection(name, P, g, p, o, i)
        else:
            bias_grad = None
            if with_bias:
                bias_grad = bias_of(norm.normalize_bias(g) if norm is not None else g)
            if isinstance(norm, AdafactorNormalizer):
                g = g * self.adafactor_scales(name, norm)[0].type_as(g)
            if with_bias and p is not None:
                P = self.double_sided_projection_with_bias(name, g, a, bias_grad, p, o, i)
            else:
                if p is not None:
                    g = g @ self.projection(name, p, o, "left", g.device, g.dtype).T
                P = outer(g, a)
                if with_bias:
                    P = torch.cat([P, bias_grad.unsqueeze(-1)], dim=-1)
        if tokens:
            P = P.flatten(2)[self._current_collection_mask]
        return P.flatten(1).clamp_(self.lo, self.hi)

    def compute_gradient_fused(self, module: nn.Module, g: Tensor) -> bool:
        """Fused counterpart of ``_compute_gradient``: accumulates the block into the
        batch's row accumulator.  Returns False when the module is on the torch path."""
        if not getattr(module, "_fused", False):
            return False
        from ..ops import native

        name = module._name
        o = g.shape[-1]
        i = getattr(module, LayerAdapter.in_attr(module))
        _, p_out = self._fused_matrices(name, o, i, g.device, g.dtype)
        native.proj_left_outer(
            g.contiguous(), p_out, module._inputs, self._row_acc[: self._fused_rows], self._col_offsets[name]
        )
        self._fused_written.add(name)
        return True


def check_kernel_status(device) -> None:
    """Raise if a kernel on ``device`` gave up on one of its bounded waits (its output is
    then incomplete).  Called once at the end of a run, before results are finalised: it
    synchronises the device."""
    device = torch.device(device)
    if device.type != "cuda":
        return
    from ..ops import attribution, native

    if not native.available():
        return
    status = attribution.kernel_status(device.index if device.index is not None else torch.cuda.current_device())
    if status != 0:
        raise RuntimeError(
            f"a bergson_b200 kernel on {device} gave up on a bounded wait (status {status}); the rows or factors "
            "accumulated in this run are incomplete and were not finalised")


class CollectorComputer:
    """Runs forward/backward over the batches with a collector attached.

    The loop never synchronises the device: inputs are staged through pinned memory,
    per-document losses and the processed-position counter stay on the device, and the
    collector hands finished rows to asynchronous writers.
    """

    def __init__(self, model, data, *, collector: HookCollectorBase, batches=None, cfg: IndexConfig):
        self.model = model
        self.device = torch.device(model.device)
        self.data = data
        self.batches = batches if batches is not None else [[i] for i in range(len(data))]
        self.forward_backward = fwd_bwd_factory(cfg)
        self.collector = collector
        self.cfg = cfg
        self.logger = get_logger("CollectorComputer", level="DEBUG" if cfg.debug else "INFO")
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.world_size = dist.get_world_size() if dist.is_initialized() else 1
        self.logger.info("Tracking %d modules", len(collector.target_info))

    def _setup_profiler(self):
        if not self.cfg.profile:
            return nullcontext()
        from torch.profiler import ProfilerActivity, profile, schedule, tensorboard_trace_handler

        os.makedirs("profiler_logs", exist_ok=True)
        acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
        return profile(
            activities=acts,
            on_trace_ready=tensorboard_trace_handler("profiler_logs", worker_name=f"rank_{self.rank}", use_gzip=True),
            schedule=schedule(wait=0, warmup=0, active=4, repeat=1),
            record_shapes=True,
            with_stack=True,
            profile_memory=True,
            with_modules=True,
        )

    def stage(self, indices: list[int]):
        """Host side of a batch: fetch rows, pad, copy to the device through pinned memory
        (asynchronously).  Returns ``(x, y, collection_mask, batch)``."""
        batch = self.data[indices]
        x, y, _, mask = pad_and_tensor(
            batch["input_ids"], labels=batch.get("labels"), device=self.device,
            sync_max_len=False, pinned=self.device.type == "cuda",
        )
        return x, y, mask, batch

    def run_staged(self, indices: list[int], x: Tensor, y: Tensor, mask: Tensor, batch: dict) -> Tensor:
        """Device side of a batch: forward/backward under the hooks, hand off rows."""
        if not hasattr(self, "_total_processed"):
            self._total_processed = torch.zeros((), dtype=torch.long, device=self.device)
        self._total_processed += mask.sum()
        self.collector.begin_fused_batch(len(indices), self.device, mask)
        with self.collector.with_batch(mask):
            losses = self.forward_backward(self.model, x, y, batch)
        self.collector.process_batch(indices, losses=losses)
        return losses

    def step(self, indices: list[int]) -> Tensor:
        """One batch end to end; returns the per-document losses (on the device)."""
        return self.run_staged(indices, *self.stage(indices))

    def run_with_collector_hooks(self, desc: Optional[str] = None):
        self._total_processed = torch.zeros((), dtype=torch.long, device=self.device)
        prof = self._setup_profiler()
        with prof, self.collector:
            for step, indices in enumerate(tqdm(self.batches, desc=f"Computing {desc}", disable=self.rank != 0)):
                self.collector.on_batch_start(step, len(self.batches))
                if self.cfg.profile:
                    from torch.profiler import record_function

                    with record_function(f"step_{step}"):
                        self.step(indices)
                    prof.step()  # type: ignore[union-attr]
                else:
                    self.step(indices)
        check_kernel_status(self.device)
        self.collector.teardown()
        total = self._total_processed
        if dist.is_initialized():
            from ..parallel import topology

            dist.all_reduce(total, op=dist.ReduceOp.SUM)
            total = total // topology.tp_size()  # tensor-parallel peers counted the same positions
        if self.rank == 0:
            torch.save(total.cpu(), os.path.join(self.cfg.partial_run_path, "total_processed.pt"))
        self.logger.info(f"Total processed: {total.item()}")


def _direct_hidden_ok(model) -> bool:
    """In-tree models can skip the last position's logits by calling ``hidden`` and the head
    themselves, unless the model is wrapped by FSDP2: its parameters are only gathered by the
    hooks of ``__call__``."""
    if not isinstance(model, NativeCausalLM):
        return False
    try:
        from torch.distributed.fsdp import FSDPModule
    except ImportError:  # older torch: no fully_shard, nothing to bypass
        return True
    return not isinstance(model, FSDPModule)


def _per_token_losses(model, x: Tensor, targets: Tensor, label_smoothing: float = 0.0) -> tuple[Tensor, Tensor]:
    """(per-token CE ``[N, S-1]`` in fp32, logits or None).  In-tree models skip the
    last position's logits and use the fused CE kernel; other models go through
    ``model(x).logits``."""
    if _direct_hidden_ok(model):
        h = model.hidden(x)[:, :-1]
        logits = model.get_output_embeddings()(h)
    else:
        logits = model(x).logits[:, :-1]
    V = logits.size(-1)
    tok = ops.token_cross_entropy(logits.reshape(-1, V), targets.reshape(-1), label_smoothing=label_smoothing)
    return tok.view(targets.shape), logits


def fwd_bwd_factory(cfg: IndexConfig) -> Callable:
    """``fwd_bwd(model, x, y, batch) -> per-document losses``; runs the backward pass of
    the summed document losses (reference ``collector.py:926-985``)."""

    def fwd_bwd(model, x: Tensor, y: Tensor, batch: dict):
        targets = y[:, 1:]
        masks = targets != -100
        denoms = masks.sum(dim=1).clamp_min(1).float() if cfg.loss_reduction == "mean" else 1.0
        if cfg.loss_fn == "kl":
            from ..utils.peft import set_peft_enabled

            logits = model(x).logits[:, :-1]
            with torch.inference_mode():
                set_peft_enabled(model, False)
                ref_lps = torch.log_softmax(model(x).logits[:, :-1], dim=-1)
                set_peft_enabled(model, True)
            ft_lps = torch.log_softmax(logits, dim=-1)
            kls = torch.sum(ft_lps.exp() * (ft_lps - ref_lps), dim=-1)
            losses = torch.sum(kls * masks, dim=-1) / denoms
        else:
            tok, _ = _per_token_losses(model, x, targets, cfg.label_smoothing)
            losses = tok.sum(1) / denoms
        if "advantage" in batch:
            losses = losses * torch.tensor(batch["advantage"], device=losses.device, dtype=losses.dtype)
        losses.sum().backward()
        model.zero_grad(set_to_none=True)
        return losses.detach()

    return fwd_bwd


def fwd_bwd_hessian_factory(index_cfg: IndexConfig, hessian_cfg: HessianConfig) -> Callable:
    """Like ``fwd_bwd_factory`` but with labels sampled from the model's own predictive
    distribution (true Fisher) unless ``use_dataset_labels``."""

    def fwd_bwd_hessian(model, x: Tensor, y: Tensor, batch: dict):
        targets = y[:, 1:]
        masks = targets != -100
        denoms = masks.sum(dim=1).clamp_min(1).float() if index_cfg.loss_reduction == "mean" else 1.0
        if _direct_hidden_ok(model):
            logits = model.get_output_embeddings()(model.hidden(x)[:, :-1])
        else:
            logits = model(x).logits[:, :-1]
        V = logits.size(-1)
        if not hessian_cfg.use_dataset_labels:
            with torch.no_grad():
                probs = F.softmax(logits.float(), dim=-1)
                targets = torch.multinomial(probs.reshape(-1, V), 1, replacement=True).view(targets.shape)
        tok = ops.token_cross_entropy(logits.reshape(-1, V), targets.reshape(-1)).view(targets.shape)
        losses = tok.sum(1) / denoms
        losses.sum().backward()
        model.zero_grad(set_to_none=True)
        return losses.detach()

    return fwd_bwd_hessian
