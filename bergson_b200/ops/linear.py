"""Linear layers on the persistent tcgen05 GEMM.

``linear(x, weight, bias)`` computes ``x @ weight^T + bias`` (``layout="oi"``, an
``nn.Linear`` weight ``[out, in]``) or ``x @ weight + bias`` (``layout="io"``, a GPT-2
``Conv1D`` weight ``[in, out]``).  On CUDA with 16-bit tensors the forward product, the
input-gradient product ``g @ W`` and the weight-gradient product ``g^T x`` all run on
``native.gemm``, which reads the weight in place in whichever orientation the product
needs (no transposed copies).  Everywhere else, and inside ``ops.composable()``, the
call is ``F.linear`` / ``addmm`` and stays differentiable to any order.

A *tap* lets a gradient collector ride on the same passes over the data: when the
module carries a tap that accepts the call, the forward GEMM also emits
``x @ P_in^T`` and the input-gradient GEMM ``g @ P_out^T`` as small fp32 side outputs
(one extra 16..64-column tile per 128 rows), and the tap receives both in backward.  That
replaces the separate projection kernels, which had to stream the activations and the
output gradients from memory a second time.
"""

from __future__ import annotations

import os
from typing import Protocol

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from .functional import use_fused

_TC_DTYPES = (torch.bfloat16, torch.float16)


def _gemm_form() -> dict:
    """Keyword arguments selecting the GEMM form: the wide CTA-pair kernel by default;
    ``BERGSON_B200_GEMM_FORM=pair`` / ``single`` select the 256 x 256 pair tile or the
    single-CTA kernel (debugging, comparisons)."""
    form = os.environ.get("BERGSON_B200_GEMM_FORM", "wide")
    if form == "single":
        return dict(cta_group=1)
    if form == "pair":
        return dict(cta_group=2)
    return dict(cta_group=2, wide=True)


class ProjectionTap(Protocol):
    """What a collector attaches to a module (attribute ``_tap``)."""

    def operands(self, module: nn.Module, x: Tensor) -> tuple[Tensor, Tensor] | None:
        """``(P_in [p16, in], P_out [p16, out])`` in ``x``'s dtype (rows padded with zeros to a
        multiple of 16), or None when this call is not collected."""

    def collect(self, module: nn.Module, a_proj: Tensor, g_proj: Tensor, lead_shape: torch.Size) -> None:
        """Called in backward with ``a_proj = x P_in^T`` and ``g_proj = g P_out^T`` (fp32
        ``[tokens, p16]``); ``lead_shape`` is the shape of ``x`` without its last dimension."""


def gemm_eligible(x: Tensor, weight: Tensor) -> bool:
    return (
        x.dtype in _TC_DTYPES
        and weight.dtype == x.dtype
        and weight.dim() == 2
        and weight.is_contiguous()
        and weight.shape[0] % 8 == 0
        and weight.shape[1] % 8 == 0
        and x.numel() > 0
        and use_fused(x, weight)
    )


def _aux_fits(rows: int, cols: int, device) -> bool:
    """Whether the projection side output rides along for free.  It is one more (cheap) tile
    per 512-row block; the persistent kernel deals tiles round-robin over the CTA pairs, so
    the extra tiles are free unless they push the tile count over a multiple of the number
    of pairs, in which case a separate pass over the operand is cheaper."""
    pairs = max(1, torch.cuda.get_device_properties(device).multi_processor_count // 2)
    tiles_m, tiles_n = -(-rows // 512), -(-cols // 256)
    return -(-(tiles_m * (tiles_n + 1)) // pairs) == -(-(tiles_m * tiles_n) // pairs)


def _project(x2: Tensor, p: Tensor) -> Tensor:
    """``x2 @ p^T`` in fp32 as its own pass (16-row operands on the skinny tcgen05 kernel)."""
    from . import native

    if p.shape[0] == 16 and x2.shape[1] % 8 == 0:
        return native.proj_right(x2, p)
    return x2.float() @ p.float().T


def _gemm_with_projection(x2: Tensor, w: Tensor, b_mn: bool, bias, p: Tensor | None, out_cols: int, form: dict):
    from . import native

    if p is None or _aux_fits(x2.shape[0], out_cols, x2.device):
        return native.gemm(x2, w, False, b_mn, None, False, bias, False, p, **form)
    y, _ = native.gemm(x2, w, False, b_mn, None, False, bias, False, None, **form)
    return y, _project(x2, p)


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, weight: Tensor, bias: Tensor | None, layout: str, module, tap):
        from . import native

        oi = layout == "oi"
        in_f = weight.shape[1] if oi else weight.shape[0]
        out_f = weight.shape[0] if oi else weight.shape[1]
        lead = x.shape[:-1]
        x2 = x.reshape(-1, in_f)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        taps = tap.operands(module, x) if tap is not None else None
        form = _gemm_form()
        y, a_proj = _gemm_with_projection(x2, weight, not oi, bias, taps[0] if taps is not None else None, out_f, form)
        ctx.save_for_backward(x2 if weight.requires_grad else None, weight, taps[1] if taps is not None else None,
                              a_proj if taps is not None else None)
        ctx.layout, ctx.lead, ctx.form = layout, lead, form
        ctx.module, ctx.tap = (module, tap) if taps is not None else (None, None)
        ctx.has_bias = bias is not None
        return y.view(*lead, out_f)

    @staticmethod
    def backward(ctx, g: Tensor):
        from . import native

        x2, weight, p_out, a_proj = ctx.saved_tensors
        oi = ctx.layout == "oi"
        out_f = weight.shape[0] if oi else weight.shape[1]
        g2 = g.reshape(-1, out_f)
        if not g2.is_contiguous():
            g2 = g2.contiguous()
        dx = dw = db = None
        g_proj = None
        if ctx.needs_input_grad[0]:
            # dx = g W (oi: W read as [K = out, N = in]) or g W^T (io: W read as [N = in, K = out]).
            in_f = weight.shape[1] if oi else weight.shape[0]
            dx2, g_proj = _gemm_with_projection(g2, weight, oi, None, p_out, in_f, ctx.form)
            dx = dx2.view(*ctx.lead, dx2.shape[1])
        if ctx.tap is not None:
            if g_proj is None or g_proj.numel() == 0:
                g_proj = g2.float() @ p_out.float().T
            ctx.tap.collect(ctx.module, a_proj, g_proj, ctx.lead)
        if ctx.needs_input_grad[1]:
            # dW = g^T x ([out, in]) or x^T g ([in, out]): both operands read along the tokens.
            lhs, rhs = (g2, x2) if oi else (x2, g2)
            dw, _ = native.gemm(lhs, rhs, True, True, None, False, None, False, None, **ctx.form)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = g2.sum(0)
        return dx, dw, db, None, None, None


def linear(x: Tensor, weight: Tensor, bias: Tensor | None = None, *, layout: str = "oi", module=None,
           tap: ProjectionTap | None = None) -> Tensor:
    """``x @ weight^T + bias`` (``layout="oi"``) or ``x @ weight + bias`` (``layout="io"``)."""
    if gemm_eligible(x, weight) and (bias is None or bias.dtype in (x.dtype, torch.float32)):
        # A tap only makes sense when a backward pass will follow (grad mode is off inside
        # ``Function.forward``, so the decision is taken here).
        if tap is not None and not (torch.is_grad_enabled() and x.requires_grad):
            tap = None
        return _LinearFn.apply(x, weight, bias, layout, module, tap)
    if layout == "oi":
        return F.linear(x, weight, bias)
    y = x.reshape(-1, x.shape[-1]) @ weight
    if bias is not None:
        y = y + bias
    return y.view(*x.shape[:-1], weight.shape[1])


class Linear(nn.Linear):
    """``nn.Linear`` whose products run on the tcgen05 GEMM (see module docstring).  It *is*
    an ``nn.Linear`` for every ``isinstance`` check, state dict and optimizer."""

    def forward(self, x: Tensor) -> Tensor:
        return linear(x, self.weight, self.bias, layout="oi", module=self, tap=getattr(self, "_tap", None))
