"""Linear layers on the persistent tcgen05 GEMM.

``linear(x, weight, bias)`` computes ``x @ weight^T + bias`` (``layout="oi"``, an
``nn.Linear`` weight ``[out, in]``) or ``x @ weight + bias`` (``layout="io"``, a GPT-2
``Conv1D`` weight ``[in, out]``).  On CUDA with 16-bit tensors the forward product, the
input-gradient product ``g @ W`` and the weight-gradient product ``g^T x`` all run on
``native.gemm``, which reads the weight in place in whichever orientation the product
needs (no transposed copies).  Inside ``ops.composable()`` (graphs that will be
differentiated again, as in MAGIC's traced step) the products run on the same kernel through
``_GemmFn``, whose backward is written with ``_GemmFn`` itself: the derivative of a matrix
product is two matrix products, so the family is closed under differentiation and every
order of derivative stays on the tensor cores.  A weight whose output size is not a multiple
of 8 (GPT-2's 50257-row vocabulary) is zero-padded to the next multiple for the product and
the result sliced back.  Everywhere else the call is ``F.linear`` / ``addmm``.

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

from .functional import _composable, use_fused

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


def _kernel_ready(x: Tensor, weight: Tensor) -> bool:
    """CUDA 16-bit operands and a loaded extension (whether or not composable mode is on)."""
    if not (x.is_cuda and weight.is_cuda and x.dtype in _TC_DTYPES and weight.dtype == x.dtype and x.numel() > 0):
        return False
    from . import native

    return native.available()


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


def _operand_ok(t: Tensor) -> bool:
    """What a tensor map over a 2-D operand needs: unit inner stride, rows and base on 16 bytes."""
    return t.dim() == 2 and t.stride(1) == 1 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0 and t.shape[1] % 8 == 0


def _as_operand(t: Tensor) -> Tensor:
    return t if _operand_ok(t) else t.contiguous()


class _GemmFn(torch.autograd.Function):
    """``d = A B`` in the kernel's storage convention: ``a`` holds A as ``[M, K]`` (``a_mn``
    False) or ``[K, M]`` (True); ``b`` holds B as ``[N, K]`` (``b_mn`` False) or ``[K, N]``
    (True); ``bias`` ``[N]`` is optional.  The backward calls ``_GemmFn`` again, so a graph
    built with ``create_graph=True`` can itself be differentiated."""

    @staticmethod
    def forward(ctx, a: Tensor, b: Tensor, a_mn: bool, b_mn: bool, bias: Tensor | None):
        from . import native

        # The inputs themselves are saved: only a saved input keeps its place in the graph, which
        # the backward of the backward needs; copies for alignment are made again (tracked) there.
        ctx.save_for_backward(a, b)
        ctx.layout = (a_mn, b_mn)
        ctx.has_bias = bias is not None
        d, _ = native.gemm(_as_operand(a), _as_operand(b), a_mn, b_mn, None, False, bias, False, None, **_gemm_form())
        return d

    @staticmethod
    def backward(ctx, g: Tensor):
        a, b = ctx.saved_tensors
        a_mn, b_mn = ctx.layout
        da = db = dbias = None
        if ctx.needs_input_grad[0]:
            # [M, K] = g B, or in A's transposed storage [K, M] = B^T g^T.
            da = _GemmFn.apply(b, g, not b_mn, False, None) if a_mn else _GemmFn.apply(g, b, False, not b_mn, None)
        if ctx.needs_input_grad[1]:
            # [N, K] = g^T A, or in B's transposed storage [K, N] = A^T g.
            db = _GemmFn.apply(a, g, not a_mn, True, None) if b_mn else _GemmFn.apply(g, a, True, not a_mn, None)
        if ctx.has_bias and ctx.needs_input_grad[4]:
            dbias = g.sum(0)
        return da, db, None, None, dbias


PAD_LOGIT = -30000.0  # what padded output columns hold when the caller keeps them (exp underflows to 0)


def _composable_linear(x: Tensor, weight: Tensor, bias: Tensor | None, layout: str, keep_pad: bool = False) -> Tensor | None:
    """The any-order-differentiable product on the kernel, or None when the shapes do not fit.
    With ``keep_pad`` the padded columns stay in the result, filled with ``PAD_LOGIT`` through
    the GEMM's bias epilogue (for a softmax / cross-entropy that runs on the padded width)."""
    oi = layout == "oi"
    in_f = weight.shape[1] if oi else weight.shape[0]
    out_f = weight.shape[0] if oi else weight.shape[1]
    if weight.dim() != 2 or in_f % 8 or x.shape[-1] != in_f:
        return None
    pad = -out_f % 8
    if pad and not oi:
        return None
    if bias is not None and bias.dtype not in (x.dtype, torch.float32):
        return None
    w = F.pad(weight, (0, 0, 0, pad)) if pad else weight
    bb = F.pad(bias, (0, pad)) if (pad and bias is not None) else bias
    if pad and keep_pad:
        fill = x.new_zeros(out_f + pad)
        fill[out_f:] = PAD_LOGIT
        bb = fill if bb is None else bb + fill
    y = _GemmFn.apply(x.reshape(-1, in_f), w, False, not oi, bb)
    y = y.view(*x.shape[:-1], out_f + pad)
    return y[..., :out_f] if (pad and not keep_pad) else y


def linear_keep_padding(x: Tensor, weight: Tensor) -> Tensor | None:
    """``x @ weight^T`` on the kernel with the output width rounded up to a multiple of 8 and the
    extra columns set to ``PAD_LOGIT`` (contiguous result), or None when the kernel path does
    not apply.  For heads whose vocabulary size is not a multiple of 8."""
    if not _kernel_ready(x, weight) or weight.dim() != 2:
        return None
    return _composable_linear(x, weight, None, "oi", keep_pad=True)


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
    if _kernel_ready(x, weight) and (_composable() or weight.dim() == 2 and weight.shape[0] % 8 and layout == "oi"):
        # Graphs that will be differentiated again, and weights that need padding.
        y = _composable_linear(x, weight, bias, layout)
        if y is not None:
            return y
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
