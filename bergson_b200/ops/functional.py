"""Model-side ops with two execution paths.

* **fused** (default on CUDA): each op is one hand-written sm_100a kernel for the
  forward and one for the backward, wrapped in an ``autograd.Function``.  The
  backward kernels are not themselves differentiable.
* **composable**: the op is written with differentiable torch primitives so that
  ``create_graph=True`` works to any order.  This is the CPU path and the path the
  twice-differentiable trainer selects with ``ops.composable()``.

The numerics of both paths are the same formulas; GPU tests compare each kernel
against the composable expression evaluated in fp32.
"""

from __future__ import annotations

import contextlib
import math
import threading

import torch
import torch.nn.functional as F
from torch import Tensor

_state = threading.local()


def _composable() -> bool:
    return getattr(_state, "composable", False)


@contextlib.contextmanager
def composable(enabled: bool = True):
    """Force the any-order-differentiable torch path inside the block."""
    prev = _composable()
    _state.composable = enabled
    try:
        yield
    finally:
        _state.composable = prev


def use_fused(*tensors: Tensor) -> bool:
    """True when the fused CUDA kernels should run for these operands."""
    if _composable():
        return False
    if not all(t.is_cuda for t in tensors if t is not None):
        return False
    from . import native

    return native.available()


def _kernels_ready(*tensors: Tensor) -> bool:
    """CUDA tensors and a loaded extension, whether or not composable mode is on (for the ops
    whose kernels cover the backward of the backward as well)."""
    if not all(t is None or t.is_cuda for t in tensors):
        return False
    from . import native

    return native.available()


# --------------------------------------------------------------------------- #
# normalisation
# --------------------------------------------------------------------------- #


def rms_norm_ref(x: Tensor, weight: Tensor, eps: float) -> Tensor:
    xf = x if x.dtype == torch.float64 else x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y.to(x.dtype)) * weight


class _RMSNormBwdFn(torch.autograd.Function):
    """``(dy, x, w) -> (dx, dw)`` of RMSNorm with its own backward kernel (the backward of the
    backward); ``rstd`` is the forward's row statistic of ``x``."""

    @staticmethod
    def forward(ctx, dy2, x2, weight, rstd):
        from . import native

        dy2 = dy2.contiguous()
        dx, dw = native.rmsnorm_bwd(dy2, x2, weight, rstd, True)
        ctx.save_for_backward(dy2, x2, weight, rstd)
        return dx, dw

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, cu, cw):
        from . import native

        dy2, x2, weight, rstd = ctx.saved_tensors
        cu = torch.zeros_like(x2) if cu is None else cu.contiguous()
        cw = torch.zeros_like(weight) if cw is None else cw
        d_dy, d_x, d_w = native.rmsnorm_bwd_bwd(cu, cw, dy2, x2, weight, rstd)
        return d_dy, d_x, d_w, None


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        from . import native

        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        y, rstd = native.rmsnorm_fwd(x2, weight, eps)
        ctx.save_for_backward(x, weight, rstd)  # the input itself: it keeps its place in the graph
        ctx.shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x, weight, rstd = ctx.saved_tensors
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not ctx.needs_input_grad[1] and not torch.is_grad_enabled():
            from . import native

            dx, _ = native.rmsnorm_bwd(dy2.contiguous(), x2, weight, rstd, False)
            return dx.view(ctx.shape), None, None
        dx, dw = _RMSNormBwdFn.apply(dy2, x2, weight, rstd)
        return dx.view(ctx.shape), dw, None


def rms_norm(x: Tensor, weight: Tensor, eps: float) -> Tensor:
    """RMSNorm on the kernels: forward, backward and the backward of the backward."""
    d, packet = x.shape[-1], 16 // max(x.element_size(), 1)
    if (x.is_cuda and x.dtype in (torch.bfloat16, torch.float16, torch.float32) and _kernels_ready(x, weight)
            and d % packet == 0 and d <= 2048 * packet):
        return _RMSNormFn.apply(x, weight, eps)
    return rms_norm_ref(x, weight, eps)


def layer_norm_ref(x: Tensor, weight: Tensor, bias: Tensor | None, eps: float) -> Tensor:
    return F.layer_norm(x, (x.shape[-1],), weight, bias, eps)


class _LayerNormBwdFn(torch.autograd.Function):
    """``(dy, x, w) -> (dx, dw, db)`` of LayerNorm as a function with its own backward kernel
    (the backward of the backward), so that a graph built with ``create_graph=True`` can be
    differentiated once more.  ``mean`` and ``rstd`` are the forward's row statistics of ``x``;
    their dependence on ``x`` is part of the kernel's formulas."""

    @staticmethod
    def forward(ctx, dy2, x2, weight, mean, rstd):
        from . import native

        dy2 = dy2.contiguous()
        dx, dw, db = native.layernorm_bwd(dy2, x2, weight, mean, rstd, True)
        ctx.save_for_backward(dy2, x2, weight, mean, rstd)
        return dx, dw, db

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, cu, cw, cb):
        from . import native

        dy2, x2, weight, mean, rstd = ctx.saved_tensors
        cu = torch.zeros_like(x2) if cu is None else cu.contiguous()
        cw = torch.zeros_like(weight) if cw is None else cw
        cb = torch.zeros_like(weight) if cb is None else cb
        d_dy, d_x, d_w = native.layernorm_bwd_bwd(cu, cw, cb, dy2, x2, weight, mean, rstd)
        return d_dy, d_x, d_w, None, None


class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        from . import native

        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        y, mean, rstd = native.layernorm_fwd(x2, weight, bias, eps)
        # The input itself is saved (not the reshaped copy): only a saved *input* keeps its place
        # in the graph, which the backward of the backward needs to reach x.
        ctx.save_for_backward(x, weight, mean, rstd)
        ctx.shape = x.shape
        ctx.has_bias = bias is not None
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x, weight, mean, rstd = ctx.saved_tensors
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        dy2 = dy.reshape(-1, dy.shape[-1])
        need_w = ctx.needs_input_grad[1] or (ctx.has_bias and ctx.needs_input_grad[2])
        if not need_w and not torch.is_grad_enabled():
            # Frozen affine parameters and no graph to build: skip the weight-gradient partials.
            from . import native

            dx, _, _ = native.layernorm_bwd(dy2.contiguous(), x2, weight, mean, rstd, False)
            return dx.view(ctx.shape), None, None, None
        dx, dw, db = _LayerNormBwdFn.apply(dy2, x2, weight, mean, rstd)
        return dx.view(ctx.shape), dw, (db if ctx.has_bias else None), None


def layer_norm(x: Tensor, weight: Tensor, bias: Tensor | None, eps: float) -> Tensor:
    """LayerNorm on the kernels: forward, backward and the backward of the backward."""
    d, packet = x.shape[-1], 16 // max(x.element_size(), 1)
    if (x.is_cuda and x.dtype in (torch.bfloat16, torch.float16, torch.float32) and _kernels_ready(x, weight)
            and d % packet == 0 and d <= 2048 * packet):
        return _LayerNormFn.apply(x, weight, bias, eps)
    return layer_norm_ref(x, weight, bias, eps)


# --------------------------------------------------------------------------- #
# rotary embedding (rotate-half convention, optional partial rotation)
# --------------------------------------------------------------------------- #


def rotary_tables(seq_len: int, rot_dim: int, theta: float, device, dtype=torch.float32):
    inv = 1.0 / (theta ** (torch.arange(0, rot_dim, 2, device=device, dtype=torch.float64) / rot_dim))
    ang = torch.outer(torch.arange(seq_len, device=device, dtype=torch.float64), inv)
    return ang.cos().to(dtype), ang.sin().to(dtype)  # [S, rot_dim/2]


def rotary_ref(x: Tensor, cos: Tensor, sin: Tensor, rot_dim: int) -> Tensor:
    """x: [B, S, H, D]; rotate the first ``rot_dim`` features of each head."""
    half = rot_dim // 2
    c = cos[None, : x.shape[1], None, :].to(x.dtype)
    s = sin[None, : x.shape[1], None, :].to(x.dtype)
    x1, x2, rest = x[..., :half], x[..., half:rot_dim], x[..., rot_dim:]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, rest], dim=-1)


class _RotaryFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, rot_dim):
        from . import native

        ctx.save_for_backward(cos, sin)
        ctx.rot_dim = rot_dim
        return native.rotary(x.contiguous(), cos, sin, rot_dim, False)

    @staticmethod
    def backward(ctx, dy):
        from . import native

        cos, sin = ctx.saved_tensors
        return native.rotary(dy.contiguous(), cos, sin, ctx.rot_dim, True), None, None, None


def rotary(x: Tensor, cos: Tensor, sin: Tensor, rot_dim: int) -> Tensor:
    if use_fused(x) and x.dtype in (torch.bfloat16, torch.float16, torch.float32):
        return _RotaryFn.apply(x, cos, sin, rot_dim)
    return rotary_ref(x, cos, sin, rot_dim)


# --------------------------------------------------------------------------- #
# MLP activations
# --------------------------------------------------------------------------- #


def swiglu_ref(gate: Tensor, up: Tensor) -> Tensor:
    return F.silu(gate) * up


class _SwiGLUBwdFn(torch.autograd.Function):
    """``(dy, gate, up) -> (dgate, dup)`` with its own backward kernel."""

    @staticmethod
    def forward(ctx, dy, gate, up):
        from . import native

        dy, gate, up = dy.contiguous(), gate.contiguous(), up.contiguous()
        ctx.save_for_backward(dy, gate, up)
        dg, du = native.swiglu_bwd(dy, gate, up)
        return dg, du

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, cg, cu):
        from . import native

        dy, gate, up = ctx.saved_tensors
        cg = torch.zeros_like(gate) if cg is None else cg.contiguous()
        cu = torch.zeros_like(gate) if cu is None else cu.contiguous()
        d_dy, d_g, d_u = native.swiglu_bwd_bwd(cg, cu, dy, gate, up)
        return d_dy, d_g, d_u


class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate, up):
        from . import native

        ctx.save_for_backward(gate, up)  # the inputs themselves: they keep their place in the graph
        return native.swiglu_fwd(gate.contiguous(), up.contiguous())

    @staticmethod
    def backward(ctx, dy):
        gate, up = ctx.saved_tensors
        return _SwiGLUBwdFn.apply(dy, gate, up)


def swiglu(gate: Tensor, up: Tensor) -> Tensor:
    """``silu(gate) * up`` on the kernels: forward, backward and the backward of the backward."""
    if (gate.dtype in (torch.bfloat16, torch.float16, torch.float32) and up.dtype == gate.dtype
            and _kernels_ready(gate, up) and gate.numel() % (16 // gate.element_size()) == 0
            and gate.shape == up.shape):
        return _SwiGLUFn.apply(gate, up)
    return swiglu_ref(gate, up)


def gelu_ref(x: Tensor, approximate: str = "none") -> Tensor:
    return F.gelu(x, approximate=approximate)


class _GELUBwdFn(torch.autograd.Function):
    """``dx = dy * gelu'(x)`` as a function of ``(dy, x)`` with its own backward kernel, so that
    a graph built with ``create_graph=True`` can be differentiated once more."""

    @staticmethod
    def forward(ctx, dy, x, tanh_approx):
        from . import native

        dy, x = dy.contiguous(), x.contiguous()
        ctx.save_for_backward(dy, x)
        ctx.tanh_approx = tanh_approx
        return native.gelu_bwd(dy, x, tanh_approx)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, c):
        from . import native

        dy, x = ctx.saved_tensors
        d_dy, d_x = native.gelu_bwd_bwd(c.contiguous(), dy, x, ctx.tanh_approx)
        return d_dy, d_x, None


class _GELUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tanh_approx):
        from . import native

        ctx.save_for_backward(x)  # the input itself, so that it keeps its place in the graph
        ctx.tanh_approx = tanh_approx
        return native.gelu_fwd(x.contiguous(), tanh_approx)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        return _GELUBwdFn.apply(dy, x, ctx.tanh_approx), None


def gelu(x: Tensor, approximate: str = "none") -> Tensor:
    """GELU on the kernels: forward, backward and the backward of the backward (what a traced
    training step needs); a third derivative is refused by autograd."""
    if (_kernels_ready(x) and x.dtype in (torch.bfloat16, torch.float16, torch.float32)
            and x.numel() % (16 // x.element_size()) == 0):
        return _GELUFn.apply(x, approximate == "tanh")
    return gelu_ref(x, approximate)


# --------------------------------------------------------------------------- #
# attention
# --------------------------------------------------------------------------- #


class _SoftmaxBwdFn(torch.autograd.Function):
    """``dx = y * (dy - sum(dy y))`` as a function of ``(dy, y)`` whose own backward is one kernel."""

    @staticmethod
    def forward(ctx, dy, y):
        dy, y = dy.contiguous(), y.contiguous()
        ctx.save_for_backward(dy, y)
        return torch._softmax_backward_data(dy, y, -1, y.dtype)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, c):
        from . import native

        dy, y = ctx.saved_tensors
        d_dy, d_y = native.softmax_bwd_bwd(c.contiguous(), dy, y)
        return d_dy, d_y


class _SoftmaxFn(torch.autograd.Function):
    """Row softmax over the last dimension, differentiable twice (the second time on a kernel)."""

    @staticmethod
    def forward(ctx, x):
        y = torch.softmax(x, dim=-1)
        ctx.save_for_backward(y)
        return y

    @staticmethod
    def backward(ctx, dy):
        (y,) = ctx.saved_tensors
        return _SoftmaxBwdFn.apply(dy, y)


def _softmax_last(x: Tensor) -> Tensor:
    if (x.dtype in (torch.bfloat16, torch.float16, torch.float32) and _kernels_ready(x)
            and x.shape[-1] % (16 // x.element_size()) == 0):
        return _SoftmaxFn.apply(x)
    return torch.softmax(x, dim=-1)


_CAUSAL_BIAS: dict = {}


def _causal_bias(S: int, dtype: torch.dtype, device) -> Tensor:
    """``[S, S]`` additive mask: 0 on and below the diagonal, -inf above (cached per shape)."""
    key = (S, dtype, str(device))
    bias = _CAUSAL_BIAS.get(key)
    if bias is None:
        if len(_CAUSAL_BIAS) > 16:
            _CAUSAL_BIAS.clear()
        bias = torch.full((S, S), float("-inf"), dtype=dtype, device=device).triu_(1)
        _CAUSAL_BIAS[key] = bias
    return bias


def causal_attention(q: Tensor, k: Tensor, v: Tensor, scale: float | None = None) -> Tensor:
    """q: [B, Hq, S, D]; k, v: [B, Hkv, S, D] (Hq a multiple of Hkv). Causal."""
    B, Hq, S, D = q.shape
    Hkv = k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if _composable() or not q.is_cuda:
        # Explicit softmax(QK^T)V: differentiable to any order on every backend.  Three passes
        # over the [B, H, S, S] scores instead of six: the scale goes onto q, the causal mask
        # is the additive input of the batched product, and the softmax reads and writes the
        # tensors' own dtype (its arithmetic is fp32 inside the kernel for 16-bit inputs).
        if Hkv != Hq:
            rep = Hq // Hkv
            k = k.repeat_interleave(rep, dim=1)
            v = v.repeat_interleave(rep, dim=1)
        bias = _causal_bias(S, q.dtype, q.device)
        att = torch.baddbmm(bias, (q * scale).reshape(B * Hq, S, D), k.reshape(B * Hq, S, D).transpose(1, 2))
        att = _softmax_last(att)
        return torch.bmm(att, v.reshape(B * Hq, S, D)).view(B, Hq, S, D)
    return F.scaled_dot_product_attention(
        q, k, v, is_causal=True, scale=scale, enable_gqa=(Hkv != Hq)
    )


# --------------------------------------------------------------------------- #
# cross entropy on logits (per-token losses)
# --------------------------------------------------------------------------- #


def token_cross_entropy_ref(
    logits: Tensor, targets: Tensor, ignore_index: int = -100, label_smoothing: float = 0.0
) -> Tensor:
    z = logits if logits.dtype == torch.float64 else logits.float()
    return F.cross_entropy(
        z, targets, reduction="none", ignore_index=ignore_index, label_smoothing=label_smoothing
    )


class _TokenCEBwdFn(torch.autograd.Function):
    """``dlogits = (softmax(logits) - onehot) * dloss`` as a function of ``(logits, dloss)`` with
    its own backward kernel, so that a graph built with ``create_graph=True`` can be
    differentiated once more (``lse`` is the forward's log-sum-exp of ``logits``; its
    dependence on ``logits`` is part of the kernel's formula)."""

    @staticmethod
    def forward(ctx, logits, dloss, targets, lse, ignore_index):
        from . import native

        dloss = dloss.contiguous().float()
        ctx.save_for_backward(logits, dloss, targets, lse)
        ctx.ignore_index = ignore_index
        return native.ce_bwd(logits, targets, lse, dloss, ignore_index)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, c):
        from . import native

        logits, dloss, targets, lse = ctx.saved_tensors
        d_logits, d_dloss = native.ce_bwd_bwd(c.contiguous(), logits, targets, lse, dloss, ctx.ignore_index)
        return d_logits, d_dloss, None, None, None


class _TokenCEFn(torch.autograd.Function):
    """Per-row CE over ``[T, V]`` logits: one pass computes loss and log-sum-exp;
    the backward rewrites ``(softmax - onehot) * dloss`` in one pass, in the logits'
    own dtype, without an fp32 ``[T, V]`` intermediate; the backward of that backward is a
    kernel as well."""

    @staticmethod
    def forward(ctx, logits, targets, ignore_index):
        from . import native

        loss, lse = native.ce_fwd(logits.contiguous(), targets, ignore_index)
        ctx.save_for_backward(logits, targets, lse)  # the input itself: it keeps its place in the graph
        ctx.ignore_index = ignore_index
        return loss

    @staticmethod
    def backward(ctx, dloss):
        logits, targets, lse = ctx.saved_tensors
        return _TokenCEBwdFn.apply(logits.contiguous(), dloss, targets, lse, ctx.ignore_index), None, None


def token_cross_entropy(
    logits: Tensor, targets: Tensor, ignore_index: int = -100, label_smoothing: float = 0.0
) -> Tensor:
    """``[T, V]`` logits, ``[T]`` targets -> ``[T]`` fp32 losses (0 where ignored)."""
    if (
        label_smoothing == 0.0
        and logits.dtype in (torch.bfloat16, torch.float16, torch.float32)
        and _kernels_ready(logits, targets)
        and logits.shape[0] > 0
    ):
        return _TokenCEFn.apply(logits, targets, ignore_index)
    return token_cross_entropy_ref(logits, targets, ignore_index, label_smoothing)
