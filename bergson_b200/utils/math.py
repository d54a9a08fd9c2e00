"""Loss and spectrum helpers.

``weighted_causal_lm_ce`` is the training / attribution loss
(reference ``bergson/utils/math.py:11-111``); ``compute_lambda`` picks the TrackStar
Hessian mixing coefficient (``:149-226``).
"""

from __future__ import annotations

import math
from typing import Mapping

import torch
import torch.nn.functional as F
from torch import Tensor

_REDUCTIONS = ("mean", "sum", "sum_of_means")


def weighted_causal_lm_ce(
    logits: Tensor,
    labels: Tensor,
    *,
    example_weight: Tensor | None = None,
    ignore_index: int = -100,
    shift_loss_mask: Tensor | None = None,
    vocab_size: int | None = None,
    reduction: str = "mean",
    padded_vocab: bool = False,
    **_ignored,
) -> Tensor:
    """Next-token cross entropy with per-example ``[B]`` or per-token ``[B, T]``
    weights.  Logits are upcast to fp32 (fp64 stays fp64).  ``reduction``:

    * ``mean``: weighted sum / number of supervised tokens in the batch;
    * ``sum``: weighted sum;
    * ``sum_of_means``: per-row weighted mean, summed over rows.
    """
    if reduction not in _REDUCTIONS:
        raise ValueError(f"Unknown reduction {reduction!r}")
    assert logits.ndim == 3 and labels.ndim == 2
    B, T, V = logits.shape
    assert labels.shape == (B, T)
    if vocab_size is not None and not padded_vocab:
        assert V == vocab_size, f"Expected vocab size {vocab_size}, got {V}"
    if padded_vocab:
        # Columns from vocab_size on hold a large negative constant: they vanish from the softmax.
        assert vocab_size is not None and vocab_size <= V < vocab_size + 8, (vocab_size, V)
    if example_weight is not None:
        assert example_weight.shape in ((B,), (B, T))

    z = logits[:, :-1]
    tgt = labels[:, 1:].reshape(-1)
    if z.is_cuda and z.dtype in (torch.bfloat16, torch.float16, torch.float32):
        # Per-token CE on the kernels (fp32 arithmetic on the logits' own dtype, no fp32 copy of
        # the [tokens, vocabulary] matrix; differentiable twice).
        from ..ops import token_cross_entropy

        if logits.is_contiguous():
            # All T positions with the targets shifted and the last one ignored: the [B, T, V]
            # logits are read in place instead of copying the [:, :-1] slice.
            shifted = torch.cat([labels[:, 1:], labels.new_full((B, 1), ignore_index)], dim=1).reshape(-1)
            tok = token_cross_entropy(logits.view(-1, V), shifted, ignore_index=ignore_index).view(B, T)[:, :-1]
        else:
            tok = token_cross_entropy(z.reshape(-1, V), tgt, ignore_index=ignore_index).view(B, T - 1)
        if example_weight is None and reduction == "mean":
            return tok.sum() / (tgt != ignore_index).sum().clamp_min(1)
    else:
        z = (z if z.dtype == torch.float64 else z.float()).reshape(-1, V)
        if example_weight is None and reduction == "mean":
            return F.cross_entropy(z, tgt, ignore_index=ignore_index)
        tok = F.cross_entropy(z, tgt, reduction="none", ignore_index=ignore_index)
        tok = tok.view(B, T - 1)
    if example_weight is None:
        w = tok.new_ones(B, 1)
    elif example_weight.ndim == 2:
        w = example_weight[:, :-1].to(tok.dtype)
    else:
        w = example_weight.to(tok.dtype).view(B, 1)
    weighted = tok * w

    if reduction == "sum":
        return weighted.sum()
    valid = (
        shift_loss_mask[:, :-1]
        if shift_loss_mask is not None
        else labels[:, 1:] != ignore_index
    )
    if reduction == "sum_of_means":
        counts = valid.to(tok.dtype).sum(1).clamp_min(1.0)
        return (weighted.sum(1) / counts).sum()
    return weighted.sum() / valid.sum().clamp_min(1)


def reshape_to_nearest_square(a: Tensor) -> Tensor:
    """View the last two dims as the most-square factorisation of their product."""
    n = math.prod(a.shape[-2:])
    if n == 0:
        raise ValueError("empty tensor")
    rows = next(d for d in range(math.isqrt(n), 0, -1) if n % d == 0)
    return a.reshape(*a.shape[:-2], rows, n // rows)


def trace(matrices: Tensor) -> Tensor:
    """Batched trace with two trailing singleton dims (broadcasts against matrices)."""
    return torch.linalg.diagonal(matrices).sum(-1)[..., None, None]


def compute_lambda(
    query_eigen: Mapping[str, tuple[Tensor, Tensor]],
    index_eigen: Mapping[str, tuple[Tensor, Tensor]],
    target_components: int = 1000,
) -> float:
    """Mixing coefficient ``lam`` with ``lam*s_q[k] = (1-lam)*s_i[k]`` at the k-th
    largest pooled eigenvalue (k = ``target_components``), i.e.
    ``lam = s_i[k] / (s_q[k] + s_i[k])`` clipped to [0, 1]."""
    q_vals, i_vals = [], []
    for name, (qv, _) in query_eigen.items():
        if name in index_eigen:
            q_vals.append(qv.double().clamp(min=0))
            i_vals.append(index_eigen[name][0].double().clamp(min=0))
    if not q_vals:
        return 0.99
    q = torch.cat(q_vals).sort(descending=True).values
    i = torch.cat(i_vals).sort(descending=True).values
    if target_components <= 0:
        return 1.0
    k = min(target_components, len(q)) - 1
    sq, si = q[k].item(), i[k].item()
    if sq + si == 0:
        return 0.99
    return max(0.0, min(1.0, si / (sq + si)))
