"""Python entry points of the attribution kernels with torch fallbacks.

* ``project_right`` / ``project_left_outer``: the two halves of the per-example
  projected gradient (see ``csrc/attribution.cu``).
* ``score_rows``: ``rows @ queries^T`` (+ per-row sum of squares) on the tcgen05 TN GEMM.
* ``topk_scores``: store-resident query: GEMM tiles + running top-k.
"""

from __future__ import annotations

import torch
from torch import Tensor

from . import native
from .functional import use_fused

_TC_DTYPES = (torch.bfloat16, torch.float16)


def kernel_status(device: int = 0) -> int:
    """Non-zero when a kernel gave up on one of its bounded waits (synchronises)."""
    return int(native.kernel_status(device).item())


def project_right(a: Tensor, p_in: Tensor) -> Tensor:
    """``a [T, I] @ p_in[16, I]^T`` -> fp32 ``[T, 16]``."""
    if use_fused(a, p_in) and a.dtype in _TC_DTYPES and a.shape[1] % 8 == 0:
        return native.proj_right(a.contiguous(), p_in.to(a.dtype).contiguous())
    return a.float() @ p_in.float().T


def project_left_outer(g: Tensor, p_out: Tensor, a_proj: Tensor, acc: Tensor, col_off: int) -> None:
    """``acc[n, col_off:col_off+256] += vec((g_n p_out^T)^T a_proj_n)``."""
    N, S, O = g.shape
    if use_fused(g, acc) and g.dtype in _TC_DTYPES and O % 8 == 0:
        native.proj_left_outer(g.contiguous(), p_out.to(g.dtype).contiguous(), a_proj.contiguous(), acc, col_off)
        return
    gp = g.float() @ p_out.float().T
    blk = torch.einsum("nsi,nsj->nij", gp, a_proj.view(N, S, -1).float()).reshape(N, -1)
    acc[:, col_off : col_off + blk.shape[1]] += blk


def score_rows(rows: Tensor, queries: Tensor, dtype: torch.dtype, need_sq: bool) -> tuple[Tensor, Tensor | None]:
    """``rows [B, D]``, ``queries [Q, D]`` -> (fp32 ``[B, Q]`` inner products, optional
    fp32 ``[B]`` sums of squares of the rows as rounded to ``dtype``)."""
    rows = rows.to(dtype)
    queries = queries.to(dtype)
    if use_fused(rows, queries) and dtype in _TC_DTYPES and rows.shape[1] % 8 == 0:
        rows = rows.contiguous()
        queries = queries.contiguous()
        if rows.shape[0] >= 512 and queries.shape[0] % 4 == 0:
            # Many rows on both sides (a query batch against a store chunk): the wide CTA-pair GEMM
            # with fp32 output; the 128-row kernel below serves the small per-batch products.
            scores, _ = native.gemm(rows, queries, False, False, None, True, None, False, None, cta_group=2, wide=True)
        else:
            scores = native.tn_gemm(rows, queries)
        sq = None
        if need_sq:
            sq = torch.zeros(rows.shape[0], device=rows.device, dtype=torch.float32)
            native.row_sumsq(rows, sq)
        return scores, sq
    scores = (rows @ queries.T).float()
    sq = rows.float().pow(2).sum(1) if need_sq else None
    return scores, sq


def topk_scores(store: Tensor, queries: Tensor, k: int, *, largest: bool = True, inv_norms: Tensor | None = None,
                chunk: int = 65536) -> tuple[Tensor, Tensor]:
    """Top-k of ``queries [Q, D] @ store[N, D]^T`` over N without materialising the
    ``[Q, N]`` score matrix: the store is scanned in row chunks, each chunk's scores come
    from the TN GEMM and are merged into a running top-k.  ``inv_norms`` ([N]) scales the
    columns (cosine scoring against a unit-normalised store)."""
    Q = queries.shape[0]
    N = store.shape[0]
    k = min(k, N)
    best_v = best_i = None
    for lo in range(0, N, chunk):
        hi = min(lo + chunk, N)
        part, _ = score_rows(queries, store[lo:hi], store.dtype if store.dtype in _TC_DTYPES else torch.float32, False)
        if inv_norms is not None:
            part = part * inv_norms[lo:hi].unsqueeze(0)
        v, i = torch.topk(part, min(k, hi - lo), dim=1, largest=largest)
        i = i + lo
        if best_v is None:
            best_v, best_i = v, i
        else:
            cat_v, cat_i = torch.cat([best_v, v], 1), torch.cat([best_i, i], 1)
            best_v, sel = torch.topk(cat_v, k, dim=1, largest=largest)
            best_i = cat_i.gather(1, sel)
    assert best_v is not None and best_i is not None
    return best_v, best_i


# --------------------------------------------------------------------------- #
# Gram / covariance accumulation
# --------------------------------------------------------------------------- #

_UPPER_ONLY: set[int] = set()  # data_ptrs of accumulators filled through the SYRK kernel


def gram_fused_ok(x: Tensor) -> bool:
    return (
        x.dim() == 2 and x.dtype in _TC_DTYPES and x.shape[1] % 8 == 0 and x.shape[0] > 0 and use_fused(x)
    )


def gram_accumulate(acc: Tensor, x: Tensor) -> None:
    """``acc [D, D] (fp32) += x^T x`` on the tcgen05 SYRK kernel.  Only 128 x 256 tiles that
    touch the upper triangle are written; call ``gram_finalize`` before reading."""
    native.cov_syrk(x.contiguous(), [acc.data_ptr()], [0, acc.shape[0]], None)
    _UPPER_ONLY.add(acc.data_ptr())


def gram_finalize(store: dict[str, Tensor]) -> None:
    """Mirror the upper triangle of every accumulator that the SYRK kernel filled."""
    for name, m in store.items():
        if m.data_ptr() in _UPPER_ONLY:
            _UPPER_ONLY.discard(m.data_ptr())
            store[name] = torch.triu(m) + torch.triu(m, 1).T


# --------------------------------------------------------------------------- #
# fp32-accurate rotation on 16-bit tensor cores
# --------------------------------------------------------------------------- #


def split_hi_lo(q: Tensor) -> Tensor:
    """``[2 * b, a]`` bf16 operand holding the rows of ``q^T`` split as ``hi + lo`` (``q`` is
    ``[a, b]`` fp32).  ``hi`` is the bf16 rounding, ``lo`` the bf16 rounding of the residual,
    so ``hi + lo`` carries about 16 mantissa bits."""
    qt = q.float().T.contiguous()
    hi = qt.to(torch.bfloat16)
    lo = (qt - hi.float()).to(torch.bfloat16)
    return torch.cat([hi, lo], dim=0).contiguous()


def rotate(x: Tensor, q: Tensor, q_split: Tensor | None = None) -> Tensor:
    """``x [..., a] @ q [a, b]`` in fp32 accuracy.  For bf16 ``x`` on CUDA the product runs on
    the tcgen05 TN GEMM against the hi/lo split of ``q`` (the activations are exact in bf16,
    the two partial products are accumulated in fp32); otherwise a plain fp32 matmul."""
    lead, a = x.shape[:-1], x.shape[-1]
    b = q.shape[1]
    if x.dtype == torch.bfloat16 and a % 8 == 0 and use_fused(x, q):
        qs = q_split if q_split is not None else split_hi_lo(q)
        out = native.tn_gemm(x.reshape(-1, a).contiguous(), qs)  # [T, 2b] fp32
        return (out[:, :b] + out[:, b:]).view(*lead, b)
    return x.to(q.dtype) @ q


def split_matmul(a: Tensor, b: Tensor) -> Tensor:
    """``a [M, K] @ b [K, N]`` for fp32 operands at close to fp32 accuracy on the 16-bit tensor
    cores.  Each operand is written as ``hi + lo`` (bf16 rounding and bf16-rounded residual);
    ``hi hi + hi lo + lo hi`` is evaluated as *one* GEMM with the three terms laid side by side
    along the reduction axis (``[ah | ah | al] @ [bh ; bl ; bh]``), accumulated in fp32 by the
    persistent tcgen05 kernel.  The dropped ``lo lo`` term is ~2^-16 relative.  Falls back to a
    plain matmul off CUDA or for shapes the kernel does not take."""
    M, K = a.shape
    N = b.shape[1]
    if not (use_fused(a, b) and a.dtype == torch.float32 and b.dtype == torch.float32 and K % 8 == 0 and N % 8 == 0
            and M > 0):
        return a @ b
    ah = a.to(torch.bfloat16)
    al = (a - ah.float()).to(torch.bfloat16)
    bh = b.to(torch.bfloat16)
    bl = (b - bh.float()).to(torch.bfloat16)
    lhs = torch.cat([ah, ah, al], dim=1).contiguous()          # [M, 3K], K-major
    rhs = torch.cat([bh, bl, bh], dim=0).contiguous()          # [3K, N], read MN-major
    return native.gemm(lhs, rhs, False, True, None, True)[0]
