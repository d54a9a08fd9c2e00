"""Finalisation of autocorrelation Grams: normalise by the row count, combine the
ranks' partial sums, eigendecompose in fp64.

The reference eigendecomposes every rank's *partial* Gram before summing
(``bergson/process_autocorrelation.py:38-44,73-85``), which is only meaningful when
each module's rows live on one rank.  Here the partial Grams are summed first and the
sum is decomposed, so ``hessians_eigen`` is the eigendecomposition of ``hessians``
for any world size; with one rank both agree.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from .gradients import GradientProcessor


def process_autocorrelation_matrices(
    processor: GradientProcessor,
    hessians: dict[str, torch.Tensor],
    num_rows: int,
    grad_sizes: dict[str, int],
    rank: int,
):
    first = next(iter(hessians.values()))
    device, dtype = first.device, first.dtype
    distributed = dist.is_initialized() and dist.get_world_size() > 1
    out_h: dict[str, torch.Tensor] = {}
    out_e: dict[str, tuple[torch.Tensor, torch.Tensor]] = {}
    for name, size in grad_sizes.items():
        local = hessians.get(name)
        if local is None:
            local = torch.zeros(size, size, dtype=dtype, device=device)
        h = local / num_rows
        if distributed:
            dist.all_reduce(h, op=dist.ReduceOp.SUM)
        if rank == 0 or not distributed:
            vals, vecs = torch.linalg.eigh(h.to(torch.float64))
            out_h[name] = h.cpu()
            out_e[name] = (vals.to(dtype).contiguous().cpu(), vecs.to(dtype).contiguous().cpu())
    hessians.clear()
    if rank == 0 or not distributed:
        processor.hessians = out_h
        processor.hessians_eigen = out_e
