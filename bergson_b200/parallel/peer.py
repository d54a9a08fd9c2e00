"""Peer-memory heap over NVLink / NVSwitch and the collectives fused into our kernels.

``PeerHeap`` allocates one symmetric buffer per rank with
``torch.distributed._symmetric_memory`` (CUDA VMM allocations whose handles are exchanged
through the process group) and exposes every rank's device pointer.  Kernels then address
remote memory directly:

* ``reduce_scatter_gram``: the covariance kernel's epilogue adds every output row into the
  buffer of the rank that owns it with P2P ``red.global.add`` — optionally together with
  the last batch's ``X^T X`` product, i.e. GEMM -> reduce-scatter in one kernel;
* ``gathered_scores``: the score GEMM reads the query rows of every rank through plain
  (non-multicast) TMA loads from the owners' buffers — all-gather -> GEMM in one kernel.

No kernel of this module waits on a flag: ordering between ranks comes from host-side
barriers of the process group placed around the launches, so a missing peer can never
make a kernel spin.  NCCL remains the fallback (and the baseline in the tests).
"""

from __future__ import annotations

import torch
import torch.distributed as dist
from torch import Tensor

from ..hessians.sharded_computation import shard_bounds


def symmetric_memory_available() -> bool:
    try:
        import torch.distributed._symmetric_memory  # noqa: F401
    except Exception:
        return False
    # Peers are addressed through their device mappings: every rank must see more than its own GPU.
    return (torch.cuda.is_available() and dist.is_initialized() and dist.get_backend() != "gloo"
            and (dist.get_world_size() == 1 or torch.cuda.device_count() > 1))


class PeerHeap:
    """A symmetric allocation of ``numel`` elements of ``dtype`` on every rank."""

    def __init__(self, numel: int, dtype: torch.dtype = torch.float32, group=None):
        import torch.distributed._symmetric_memory as symm

        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        device = torch.device("cuda", torch.cuda.current_device())
        self.local = symm.empty(numel, dtype=dtype, device=device)
        self.handle = symm.rendezvous(self.local, group=self.group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.itemsize = self.local.element_size()

    def ptr(self, rank: int, offset_elems: int = 0) -> int:
        return self.ptrs[rank] + offset_elems * self.itemsize

    def barrier(self) -> None:
        """All ranks' prior writes to the heap are visible after this returns."""
        torch.cuda.synchronize()
        dist.barrier(group=self.group)


def reduce_scatter_gram(local_full: Tensor, heap: PeerHeap, offset_elems: int, x_last: Tensor | None = None) -> Tensor:
    """Sum ``local_full [D, D]`` (+ ``x_last^T x_last``) over ranks and return this rank's
    row shard ``[rows_r, D]`` (a view into the heap).  The heap region
    ``[offset, offset + rows_r * D)`` of every rank must have been zeroed and a
    ``heap.barrier()`` passed before the call; the result is complete after the
    ``heap.barrier()`` that this function issues."""
    from ..ops import native

    D = local_full.shape[0]
    bounds = [shard_bounds(D, r, heap.world) for r in range(heap.world)]
    row_start = [b[0] for b in bounds] + [D]
    if x_last is None:
        x_last = torch.zeros(64, D, device=local_full.device, dtype=torch.bfloat16)
        rows = 0
    else:
        rows = -1
    native.cov_syrk(x_last.contiguous(), [heap.ptr(r, offset_elems) for r in range(heap.world)], row_start,
                    local_full.contiguous(), True, rows)
    heap.barrier()
    lo, hi = bounds[heap.rank]
    return heap.local[offset_elems : offset_elems + (hi - lo) * D].view(hi - lo, D)


def gathered_scores(rows: Tensor, heap: PeerHeap, offset_elems: int, n_per_rank: int) -> Tensor:
    """``rows [B, K] @ concat_r(Q_r)^T`` where ``Q_r [n_per_rank, K]`` sits at
    ``offset_elems`` of rank r's heap (dtype of ``rows``).  Returns fp32 ``[B, world * n_per_rank]``."""
    from ..ops import native

    return native.tn_gemm_gathered(rows.contiguous(), [heap.ptr(r, offset_elems) for r in range(heap.world)],
                                   n_per_rank)
