"""Sequence-parallel tensor parallelism with the collectives inside the GEMM kernels.

Between the blocks of a tensor-parallel model the residual stream is kept *sharded over
tokens* (rank r holds rows ``[r T/W, (r + 1) T/W)``).  The two kinds of projection then map
onto two fused kernels over NVLink peer memory:

* column-parallel (q/k/v, gate/up; weights split by output features): **all-gather -> GEMM**.
  Every rank publishes its token shard once in a symmetric buffer.  The first projection that
  consumes it runs the gather inside its GEMM kernel: one copier warp per CTA pulls the other
  ranks' row blocks over NVLink into a local buffer while the tensor cores work on the tiles of
  the rank's own rows; tiles of remote rows start when the copiers' counters say their rows
  have landed (bounded wait).  Every remote byte crosses NVLink once (peer reads are not cached
  in the local L2, so reading A tiles straight from the peers would fetch them once per output
  tile column); the other projections of the same input then read the local copy.
* row-parallel (o_proj, down_proj; weights split by input features): **GEMM -> reduce-scatter**.
  The epilogue stores each output row block into the slot ``[source rank]`` of the row
  owner's buffer (peer stores); after a flag barrier the owner adds the W slots in rank order
  (and the residual) in one pass.  The sum is therefore deterministic.

The backward passes are the mirrored kernels (the input gradient of a column-parallel
projection is a GEMM -> reduce-scatter, that of a row-parallel one an all-gather -> GEMM), and
the collector's projection taps ride on the same GEMMs as in the single-GPU path.

Ordering between ranks comes from ``peer_barrier``: a one-block kernel on the stream that
signals every peer and waits, with a cycle budget, for their signals.  A peer that never
arrives makes the wait run out: the kernel then sets the status word that
``check_kernel_status`` reports and returns, and nothing spins for ever.  Buffers are double
buffered, which together with one barrier per use rules out overwriting data a peer still
reads (a rank can only reach use k + 2 of a buffer after every peer has signalled barrier
k + 1, i.e. after the peer's kernels of use k have finished).

The reference has no tensor parallelism.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
from torch import Tensor

from .peer import PeerHeap, symmetric_memory_available

ROW_BLOCK = 128  # rows that one CTA loads; a block must not straddle two ranks' shards
MAX_CONSUMERS = 3  # projections sharing one published input (q/k/v): their input gradients share a reduce-scatter


class SeqParallel:
    """Peer buffers and barrier epochs of one tensor-parallel group."""

    def __init__(self, group):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self._heap: PeerHeap | None = None
        self._flags: PeerHeap | None = None
        self._shape: tuple[int, int, torch.dtype] | None = None
        self._epoch = 0
        self._gather_use = 0
        self._slot_use = 0
        self.barriers = 0  # counters read by the tests
        self.fused_gemms = 0

    # -- set-up -----------------------------------------------------------------------------

    def available(self) -> bool:
        from ..ops import native

        return self.world > 1 and self.world <= 8 and native.available() and symmetric_memory_available()

    def fits(self, tokens: int, width: int, dtype: torch.dtype) -> bool:
        return (dtype in (torch.bfloat16, torch.float16) and tokens % (ROW_BLOCK * self.world) == 0
                and width % 8 == 0)

    def ensure(self, tokens: int, width: int, dtype: torch.dtype) -> None:
        """(Re)allocate the symmetric buffers for ``tokens x width`` activations.  Collective:
        all ranks of the group see the same shapes, so they take this branch together."""
        rows = tokens // self.world
        if self._shape is not None and self._shape[0] >= rows and self._shape[1] >= width and self._shape[2] == dtype:
            return
        if self._flags is None:
            self._flags = PeerHeap(8, torch.int32, self.group)
            self._flags.local.zero_()
        per = rows * width
        self._heap = PeerHeap((2 + 2 * MAX_CONSUMERS * self.world) * per, dtype, self.group)
        self._shape = (rows, width, dtype)
        self._per = per
        self._heap.barrier()  # zeroed flags and the new mappings are in place everywhere

    # -- primitives -------------------------------------------------------------------------

    def barrier(self) -> None:
        from ..ops import native

        self._epoch += 1
        self.barriers += 1
        native.peer_barrier(self._flags.ptrs, self.rank, self._epoch)

    def gather_counters(self) -> Tensor:
        """Arrival counters of the copier warps (zeroed by every launch that uses them)."""
        if getattr(self, "_counters", None) is None:
            self._counters = torch.zeros(8, dtype=torch.int32, device=self._heap.local.device)
        return self._counters

    def _gather_offset(self, use: int) -> int:
        return (use & 1) * self._per

    def _slot_offset(self, use: int) -> int:
        return (2 + (use & 1) * MAX_CONSUMERS * self.world) * self._per

    def publish(self, shard: Tensor) -> list[int]:
        """Copy this rank's ``[rows, width]`` shard into the current gather buffer and pass the
        barrier; returns every rank's address of that buffer."""
        rows, width = shard.shape
        off = self._gather_offset(self._gather_use)
        self._gather_use += 1
        self._heap.local[off : off + rows * width].view(rows, width).copy_(shard)
        self.barrier()
        return [self._heap.ptr(r, off) for r in range(self.world)]

    def slot_targets(self) -> tuple[list[int], Tensor]:
        """Addresses of the current slot region on every rank, and this rank's own region."""
        off = self._slot_offset(self._slot_use)
        self._slot_use += 1
        local = self._heap.local[off : off + MAX_CONSUMERS * self.world * self._per]
        return [self._heap.ptr(r, off) for r in range(self.world)], local

    def reduce_slots(self, local: Tensor, rows: int, width: int, residual: Tensor | None, groups: int = 1) -> Tensor:
        """Barrier, then the sum of ``groups * world`` slots (+ residual) in a fixed order."""
        from ..ops import native

        self.barrier()
        n = groups * self.world
        slots = local[: n * rows * width].view(n, rows, width)
        return native.slot_reduce(slots, residual.contiguous() if residual is not None else None)


class Published:
    """A token shard that sits in the peers' gather buffers (valid until two publishes later),
    and the local ``[T, width]`` buffer that the first consuming GEMM completes."""

    def __init__(self, sp: SeqParallel, shard: Tensor):
        self.sp = sp
        self.shard = shard
        rows, width = shard.shape
        self.full = torch.empty(sp.world * rows, width, dtype=shard.dtype, device=shard.device)
        self.full[sp.rank * rows : (sp.rank + 1) * rows].copy_(shard.detach())
        self.ptrs = sp.publish(shard.detach())
        self.gathered = False
        self.consumers = 0        # projections whose input gradient will come back
        self._pushed = 0          # of those, how many have pushed their partial gradient so far
        self._slots = None

    def release(self) -> None:
        """Drop the gathered copy once every forward consumer has run."""
        self.full = None

    def push_target(self, rows: int, width: int) -> tuple[list[int], int]:
        """Slot addresses for the next consumer's partial input gradient, and its group index."""
        sp = self.sp
        if self._slots is None:
            self._slots = sp.slot_targets()
        idx = self._pushed
        self._pushed += 1
        skip = idx * sp.world * rows * width * sp._heap.itemsize
        return [p + skip for p in self._slots[0]], idx

    def finish_if_last(self, rows: int, width: int):
        """The reduce-scattered sum of all consumers' input gradients once the last one has
        pushed (one barrier and one reduction for the whole group), else None."""
        if self._pushed < self.consumers:
            return None
        return self.sp.reduce_slots(self._slots[1], rows, width, None, groups=self._pushed)

    def gemm(self, weight: Tensor, b_mn: bool, aux_p: Tensor | None):
        """``gather(shards) @ op(weight)`` (+ the projection side output): the first call pulls
        the remote rows inside its kernel, later calls find them in ``full``."""
        from ..ops import native

        sp = self.sp
        if self.gathered or self.full.shape[0] // sp.world % 512:
            if not self.gathered:  # blocks too small for the fused form: gather with a copy
                dist.all_gather_into_tensor(self.full, self.shard.detach().contiguous(), group=sp.group)
                self.gathered = True
            return native.gemm(self.full, weight, False, b_mn, None, False, None, False, aux_p, cta_group=2, wide=True)
        out = native.gemm(self.full, weight, False, b_mn, None, False, None, False, aux_p, cta_group=2, wide=True,
                          a_peer_ptrs=self.ptrs, gather_done=sp.gather_counters(), gather_rank=sp.rank)
        sp.fused_gemms += 1
        self.gathered = True
        return out


def _tap_operands(module, tap, lead: tuple[int, int], like: Tensor):
    if tap is None:
        return None
    probe = like.new_empty((lead[0], lead[1], 0))  # carries batch size, dtype and device only
    taps = tap.operands(module, probe)
    if taps is None and (module._forward_hooks or module._backward_hooks):
        raise RuntimeError(f"{getattr(module, '_name', type(module).__name__)}: its collector declined the fused "
                           "projection, and the sequence-parallel path cannot serve hook-based collection")
    return taps


def hooks_compatible(modules) -> bool:
    """True when no module relies on hooks that this path would bypass (a module with hooks
    must also carry a projection tap)."""
    return all(hasattr(m, "_tap") or not (m._forward_hooks or m._backward_hooks or m._forward_pre_hooks)
               for m in modules)


def _check_hooks(module, taps) -> None:
    if taps is None and torch.is_grad_enabled() and (module._forward_hooks or module._backward_hooks):
        raise RuntimeError(
            f"{getattr(module, '_name', type(module).__name__)}: the sequence-parallel path runs the projection "
            "without calling the module, so hook-based collection would miss it; use the fused collection path "
            "or disable sequence parallelism (BERGSON_B200_DISABLE_PEER=1)")


class _GatherLinearFn(torch.autograd.Function):
    """``y [T, N] = gather(x_shard) @ W^T`` with the gather inside the GEMM's A loads."""

    @staticmethod
    def forward(ctx, shard: Tensor, weight: Tensor, pub: Published, module, tap, lead):
        from ..ops import native

        sp = pub.sp
        taps = _tap_operands(module, tap, lead, shard) if tap is not None else None
        y, a_proj = pub.gemm(weight, False, taps[0] if taps is not None else None)
        ctx.pub = pub
        ctx.save_for_backward(weight, taps[1] if taps is not None else None, a_proj if taps is not None else None)
        ctx.sp, ctx.module, ctx.tap, ctx.lead = sp, module, tap if taps is not None else None, lead
        ctx.rows = shard.shape[0]
        return y

    @staticmethod
    def backward(ctx, g: Tensor):
        from ..ops import native

        weight, p_out, a_proj = ctx.saved_tensors
        sp = ctx.sp
        g = g.contiguous()
        rows, width = ctx.rows, weight.shape[1]
        if weight.requires_grad:
            raise NotImplementedError("sequence-parallel projections do not produce weight gradients")
        ptrs, _ = ctx.pub.push_target(rows, width)
        _, g_proj = native.gemm(g, weight, False, True, None, False, None, False, p_out, cta_group=2, wide=True,
                                d_peer_ptrs=ptrs, d_rows_per_rank=rows, d_slot=sp.rank)
        sp.fused_gemms += 1
        if ctx.tap is not None:
            ctx.tap.collect(ctx.module, a_proj, g_proj, torch.Size(ctx.lead))
        # The projections that share this input share one reduce-scatter: the last one to push
        # returns the summed gradient, the others contribute nothing of their own.
        return ctx.pub.finish_if_last(rows, width), None, None, None, None, None


class _ScatterLinearFn(torch.autograd.Function):
    """``y_shard [T / W, N] = residual + reduce_scatter(x @ W^T)`` with the scatter in the
    GEMM's epilogue (``x`` holds this rank's slice of the input features for all tokens)."""

    @staticmethod
    def forward(ctx, x: Tensor, weight: Tensor, residual: Tensor | None, sp: SeqParallel, module, tap, lead):
        from ..ops import native

        taps = _tap_operands(module, tap, lead, x) if tap is not None else None
        x = x.contiguous()
        rows = x.shape[0] // sp.world
        ptrs, local = sp.slot_targets()
        _, a_proj = native.gemm(x, weight, False, False, None, False, None, False,
                                taps[0] if taps is not None else None, cta_group=2, wide=True,
                                d_peer_ptrs=ptrs, d_rows_per_rank=rows, d_slot=sp.rank)
        sp.fused_gemms += 1
        y = sp.reduce_slots(local, rows, weight.shape[0], residual)
        ctx.save_for_backward(weight, taps[1] if taps is not None else None, a_proj if taps is not None else None)
        ctx.sp, ctx.module, ctx.tap, ctx.lead = sp, module, tap if taps is not None else None, lead
        ctx.has_residual = residual is not None
        return y

    @staticmethod
    def backward(ctx, g: Tensor):
        from ..ops import native

        weight, p_out, a_proj = ctx.saved_tensors
        sp = ctx.sp
        if weight.requires_grad:
            raise NotImplementedError("sequence-parallel projections do not produce weight gradients")
        dx, g_proj = Published(sp, g.contiguous()).gemm(weight, True, p_out)
        if ctx.tap is not None:
            ctx.tap.collect(ctx.module, a_proj, g_proj, torch.Size(ctx.lead))
        return dx, None, (g if ctx.has_residual else None), None, None, None, None


def gather_linear(pub: Published, module, lead: tuple[int, int]) -> Tensor:
    """Column-parallel projection of a published token shard: ``[T, out_local]``."""
    tap = getattr(module, "_tap", None)
    if tap is not None and not (torch.is_grad_enabled() and pub.shard.requires_grad):
        tap = None
    if tap is None:
        _check_hooks(module, None)
    if torch.is_grad_enabled() and pub.shard.requires_grad:
        if pub.consumers >= MAX_CONSUMERS:
            raise RuntimeError(f"at most {MAX_CONSUMERS} projections may share one published input")
        pub.consumers += 1
    return _GatherLinearFn.apply(pub.shard, module.weight, pub, module, tap, lead)


def scatter_linear(x: Tensor, module, sp: SeqParallel, lead: tuple[int, int], residual: Tensor | None = None) -> Tensor:
    """Row-parallel projection: ``[T / W, out]`` token shard of the summed output (+ residual)."""
    tap = getattr(module, "_tap", None)
    if tap is not None and not (torch.is_grad_enabled() and x.requires_grad):
        tap = None
    if tap is None:
        _check_hooks(module, None)
    return _ScatterLinearFn.apply(x, module.weight, residual, sp, module, tap, lead)


class _GatherTokensFn(torch.autograd.Function):
    """Token shards -> all tokens on every rank, for a consumer that every rank evaluates
    identically (the replicated head and loss): the backward is this rank's slice."""

    @staticmethod
    def forward(ctx, shard: Tensor, sp: SeqParallel):
        shard = shard.contiguous()
        out = torch.empty((sp.world * shard.shape[0], shard.shape[1]), dtype=shard.dtype, device=shard.device)
        dist.all_gather_into_tensor(out, shard, group=sp.group)
        ctx.rows, ctx.rank = shard.shape[0], sp.rank
        return out

    @staticmethod
    def backward(ctx, g: Tensor):
        return g[ctx.rank * ctx.rows : (ctx.rank + 1) * ctx.rows].contiguous(), None


def gather_tokens(shard: Tensor, sp: SeqParallel) -> Tensor:
    return _GatherTokensFn.apply(shard, sp)
