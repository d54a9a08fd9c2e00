"""Eigendecomposition of Kronecker factors and EK-FAC eigenvalue correction
(reference ``bergson/hessians/eigenvectors.py``).

Directory layout produced (all row-sharded with ``shard_bounds``):
``eigen_activation_sharded/``, ``eigen_gradient_sharded/`` (rows of the eigenvector
matrix, columns = eigenvectors, ascending eigenvalues), ``eigenvalue_sharded/``
(``outer(l_G, l_A) * total_processed``), ``factor_eig_a/`` (full ``l_A * sqrt(T)``
replicated), ``factor_eig_g/`` (``l_G * sqrt(T)`` shard), and
``eigenvalue_correction_sharded/`` (``sum_n (Q_G^T G_n Q_A)^2``, un-normalised).
"""

from __future__ import annotations

import gc
import os
from contextlib import nullcontext
from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn as nn
from safetensors import safe_open
from safetensors.torch import load_file, save_file
from torch import Tensor

from ..collector.collector import HookCollectorBase
from ..utils.logger import get_logger
from ..utils.streamed_safetensors import StreamedSafetensors, save_tensors
from ..utils.utils import assert_type, get_device
from .sharded_computation import ShardedMul, shard_bounds


# Factors decomposed concurrently per rank (one host thread and one stream each).
EIGH_CONCURRENCY = int(os.environ.get("BERGSON_B200_EIGH_CONCURRENCY", "6"))


def fair_distribute_by_cost(key_dimensions: dict[str, int], world_size: int) -> list[list[str]]:
    """Deal keys to ranks in snake order of decreasing ``d^3`` cost."""
    order = sorted(key_dimensions, key=lambda k: key_dimensions[k] ** 3, reverse=True)
    out: list[list[str]] = [[] for _ in range(world_size)]
    for i, key in enumerate(order):
        rnd, pos = divmod(i, world_size)
        out[pos if rnd % 2 == 0 else world_size - 1 - pos].append(key)
    return out


@dataclass(kw_only=True)
class LambdaCollector(HookCollectorBase):
    """EK-FAC corrected eigenvalues ``L*[o, i] = sum_n (Q_G^T G_n Q_A)^2[o, i]`` with
    per-document gradients ``G_n``.  The eigenvector shards are gathered into local
    memory once in ``setup`` and reused by every batch; accumulation stays on the device."""

    path: str
    eigen_path: str | None = None
    output_subdir: str = "eigenvalue_correction_sharded"
    dtype: torch.dtype = torch.float32

    def setup(self) -> None:
        self.shard_computer = sc = ShardedMul()
        self.device = get_device(self.rank)
        src = self.eigen_path or self.path

        def load(sub: str) -> dict[str, Tensor]:
            shard = load_file(os.path.join(src, f"{sub}/shard_{self.rank}.safetensors"), device=self.device)
            return {k: sc.gather_rows(v.to(self.dtype), v.shape[1]) for k, v in shard.items()}

        self.eigen_a = load("eigen_activation_sharded")
        self.eigen_g = load("eigen_gradient_sharded")
        self.eigenvalue_corrections: dict[str, Tensor] = {}
        self.transformed_a_cache: dict[str, Tensor] = {}
        self._splits: dict[tuple[str, str], Tensor] = {}

    def _rotate(self, kind: str, name: str, x: Tensor, q: Tensor) -> Tensor:
        """``x @ q`` in the accumulation dtype; bf16 activations on CUDA go through the
        tensor-core rotation with an fp32-accurate split of ``q`` (cached per module)."""
        from ..ops import attribution

        if self.dtype == torch.float32 and x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
            key = (kind, name)
            if key not in self._splits:
                self._splits[key] = attribution.split_hi_lo(q)
            return attribution.rotate(x, q, self._splits[key])
        return x.to(self.dtype) @ q

    def forward_hook(self, module: nn.Module, a: Tensor) -> None:
        name = assert_type(str, module._name)
        if module._collect_bias:
            a = torch.cat([a, a.new_ones(*a.shape[:-1], 1)], dim=-1)
        self.transformed_a_cache[name] = self._rotate("a", name, a, self.eigen_a[name])

    def backward_hook(self, module: nn.Module, g: Tensor) -> None:
        name = assert_type(str, module._name)
        tg = self._rotate("g", name, g, self.eigen_g[name])  # [N, S, O]
        ta = self.transformed_a_cache.pop(name)  # [N, S, I]
        from ..ops.functional import use_fused

        if (tg.dtype == torch.float32 and tg.dim() == 3 and use_fused(tg, ta) and tg.shape[-1] % 8 == 0
                and ta.shape[-1] % 8 == 0 and tg.shape[1] > 0):
            # One batched tensor-core launch: per document (G_n Q_G)^T (A_n Q_A) in TMEM, squared and
            # added into the [O, I] grid by the epilogue -- the [N, O, I] products are never stored.
            from ..ops import native

            acc = self.eigenvalue_corrections.get(name)
            if acc is None:
                acc = self.eigenvalue_corrections[name] = torch.zeros(tg.shape[-1], ta.shape[-1], device=tg.device)
            native.gemm(tg.to(torch.bfloat16).contiguous(), ta.to(torch.bfloat16).contiguous(), True, True, acc, True,
                        None, False, None, 2, sq_accumulate=True)
            return
        if tg.is_cuda and tg.dtype == torch.float32:
            # Per-document outer products on TF32 tensor cores (fp32 accumulate); the result is
            # squared and summed over documents, so 10-bit operand mantissas are ample.
            prev = torch.backends.cuda.matmul.allow_tf32
            torch.backends.cuda.matmul.allow_tf32 = True
            try:
                per_doc = tg.mT @ ta  # [N, O, I]
            finally:
                torch.backends.cuda.matmul.allow_tf32 = prev
        else:
            per_doc = tg.mT @ ta
        upd = per_doc.square_().sum(dim=0)
        if name in self.eigenvalue_corrections:
            self.eigenvalue_corrections[name].add_(upd)
        else:
            self.eigenvalue_corrections[name] = upd

    def process_batch(self, indices: list[int], **kwargs) -> None:
        pass

    def teardown(self) -> None:
        sc = self.shard_computer
        out = {}
        for name, full in self.eigenvalue_corrections.items():
            if sc.dist:
                dist.all_reduce(full, op=dist.ReduceOp.SUM)
            lo, hi = sc.shard_bounds(full.shape[0])
            out[name] = full[lo:hi].contiguous()
        d = os.path.join(self.path, self.output_subdir)
        os.makedirs(d, exist_ok=True)
        save_tensors(out, os.path.join(d, f"shard_{self.rank}.safetensors"))


def _gather_and_shard_along_dim_0(input_dict, full_shape_per_key, dtype, rank, world_size, device, sink=None):
    """Every key lives on exactly one rank; sum-reduce (others contribute zeros) and keep
    this rank's rows.  With ``sink`` the shards are handed to ``sink(key, shard)`` on a helper
    thread (copy to the host and file write overlap the next key's reduction) and nothing is
    returned; otherwise the shards come back as host tensors."""
    if world_size == 1:
        assert sink is None
        return {k: v.cpu() for k, v in input_dict.items()}
    out = {}
    pool = None
    if sink is not None:
        from concurrent.futures import ThreadPoolExecutor

        pool = ThreadPoolExecutor(max_workers=2)
        dev = torch.device(device)

        def deliver(key, shard):
            if dev.type == "cuda":
                torch.cuda.set_device(dev)
            sink(key, shard)

    pending = []
    try:
        for key, shape in full_shape_per_key.items():
            t = (input_dict.pop(key).to(device=device, dtype=dtype) if key in input_dict
                 else torch.zeros(shape, device=device, dtype=dtype))
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
            lo, hi = shard_bounds(shape[0], rank, world_size)
            shard = t[lo:hi].contiguous()
            if pool is not None:
                if shard.is_cuda:
                    # The helper thread copies on its own stream: order it after the reduction.
                    shard.record_stream(torch.cuda.current_stream())
                    ev = torch.cuda.Event()
                    ev.record()
                    pending.append(pool.submit(_after_event, ev, deliver, key, shard))
                else:
                    pending.append(pool.submit(deliver, key, shard))
            else:
                out[key] = shard.cpu()
        for fut in pending:
            fut.result()
    finally:
        if pool is not None:
            pool.shutdown(wait=True)
    return out


def _after_event(event, fn, *args):
    event.synchronize()
    return fn(*args)


def compute_eigendecomposition(covariance_path: str, total_processed) -> dict[str, Tensor]:
    """``eigh`` (fp64) of every factor in ``covariance_path`` divided by
    ``total_processed`` and symmetrised; writes ``eigen_<basename>/shard_<rank>`` and
    returns this rank's eigenvalue shards."""
    rank = dist.get_rank() if dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_initialized() else 1
    device = get_device(rank)
    total = torch.as_tensor(total_processed).to(device)

    with safe_open(os.path.join(covariance_path, "shard_0.safetensors"), framework="pt") as f:
        keys = list(f.keys())
        out_dtype = f.get_tensor(keys[0]).dtype
        dims = {k: f.get_slice(k).get_shape()[-1] for k in keys}

    vecs: dict[str, Tensor] = {}
    vals: dict[str, Tensor] = {}
    finite: dict[str, Tensor] = {}
    mine = fair_distribute_by_cost(dims, world)[rank]
    on_gpu = torch.device(device).type == "cuda"
    # Every shard file is opened once and this rank's factors are read straight onto the device
    # (row order = rank order); results stay on the device until they are gathered and written.
    n_files = sum(f.endswith(".safetensors") for f in os.listdir(covariance_path))
    assert n_files == world, f"Expected {world} shards, found {n_files} in {covariance_path}"
    out_dir = os.path.join(os.path.dirname(covariance_path), "eigen_" + os.path.basename(covariance_path))
    os.makedirs(out_dir, exist_ok=True)
    layout = {k: ((shard_bounds(m, rank, world)[1] - shard_bounds(m, rank, world)[0], m), out_dtype)
              for k, m in dims.items()}
    writer = StreamedSafetensors(os.path.join(out_dir, f"shard_{rank}.safetensors"), layout)
    parts: dict[str, list[Tensor]] = {k: [] for k in mine}
    for r in range(world):
        with safe_open(os.path.join(covariance_path, f"shard_{r}.safetensors"), framework="pt", device=str(device)) as f:
            for key in mine:
                parts[key].append(f.get_tensor(key))

    def decompose(key: str, stream) -> None:
        ctx = torch.cuda.stream(stream) if stream is not None else nullcontext()
        with ctx:
            rows = parts.pop(key)
            m = (rows[0] if len(rows) == 1 else torch.cat(rows, dim=0)).to(torch.float64) / total
            m = (m + m.T) / 2
            finite[key] = torch.isfinite(m).all()  # read once, after all factors are queued
            try:
                w, q = torch.linalg.eigh(m)
            except Exception as e:
                if not bool(finite[key]):
                    raise ValueError(f"Covariance matrix for {key} contains NaNs or Infs. Consider using fp32.") from e
                raise RuntimeError(f"Eigendecomposition failed for {key}") from e
            q = q.to(out_dtype).contiguous()  # the solver returns column-major storage
            vals[key] = w.to(out_dtype)
            if world == 1:
                writer.write(key, q)  # copy to the host and file write overlap the other threads' solves
            else:
                vecs[key] = q

    try:
        if on_gpu and len(mine) > 1:
            # A dense symmetric eigensolver of a few thousand rows cannot fill the GPU on its own (long
            # chains of small kernels with host round trips in between): several factors are
            # decomposed at once, each on its own stream from its own host thread.
            from concurrent.futures import ThreadPoolExecutor

            workers = min(EIGH_CONCURRENCY, len(mine))
            # torch loads its dense linear-algebra backend lazily and not thread-safely: trigger that
            # from this thread before the workers start.
            torch.linalg.eigh(torch.eye(2, device=device, dtype=torch.float64))
            main = torch.cuda.current_stream()
            streams = [torch.cuda.Stream() for _ in range(workers)]
            for st in streams:
                st.wait_stream(main)

            import threading

            queue = iter(sorted(mine, key=lambda k: -dims[k]))  # largest first, taken as workers free up
            queue_lock = threading.Lock()

            def work(i: int) -> None:
                torch.cuda.set_device(torch.device(device))
                while True:
                    with queue_lock:
                        key = next(queue, None)
                    if key is None:
                        return
                    decompose(key, streams[i])

            with ThreadPoolExecutor(max_workers=workers) as pool:
                list(pool.map(work, range(workers)))
            for st in streams:
                main.wait_stream(st)
        else:
            for key in mine:
                decompose(key, None)
    except BaseException:
        writer.abort()
        raise

    try:
        bad = [k for k, ok in finite.items() if not bool(ok)]
        if bad:
            raise ValueError(f"Covariance matrix for {bad[0]} contains NaNs or Infs. Consider using fp32.")
        if world > 1:
            _gather_and_shard_along_dim_0(vecs, {k: (m, m) for k, m in dims.items()}, out_dtype, rank, world, device,
                                          sink=writer.write)
        vals = _gather_and_shard_along_dim_0(vals, {k: (m,) for k, m in dims.items()}, out_dtype, rank, world, device)
    except BaseException:
        writer.abort()
        raise
    writer.close()
    gc.collect()
    get_logger().info(f"Saved eigenvectors to {out_dir}")
    return vals


def save_uncorrected_eigenvalues(partial_run_path, eigenvalues_a, eigenvalues_g, total_processed, rank: int,
                                 world_size: int) -> None:
    """``eigenvalue_sharded`` = ``outer(l_G shard, l_A full) * T`` and the per-factor
    eigenvalues scaled by ``sqrt(T)`` (their product equals the grid)."""
    root = str(partial_run_path)
    dirs = {k: os.path.join(root, k) for k in ("eigenvalue_sharded", "factor_eig_a", "factor_eig_g")}
    for d in dirs.values():
        os.makedirs(d, exist_ok=True)
    device = get_device(rank)
    total = torch.as_tensor(total_processed).to(device)
    sc = ShardedMul()
    fa, fg = {}, {}
    a_full_by_key = {}
    for key in eigenvalues_g:
        a_shard = eigenvalues_a[key].to(device)
        if world_size > 1:
            m = torch.tensor(a_shard.shape[0], device=device)
            dist.all_reduce(m, op=dist.ReduceOp.SUM)
            a_shard = sc.gather_rows(a_shard, int(m.item()))
        a_full_by_key[key] = a_shard
    # The grids are the large output: each goes to its byte range of the file from a helper thread
    # while the next one is computed.
    from concurrent.futures import ThreadPoolExecutor

    layout = {k: ((g.shape[0], a_full_by_key[k].shape[0]), torch.result_type(g, a_full_by_key[k]))
              for k, g in eigenvalues_g.items()}
    writer = StreamedSafetensors(os.path.join(dirs["eigenvalue_sharded"], f"shard_{rank}.safetensors"), layout)
    try:
        with ThreadPoolExecutor(max_workers=2) as pool:
            jobs = []
            for key, g_shard in eigenvalues_g.items():
                g_shard = g_shard.to(device)
                a_full = a_full_by_key[key]
                grid = torch.outer(g_shard, a_full) * total.to(layout[key][1])
                if grid.is_cuda:
                    torch.cuda.current_stream().synchronize()  # the helper thread reads it from another stream
                jobs.append(pool.submit(writer.write, key, grid))
                scale = total.to(a_full.dtype).sqrt()
                fa[key] = (a_full * scale).cpu().contiguous()
                fg[key] = (g_shard * scale).cpu().contiguous()
            for job in jobs:
                job.result()
    except BaseException:
        writer.abort()
        raise
    writer.close()
    save_file(fa, os.path.join(dirs["factor_eig_a"], f"shard_{rank}.safetensors"))
    save_file(fg, os.path.join(dirs["factor_eig_g"], f"shard_{rank}.safetensors"))
    get_logger().info(f"Saved uncorrected eigenvalues to {dirs['eigenvalue_sharded']}")
