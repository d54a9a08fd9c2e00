"""Process launch and small distributed helpers.

One process per GPU.  ``launch_distributed_run`` spawns ``nproc_per_node`` children
with ``CUDA_VISIBLE_DEVICES`` pinned per child before the interpreter starts, a free
rendezvous port, and ``RANK/LOCAL_RANK/WORLD_SIZE/MASTER_*`` set; it raises if a child
exits non-zero (reference ``bergson/distributed.py:119-200``).  When the process was
already started by ``torchrun`` (``RANK`` and ``WORLD_SIZE`` in the environment and
``BERGSON_B200_EXTERNAL_LAUNCH=1``), the worker runs in-process instead.
"""

from __future__ import annotations

import io
import os
import socket
from contextlib import nullcontext, redirect_stdout
from copy import deepcopy
from datetime import timedelta
from typing import Any, Callable, Mapping

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from .config.config import DistributedConfig
from .utils.utils import dist_backend, dist_device_id, get_device_index


def init_dist(rank: int, local_rank: int, world_size: int, *, mixed: bool = False,
              timeout: timedelta = timedelta(hours=1)) -> None:
    """Pin the CUDA device and join the process group named by MASTER_ADDR/PORT."""
    if torch.cuda.is_available():
        torch.cuda.set_device(get_device_index(local_rank))
    if world_size > 1 and not dist.is_initialized():
        addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
        port = os.environ.get("MASTER_PORT", "29500")
        dist.init_process_group(
            dist_backend(mixed),
            init_method=f"tcp://{addr}:{port}",
            device_id=dist_device_id(local_rank),
            rank=rank,
            timeout=timeout,
            world_size=world_size,
        )


def cap_world_size_to_dataset(cfg: DistributedConfig, dataset_size: int) -> DistributedConfig:
    """Single-node config with at most one rank per document."""
    if dataset_size >= cfg.world_size:
        return cfg
    out = deepcopy(cfg)
    out.nnode = 1
    out.nproc_per_node = max(1, min(dataset_size, cfg.nproc_per_node))
    return out


def parent_barrier(dist_config: DistributedConfig) -> None:
    """Barrier over the per-node parent processes (Gloo on MASTER_PORT + 1)."""
    if dist_config.nnode <= 1:
        return
    addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
    port = int(os.environ.get("MASTER_PORT", "29500")) + 1
    dist.init_process_group("gloo", init_method=f"tcp://{addr}:{port}", rank=dist_config._node_rank,
                            world_size=dist_config.nnode)
    dist.barrier()
    dist.destroy_process_group()


def grad_tree(outputs: torch.Tensor, inputs: Mapping[str, torch.Tensor], grad_outputs: dict | None = None, **kwargs):
    """``autograd.grad`` over a dict of inputs, returning a dict with the same keys."""
    if grad_outputs is not None:
        kwargs["grad_outputs"] = list(grad_outputs.values())
    grads = torch.autograd.grad(outputs, list(inputs.values()), **kwargs, allow_unused=True)
    return dict(zip(inputs, grads))


def find_free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def dist_worker(worker: Callable, rank: int, local_rank: int, world_size: int, master_addr: str, master_port: str,
                *worker_args):
    os.environ.update(LOCAL_RANK=str(local_rank), RANK=str(rank), WORLD_SIZE=str(world_size),
                      MASTER_ADDR=master_addr, MASTER_PORT=master_port)
    # Hang diagnosis: BERGSON_B200_DUMP_AFTER=<seconds> prints every thread's stack to stderr
    # that long after the worker started (and keeps running).
    if os.environ.get("BERGSON_B200_DUMP_AFTER"):
        import faulthandler
        import sys

        faulthandler.dump_traceback_later(float(os.environ["BERGSON_B200_DUMP_AFTER"]), repeat=False, file=sys.stderr)
    try:
        with nullcontext() if rank == 0 else redirect_stdout(io.StringIO()):
            worker(rank, local_rank, world_size, *worker_args)
    finally:
        if dist.is_initialized():
            try:
                dist.barrier()
            except Exception as e:  # a peer that died must not mask the original error
                print(f"Barrier failed during cleanup: {e}")
            dist.destroy_process_group()


def launch_distributed_run(process_name: str, worker, const_worker_args: list[Any],
                           dist_config: DistributedConfig | None = None):
    dist_config = dist_config or DistributedConfig()
    local_world = dist_config.nproc_per_node
    world = dist_config.world_size
    start_rank = dist_config.start_rank

    if os.environ.get("BERGSON_B200_EXTERNAL_LAUNCH") == "1" and "RANK" in os.environ:
        # Started by torchrun: this process *is* one rank.
        rank, lrank, ws = int(os.environ["RANK"]), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ["WORLD_SIZE"])
        dist_worker(worker, rank, lrank, ws, os.environ.get("MASTER_ADDR", "127.0.0.1"),
                    os.environ.get("MASTER_PORT", "29500"), *const_worker_args)
        return

    if world <= 1:
        if dist_config._node_rank == 0:
            worker(0, 0, 1, *const_worker_args)
        return

    mp.set_sharing_strategy("file_system")
    parent_cvd = os.environ.get("CUDA_VISIBLE_DEVICES")
    devices = [d.strip() for d in parent_cvd.split(",") if d.strip()] if parent_cvd else [str(j) for j in range(local_world)]
    if torch.cuda.is_available():
        assert len(devices) >= local_world, (
            f"CUDA_VISIBLE_DEVICES has {len(devices)} entries ({parent_cvd!r}) but nproc_per_node={local_world}"
        )
    # Every rank keeps all of the node's GPUs visible and selects its own by index: kernels that
    # read or add into other ranks' memory over NVLink (symmetric peer heaps) need the peers'
    # devices to be addressable.  BERGSON_B200_PIN_VISIBLE_DEVICES=1 restores one visible GPU per
    # child, at the price of the peer-memory paths.
    pin = os.environ.get("BERGSON_B200_PIN_VISIBLE_DEVICES") == "1"
    if dist_config.nnode > 1:
        master_addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
        master_port = os.environ.get("MASTER_PORT", "29500")
    else:
        master_addr, master_port = "127.0.0.1", str(find_free_port())

    ctx = mp.get_context("spawn")
    children = []
    try:
        for i in range(local_world):
            if torch.cuda.is_available() and pin:
                # Inherited through exec, before the child imports torch.
                os.environ["CUDA_VISIBLE_DEVICES"] = devices[i]
            p = ctx.Process(target=dist_worker,
                            args=(worker, start_rank + i, i, world, master_addr, master_port, *const_worker_args))
            p.start()
            children.append(p)
    finally:
        if parent_cvd is None:
            os.environ.pop("CUDA_VISIBLE_DEVICES", None)
        else:
            os.environ["CUDA_VISIBLE_DEVICES"] = parent_cvd

    failed = None
    for p in children:
        p.join()
        if p.exitcode != 0 and failed is None:
            failed = p.exitcode
    if failed is not None:
        raise RuntimeError(f"{process_name} child exited with code {failed}")


def simple_dist_worker(rank: int, local_rank: int, world_size: int, dataset, worker) -> None:
    """One rank of ``dist_main``: join the process group, then ``worker(rank, world_size, dataset)``
    (the launcher tears the group down afterwards)."""
    init_dist(rank, local_rank, world_size)
    worker(rank, world_size, dataset)


def dist_main(dataset, worker, nproc: int | None = None) -> None:
    """Run ``worker(rank, world_size, dataset)`` once per visible GPU (``nproc`` overrides the
    count); a single device runs it in this process, which keeps a debugger attached
    (reference ``bergson/distributed.py:215-250``).  ``worker`` must be importable by the
    spawned children (a module-level function)."""
    world = nproc if nproc is not None else torch.cuda.device_count()
    if world <= 1:
        worker(0, 1, dataset)
        return
    launch_distributed_run("dist_main", simple_dist_worker, [dataset, worker], DistributedConfig(nproc_per_node=world))
