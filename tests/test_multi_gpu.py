"""Fused compute+collective kernels over peer memory on 2 GPUs, against NCCL compositions.
Ranks are child processes; every kernel is wait-free (host barriers order the ranks)."""

import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from bergson_b200.ops import native
        from bergson_b200.parallel import PeerHeap, gathered_scores, reduce_scatter_gram

        torch.manual_seed(100 + rank)
        D, T, K, NQ, B = 520, 3000, 1024, 256, 300
        heap = PeerHeap(max(D * D, NQ * K), torch.float32)
        # --- GEMM -> reduce-scatter ------------------------------------------------------
        x = torch.randn(T, D, device="cuda", dtype=torch.bfloat16)
        local = torch.randn(D, D, device="cuda")
        local = local + local.T
        heap.local.zero_()
        heap.barrier()
        shard = reduce_scatter_gram(local, heap, 0, x_last=x).clone()
        full = local + x.float().T @ x.float()
        dist.all_reduce(full)
        base, rem = divmod(D, world)
        lo = 0 if rank == 0 else rem + rank * base
        hi = lo + base + (rem if rank == 0 else 0)
        err_rs = float((shard - full[lo:hi]).abs().max() / full.abs().max())
        heap.barrier()
        # --- all-gather -> GEMM ----------------------------------------------------------
        q_heap = PeerHeap(NQ * K, torch.bfloat16)
        q = torch.randn(NQ, K, device="cuda", dtype=torch.bfloat16)
        q_heap.local.copy_(q.flatten())
        q_heap.barrier()
        rows = torch.randn(B, K, device="cuda", dtype=torch.bfloat16)
        scores = gathered_scores(rows, q_heap, 0, NQ)
        gathered = [torch.empty_like(q) for _ in range(world)]
        dist.all_gather(gathered, q)
        ref = rows.float() @ torch.cat(gathered).float().T
        err_ag = float((scores - ref).abs().max() / ref.abs().max())
        torch.cuda.synchronize()
        status = int(native.kernel_status(rank).item())
        q_heap.barrier()
        out.put((rank, err_rs, err_ag, status))
    finally:
        dist.barrier()
        dist.destroy_process_group()


def test_fused_collectives_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0, f"rank exited with {p.exitcode}"
    results = sorted(out.get(timeout=10) for _ in range(2))
    for rank, err_rs, err_ag, status in results:
        assert status == 0
        assert err_rs < 2e-3, (rank, err_rs)
        assert err_ag < 2e-2, (rank, err_ag)


def test_tensor_parallel_fused_build_matches_single_gpu(tmp_path):
    """CLI build on 1 GPU vs tensor-parallel over 2 GPUs (fused projection kernels, bf16)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import subprocess
    import sys
    from pathlib import Path

    import numpy as np

    from bergson_b200.data import load_gradients

    root = Path(__file__).resolve().parents[1]
    common = [sys.executable, "-m", "bergson_b200", "build"]
    opts = ["--model", "native:llama-tiny?hidden_size=128&intermediate_size=256&vocab_size=1024&max_position_embeddings=1024", "--precision", "bf16",
            "--data.dataset", "synthetic:zipf?n=16&len=160&vocab=1024&min_len=90", "--projection_dim", "16",
            "--token_batch_size", "640", "--store_dtype", "fp32"]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    for name, extra in (("one", ["--nproc_per_node", "1"]), ("tp2", ["--nproc_per_node", "2", "--tensor_parallel", "2"])):
        out = subprocess.run(common + [str(tmp_path / name)] + opts + extra, cwd=root, env=env, capture_output=True,
                             text=True, timeout=600)
        assert out.returncode == 0, out.stderr[-2000:]
    a, b = np.asarray(load_gradients(tmp_path / "one")), np.asarray(load_gradients(tmp_path / "tp2"))
    assert np.abs(b).max() > 0
    assert np.abs(a - b).max() / np.abs(a).max() < 3e-2
