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


@pytest.mark.parametrize("data, token_batch, fused", [
    ("synthetic:zipf?n=16&len=160&vocab=1024&min_len=90", "640", False),   # ragged: all-reduce path
    ("synthetic:zipf?n=32&len=128&vocab=1024&min_len=128", "1024", True),  # 8 x 128 tokens: sequence-parallel
])
def test_tensor_parallel_fused_build_matches_single_gpu(tmp_path, data, token_batch, fused):
    """CLI build on 1 GPU vs tensor-parallel over 2 GPUs (fused projection kernels, bf16).  With
    token counts that split into 128-row blocks per rank the blocks run sequence-parallel with
    the all-gather and the reduce-scatter inside the GEMM kernels."""
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
            "--data.dataset", data, "--projection_dim", "16",
            "--token_batch_size", token_batch, "--store_dtype", "fp32"]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    for name, extra in (("one", ["--nproc_per_node", "1"]), ("tp2", ["--nproc_per_node", "2", "--tensor_parallel", "2"])):
        out = subprocess.run(common + [str(tmp_path / name)] + opts + extra, cwd=root, env=env, capture_output=True,
                             text=True, timeout=600)
        assert out.returncode == 0, out.stderr[-2000:]
        if name == "tp2":
            assert ("sequence-parallel blocks over 2 ranks" in out.stdout + out.stderr) == fused
    a, b = np.asarray(load_gradients(tmp_path / "one")), np.asarray(load_gradients(tmp_path / "tp2"))
    assert np.abs(b).max() > 0
    assert np.abs(a - b).max() / np.abs(a).max() < 3e-2


def test_score_with_sharded_queries_matches_single_gpu(tmp_path):
    """`score` on 2 GPUs keeps the query rows sharded in peer memory and reads them inside the
    score GEMM (fused all-gather); the scores must equal the 1-GPU run with replicated queries."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import subprocess
    import sys
    from pathlib import Path

    import numpy as np

    from bergson_b200.data import load_scores

    root = Path(__file__).resolve().parents[1]
    model = ["--model", "native:llama-tiny?hidden_size=128&intermediate_size=256&vocab_size=1024&max_position_embeddings=1024",
             "--index_cfg.precision", "bf16", "--projection_dim", "16", "--token_batch_size", "640"]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")

    def cli(*args):
        out = subprocess.run([sys.executable, "-m", "bergson_b200", *map(str, args)], cwd=root, env=env,
                             capture_output=True, text=True, timeout=600)
        assert out.returncode == 0, out.stderr[-2000:]
        return out

    build_model = [m if m != "--index_cfg.precision" else "--precision" for m in model]
    model = model + ["--score_cfg.precision", "bf16"]  # the fused gather needs 16-bit scoring (default: fp32)
    cli("build", tmp_path / "query", "--data.dataset", "synthetic:zipf?n=13&len=160&vocab=1024&seed=1&min_len=90",
        *build_model, "--nproc_per_node", "1")
    data = ["--data.dataset", "synthetic:zipf?n=24&len=160&vocab=1024&seed=0&min_len=90"]
    for name, n in (("one", 1), ("two", 2)):
        out = cli("score", tmp_path / name, *data, *model, "--query_path", tmp_path / "query", "--nproc_per_node", n)
        assert ("all-gather fused into the score GEMM" in out.stdout) == (n == 2), out.stdout[-500:]
    a, b = load_scores(tmp_path / "one")[:].astype(np.float32), load_scores(tmp_path / "two")[:].astype(np.float32)
    assert a.shape == b.shape == (24, 13) and np.abs(a).max() > 0
    assert np.abs(a - b).max() / np.abs(a).max() < 2e-2
    # and with cosine scoring in slices of 5 queries (uneven shards: 3 + 2 rows per slice)
    for name, n in (("one_c", 1), ("two_c", 2)):
        cli("score", tmp_path / name, *data, *model, "--query_path", tmp_path / "query", "--nproc_per_node", n,
            "--unit_normalize", "--query_batch_size", "5")
    a, b = load_scores(tmp_path / "one_c")[:].astype(np.float32), load_scores(tmp_path / "two_c")[:].astype(np.float32)
    assert np.abs(a - b).max() < 2e-2 and np.abs(a).max() <= 1.0 + 1e-2


def _sharded_query_worker(rank, world, port, store, out):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from bergson_b200 import Attributor

        attr = Attributor(store, device=f"cuda:{rank}", dtype=torch.float16, unit_norm=True, sharded=True)
        torch.manual_seed(5)
        q = torch.randn(9, 512, device=f"cuda:{rank}")
        queries = {"m0": q[:, :256].contiguous(), "m1": q[:, 256:].contiguous()}
        s, i = attr.search(queries, k=11)
        out.put((rank, s.float().cpu(), i.cpu()))
    finally:
        dist.barrier()
        dist.destroy_process_group()


def test_sharded_attributor_two_gpus(tmp_path):
    """Store rows split over 2 GPUs, per-rank top-k on the tcgen05 GEMM, merged across ranks."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import numpy as np
    import torch.multiprocessing as mp

    from bergson_b200 import Attributor
    from bergson_b200.data import create_index
    from bergson_b200.gradients import GradientProcessor

    store = tmp_path / "store"
    store.mkdir()
    mm = create_index(store, 700, {"m0": 256, "m1": 256}, np.float16)
    mm[:] = np.random.default_rng(0).standard_normal(mm.shape).astype(np.float16)
    mm.flush()
    GradientProcessor(projection_dim=16).save(store)
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_sharded_query_worker, args=(r, 2, port, str(store), out)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted([out.get(timeout=300) for _ in range(2)], key=lambda r: r[0])
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    ref = Attributor(store, device="cuda:0", dtype=torch.float16, unit_norm=True)
    torch.manual_seed(5)
    q = torch.randn(9, 512, device="cuda:0")
    s_ref, i_ref = ref.search({"m0": q[:, :256].contiguous(), "m1": q[:, 256:].contiguous()}, k=11)
    for _, s, i in results:
        torch.testing.assert_close(s, s_ref.float().cpu(), atol=2e-3, rtol=1e-2)
        assert (i == i_ref.cpu()).float().mean() > 0.95  # near-ties may swap under fp16 rounding


def test_kfac_factors_two_gpus_match_one(tmp_path):
    """K-FAC covariances on 2 GPUs: the last batch's SYRK launch folds the local accumulators in
    and adds the rows into their owners' peer memory (GEMM -> reduce-scatter); the assembled
    factors must equal the 1-GPU factors."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import subprocess
    import sys
    from pathlib import Path

    from bergson_b200.hessians.preconditioner import _load_full

    root = Path(__file__).resolve().parents[1]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    opts = ["--model", "native:llama-tiny?hidden_size=128&intermediate_size=256&vocab_size=1024&max_position_embeddings=1024",
            "--precision", "bf16", "--index_cfg.data.dataset", "synthetic:zipf?n=24&len=160&vocab=1024&seed=0&min_len=90",
            "--method", "kfac", "--use_dataset_labels", "--token_batch_size", "640"]
    for name, n in (("one", 1), ("two", 2)):
        out = subprocess.run([sys.executable, "-m", "bergson_b200", "hessian", str(tmp_path / name), *opts,
                              "--nproc_per_node", str(n)], cwd=root, env=env, capture_output=True, text=True, timeout=600)
        assert out.returncode == 0, out.stderr[-2000:]
        if n == 2:
            assert "inside the last batch's SYRK launches" in out.stdout + out.stderr
            assert "reduced through peer memory: 0 inside" not in out.stdout + out.stderr
    for sub in ("activation_sharded", "gradient_sharded"):
        one = _load_full(tmp_path / "one", sub, "cpu")
        two = _load_full(tmp_path / "two", sub, "cpu")
        assert one.keys() == two.keys() and len(one) > 0
        for k in one:
            assert one[k].shape == two[k].shape
            assert float((one[k] - two[k]).norm() / one[k].norm()) < 2e-3, (sub, k)
            assert float((two[k] - two[k].T).abs().max() / two[k].abs().max()) < 1e-5, (sub, k, "not symmetric")
    # The eigendecomposition that follows (factors split over the ranks, shards streamed to the
    # files): the assembled eigenvalue grids and orthonormal eigenvector shards.
    one, two = (_load_full(tmp_path / n, "eigenvalue_sharded", "cpu") for n in ("one", "two"))
    assert one.keys() == two.keys() and len(one) > 0
    for k in one:
        assert float((one[k] - two[k]).norm() / one[k].norm()) < 1e-2, ("eigenvalue_sharded", k)
    for sub in ("eigen_activation_sharded", "eigen_gradient_sharded"):
        for k, q in _load_full(tmp_path / "two", sub, "cpu").items():
            eye = torch.eye(q.shape[0])
            assert float((q.float().T @ q.float() - eye).abs().max()) < 1e-3, (sub, k)


def _seq_parallel_worker(rank, world, port, out):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from bergson_b200.ops import Linear, native
        from bergson_b200.parallel.sequence_parallel import Published, SeqParallel, gather_linear, scatter_linear

        sp = SeqParallel(dist.group.WORLD)
        assert sp.available()
        T, D, N_local, lead = 1024, 256, 192, (4, 256)
        rows = T // world
        sp.ensure(T, D, torch.bfloat16)
        torch.manual_seed(7 + rank)
        col = Linear(D, N_local, bias=False, device="cuda", dtype=torch.bfloat16).requires_grad_(False)
        row = Linear(N_local, D, bias=False, device="cuda", dtype=torch.bfloat16).requires_grad_(False)
        errs = []
        for step in range(3):  # several rounds: the double-buffered regions get reused
            shard = torch.randn(rows, D, device="cuda").to(torch.bfloat16).requires_grad_(True)
            y = gather_linear(Published(sp, shard), col, lead)           # [T, N_local]
            z = scatter_linear(torch.tanh(y), row, sp, lead, residual=shard)  # [rows, D]
            cot = torch.randn(rows, D, device="cuda").to(torch.bfloat16)
            (dx,) = torch.autograd.grad(z, shard, cot)
            # Reference with NCCL collectives and fp32 math.
            shards = [torch.empty_like(shard) for _ in range(world)]
            dist.all_gather(shards, shard.detach())
            x_full = torch.cat(shards).float().requires_grad_(True)
            y_ref = x_full @ col.weight.float().T
            part = torch.tanh(y_ref.to(torch.bfloat16).float()) @ row.weight.float().T
            cots = [torch.empty_like(cot) for _ in range(world)]
            dist.all_gather(cots, cot)
            (dx_part,) = torch.autograd.grad(part, x_full, torch.cat(cots).float())
            summed = part.detach().clone()
            dist.all_reduce(summed)
            dist.all_reduce(dx_part)
            z_ref = summed[rank * rows : (rank + 1) * rows] + shard.detach().float()
            dx_ref = dx_part[rank * rows : (rank + 1) * rows] + cot.float()
            errs.append(float((y.float() - y_ref.detach()).abs().max() / y_ref.abs().max()))
            errs.append(float((z.float() - z_ref).abs().max() / z_ref.abs().max()))
            errs.append(float((dx.float() - dx_ref).abs().max() / dx_ref.abs().max()))
        torch.cuda.synchronize()
        out.put((rank, max(errs), int(native.kernel_status(rank).item()), sp.barriers, sp.fused_gemms))
    finally:
        dist.barrier()
        dist.destroy_process_group()


def test_sequence_parallel_projections_two_gpus():
    """All-gather -> GEMM and GEMM -> reduce-scatter (forward and backward) against NCCL
    collectives around fp32 products."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_seq_parallel_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0, f"rank exited with {p.exitcode}"
    for rank, err, status, barriers, gemms in sorted(out.get(timeout=10) for _ in range(2)):
        assert status == 0
        assert err < 3e-2, (rank, err)
        assert barriers == 3 * 4 and gemms == 3 * 4  # publish, reduce, publish (bwd), reduce (bwd) per round


def test_magic_fsdp_matches_ddp_two_gpus(tmp_path):
    """`magic` on 2 GPUs with sharded parameters (gathered per module over NCCL, gathered again
    in the backward and the double-backward pass) against plain data parallelism."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import subprocess
    import sys
    from pathlib import Path

    import numpy as np

    from bergson_b200.data import load_scores

    root = Path(__file__).resolve().parents[1]
    opts = ["--model", "native:gpt2-tiny?vocab_size=256", "--precision", "fp32",
            "--data.dataset", "synthetic:zipf?n=16&len=16&vocab=256&min_len=16",
            "--query.dataset", "synthetic:zipf?n=4&len=16&vocab=256&seed=1&min_len=16", "--batch_size", "4",
            "--query_method", "mean", "--lr", "1e-3", "--max_grad_norm", "1.0", "--nproc_per_node", "2"]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    for name, fsdp in (("ddp", "false"), ("fsdp", "true")):
        out = subprocess.run([sys.executable, "-m", "bergson_b200", "magic", str(tmp_path / name), "--fsdp", fsdp] + opts,
                             cwd=root, env=env, capture_output=True, text=True, timeout=900)
        assert out.returncode == 0, out.stderr[-2000:]
    a, b = load_scores(tmp_path / "ddp" / "scores")[:], load_scores(tmp_path / "fsdp" / "scores")[:]
    assert np.abs(a).max() > 0
    np.testing.assert_allclose(a, b, rtol=2e-3, atol=2e-4 * np.abs(a).max())
