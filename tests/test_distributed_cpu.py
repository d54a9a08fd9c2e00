"""Two gloo ranks on CPU: same stores, factors and MAGIC scores as a single process; a rank
that fails makes the launcher raise."""

import numpy as np
import pytest
import torch

from bergson_b200.__main__ import main
from bergson_b200.data import load_gradients, load_scores
from bergson_b200.hessians.preconditioner import _load_full

MODEL = "native:llama-tiny?vocab_size=256"
TRAIN = "synthetic:zipf?n=24&len=16&vocab=256&seed=0&min_len=6"
QUERY = "synthetic:zipf?n=4&len=16&vocab=256&seed=1&min_len=8"


def run(*args):
    main([str(a) for a in args])


def test_build_two_ranks_equals_one(tmp_path):
    for n in (1, 2):
        run("build", tmp_path / f"w{n}", "--model", MODEL, "--data.dataset", TRAIN, "--projection_dim", "4",
            "--token_batch_size", "64", "--nproc_per_node", n)
    a, b = np.asarray(load_gradients(tmp_path / "w1")), np.asarray(load_gradients(tmp_path / "w2"))
    np.testing.assert_allclose(a, b, rtol=1e-4, atol=1e-6)
    assert int(torch.load(tmp_path / "w1" / "total_processed.pt")) == int(torch.load(tmp_path / "w2" / "total_processed.pt"))


def test_tensor_parallel_build_equals_single(tmp_path):
    opt = ["--model", MODEL, "--data.dataset", TRAIN, "--projection_dim", "4", "--token_batch_size", "64"]
    run("build", tmp_path / "tp1", *opt, "--nproc_per_node", 1)
    run("build", tmp_path / "tp2", *opt, "--nproc_per_node", 2, "--tensor_parallel", 2)
    a, b = np.asarray(load_gradients(tmp_path / "tp1")), np.asarray(load_gradients(tmp_path / "tp2"))
    np.testing.assert_allclose(a, b, rtol=1e-3, atol=1e-5 * np.abs(a).max())
    assert int(torch.load(tmp_path / "tp1" / "total_processed.pt")) == int(torch.load(tmp_path / "tp2" / "total_processed.pt"))


def test_ekfac_two_ranks_equals_one(tmp_path):
    for n in (1, 2):
        run("ekfac", tmp_path / f"e{n}", "--model", MODEL, "--index_cfg.data.dataset", TRAIN,
            "--hessian_pipeline_cfg.query.dataset", QUERY, "--method", "kfac", "--hessian_cfg.ev_correction", "true",
            "--use_dataset_labels", "--token_batch_size", "64", "--nproc_per_node", n)
    for sub in ("activation_sharded", "gradient_sharded", "eigenvalue_correction_sharded"):
        one = _load_full(tmp_path / "e1" / "hessian" / "kfac", sub, "cpu")
        two = _load_full(tmp_path / "e2" / "hessian" / "kfac", sub, "cpu")
        for k in one:
            assert (one[k] - two[k]).norm() / one[k].norm() < 1e-3, (sub, k)
    s1, s2 = load_scores(tmp_path / "e1" / "scores")[:], load_scores(tmp_path / "e2" / "scores")[:]
    assert np.corrcoef(s1.ravel(), s2.ravel())[0, 1] > 0.999


@pytest.mark.parametrize("fsdp", ["false", "true"])
def test_magic_two_ranks_equals_one(tmp_path, fsdp):
    for n in (1, 2):
        run("magic", tmp_path / f"m{n}", "--fsdp", fsdp, "--model", MODEL, "--data.dataset", "synthetic:zipf?n=16&len=12&vocab=256",
            "--query.dataset", "synthetic:zipf?n=4&len=12&vocab=256&seed=1", "--batch_size", "4", "--query_method", "mean",
            "--lr", "1e-3", "--nproc_per_node", n)
    a, b = load_scores(tmp_path / "m1" / "scores")[:], load_scores(tmp_path / "m2" / "scores")[:]
    # equal-length rows: the per-rank token means that DDP averages equal the global mean
    np.testing.assert_allclose(a, b, rtol=1e-3, atol=1e-4 * np.abs(a).max())


def _boom(rank, local_rank, world):
    from bergson_b200.distributed import init_dist

    init_dist(rank, local_rank, world)
    if rank == 1:
        raise RuntimeError("injected failure")


def test_failed_rank_raises_in_parent():
    from bergson_b200.config import DistributedConfig
    from bergson_b200.distributed import launch_distributed_run

    with pytest.raises(RuntimeError, match="child exited"):
        launch_distributed_run("boom", _boom, [], DistributedConfig(nproc_per_node=2))


def _exchange(rank, local_rank, world, out_dir):
    """Each rank holds a batch of its own size; module Grams end up on their owners only."""
    import torch.distributed as dist

    from bergson_b200.collector.dist_autocorrelation_gradient_collector import (
        assign_modules, exchange_hessian_gradients)
    from bergson_b200.distributed import init_dist

    init_dist(rank, local_rank, world)
    names = ["a", "b", "c"]
    widths = {"a": 3, "b": 5, "c": 2}
    owner = assign_modules(names, world)
    hessians: dict = {}
    for step in range(2):
        g = torch.Generator().manual_seed(10 * step + rank)
        rows = 2 + rank + step  # batch sizes differ between ranks and steps
        grads = {n: torch.randn(rows, widths[n], generator=g) for n in names}
        exchange_hessian_gradients(grads, hessians, owner, {n for n in names if owner[n] == rank}, rank)
    torch.save({"owner": owner, "hessians": hessians}, f"{out_dir}/rank{rank}.pt")
    dist.barrier()


def test_distributed_autocorrelation_exchange_two_ranks(tmp_path):
    from bergson_b200.config import DistributedConfig
    from bergson_b200.distributed import launch_distributed_run

    launch_distributed_run("exchange", _exchange, [str(tmp_path)], DistributedConfig(nproc_per_node=2))
    widths = {"a": 3, "b": 5, "c": 2}
    want = {n: torch.zeros(w, w) for n, w in widths.items()}
    for step in range(2):
        for rank in range(2):
            g = torch.Generator().manual_seed(10 * step + rank)
            rows = 2 + rank + step
            for n in ("a", "b", "c"):
                p = torch.randn(rows, widths[n], generator=g)
                want[n] += p.T @ p
    got = [torch.load(tmp_path / f"rank{r}.pt") for r in range(2)]
    owner = got[0]["owner"]
    assert owner == {"a": 0, "b": 0, "c": 1}  # contiguous blocks, the first rank takes the extra module
    for n, r in owner.items():
        torch.testing.assert_close(got[r]["hessians"][n], want[n], rtol=1e-5, atol=1e-5)
        assert n not in got[1 - r]["hessians"]


def test_fsdp2_build_two_ranks_equals_one(tmp_path):
    """`--fsdp true` wraps the layers with `fully_shard`; the store must not depend on it."""
    opt = ["--model", MODEL, "--data.dataset", TRAIN, "--projection_dim", "4", "--token_batch_size", "64"]
    run("build", tmp_path / "plain", *opt, "--nproc_per_node", 1)
    run("build", tmp_path / "fsdp", *opt, "--nproc_per_node", 2, "--fsdp", "true")
    a, b = np.asarray(load_gradients(tmp_path / "plain")), np.asarray(load_gradients(tmp_path / "fsdp"))
    np.testing.assert_allclose(a, b, rtol=1e-4, atol=1e-6)


def _prefetch_worker(rank, local_rank, world, out_dir):
    """Sharded parameters gathered per module, with and without requesting the next module's
    parameters ahead of time: same loss, same sharded gradients, same second-order gradients."""
    import torch.distributed as dist

    from bergson_b200.distributed import init_dist
    from bergson_b200.magic.fsdp import LazyGather, simple_fsdp

    from .helpers import tiny_model

    init_dist(rank, local_rank, world)
    torch.manual_seed(0)  # the same full model on every rank
    model = tiny_model("llama", dtype=torch.float64, num_hidden_layers=2)
    model.eval()
    full = {k: v.detach().clone() for k, v in model.named_parameters()}
    shards, shapes = simple_fsdp(full)
    shards = {k: v.requires_grad_(True) for k, v in shards.items()}
    x = torch.randint(0, 128, (2, 9), generator=torch.Generator().manual_seed(rank))

    def run(prefetch):
        with LazyGather(model, shards, shapes, prefetch=prefetch) as lazy:
            loss = model(input_ids=x, labels=x).loss
        ps = list(shards.values())
        g = torch.autograd.grad(loss, ps, create_graph=True, allow_unused=True)
        inner = sum((t * t).sum() for t in g if t is not None)
        gg = torch.autograd.grad(inner, ps, allow_unused=True)
        return loss.detach(), g, gg, lazy

    base = run(False)
    first = run(True)   # learns the call order, nothing to request yet
    second = run(True)  # requests each next module while the current one runs
    assert first[3].prefetch_hits == 0 and second[3].prefetch_hits > 0
    assert second[3].gathers == base[3].gathers
    for got in (first, second):
        torch.testing.assert_close(got[0], base[0], rtol=0, atol=0)
        for a, b in zip(got[1] + got[2], base[1] + base[2]):
            if b is None:
                assert a is None
            else:
                torch.testing.assert_close(a, b, rtol=1e-12, atol=1e-14)
    assert all(isinstance(p, torch.nn.Parameter) for p in model.parameters())
    torch.save({"hits": second[3].prefetch_hits, "gathers": second[3].gathers}, f"{out_dir}/rank{rank}.pt")
    dist.barrier()


def test_lazy_gather_prefetch_two_ranks(tmp_path):
    from bergson_b200.config import DistributedConfig
    from bergson_b200.distributed import launch_distributed_run

    launch_distributed_run("prefetch", _prefetch_worker, [str(tmp_path)], DistributedConfig(nproc_per_node=2))
    got = [torch.load(tmp_path / f"rank{r}.pt") for r in range(2)]
    assert got[0] == got[1] and got[0]["hits"] > 5


def test_optimizer_moments_are_saved_whole_under_sharding(tmp_path):
    """With row-sharded parameters the second moments are sharded too; the exported
    ``optimizer.pt`` must hold them at full shape, equal to the unsharded run's."""
    common = ["--model", MODEL, "--data.dataset", "synthetic:zipf?n=16&len=12&vocab=256&seed=0&min_len=12", "--batch_size", "4",
              "--lr", "1e-3", "--save_mode", "all", "--save_optimizer_state", "last"]
    run("train", tmp_path / "one", *common, "--nproc_per_node", 1)
    run("train", tmp_path / "two", *common, "--nproc_per_node", 2, "--fsdp", "true")
    found = {}
    for name in ("one", "two"):
        found[name] = torch.load(tmp_path / name / "optimizer.pt", weights_only=False)  # the final state's moments
    a, b = found["one"]["state"], found["two"]["state"]
    assert a.keys() == b.keys() and len(a) > 0
    for k in a:
        assert a[k]["param_name"] == b[k]["param_name"]
        assert a[k]["exp_avg_sq"].shape == b[k]["exp_avg_sq"].shape
        torch.testing.assert_close(a[k]["exp_avg_sq"], b[k]["exp_avg_sq"], rtol=2e-3, atol=1e-10)
