"""Inversion math, preconditioners, Kronecker-factor collectors against dense references,
row-sharded algebra under 2 gloo ranks."""

import os
import socket

import pytest
import torch
from safetensors.torch import load_file, save_file

from bergson_b200.config import HessianConfig, InversionConfig
from bergson_b200.gradients import GradientProcessor
from bergson_b200.hessians.eigenvectors import compute_eigendecomposition, fair_distribute_by_cost, save_uncorrected_eigenvalues
from bergson_b200.hessians.inversion import eigenvalue_multiplier, invert_psd_matrix
from bergson_b200.hessians.preconditioner import DensePreconditioner, FactoredPreconditioner, load_preconditioner
from bergson_b200.hessians.sharded_computation import shard_bounds
from bergson_b200.utils.math import compute_lambda, weighted_causal_lm_ce


def test_eigenvalue_functions():
    lam = torch.tensor([0.0, 1.0, 3.0])
    mean = lam.mean()
    torch.testing.assert_close(eigenvalue_multiplier("damped_inverse", lam, mean, 0.3), 1 / (lam + 0.4))
    torch.testing.assert_close(eigenvalue_multiplier("tikhonov_filtered", lam, mean, 0.3), lam / (lam**2 + 0.16))
    torch.testing.assert_close(eigenvalue_multiplier("pseudoinverse", lam, mean, 0.3), torch.tensor([0.0, 1.0, 1 / 3]))
    half = eigenvalue_multiplier("damped_inverse", lam, mean, 0.3, power=-0.5)
    torch.testing.assert_close(half * half, 1 / (lam + 0.4))
    grid = torch.outer(torch.tensor([1.0, 2.0]), torch.tensor([1.0, 3.0, 5.0]))
    ft = eigenvalue_multiplier("factored_tikhonov", grid, grid.mean(), 0.1, factor_a=torch.tensor([1.0, 3.0, 5.0]),
                               factor_g=torch.tensor([1.0, 2.0]), mean_a=torch.tensor(3.0), mean_g=torch.tensor(1.5))
    gamma = 0.1 * grid.mean()
    pi = (torch.tensor(3.0) / 1.5).sqrt()
    expect = 1 / (grid + pi * gamma.sqrt() * torch.tensor([1.0, 2.0])[:, None]
                  + gamma.sqrt() / pi * torch.tensor([1.0, 3.0, 5.0])[None] + gamma)
    torch.testing.assert_close(ft, expect)


def test_invert_psd_matrix():
    torch.manual_seed(0)
    a = torch.randn(6, 6, dtype=torch.float64)
    H = a @ a.T
    inv = invert_psd_matrix(H, damping_factor=0.0)
    torch.testing.assert_close(inv @ H, torch.eye(6, dtype=torch.float64), atol=1e-8, rtol=1e-8)
    half = invert_psd_matrix(H, damping_factor=0.1, power=-0.5)
    torch.testing.assert_close(half @ half, invert_psd_matrix(H, damping_factor=0.1), atol=1e-10, rtol=1e-8)


def test_shard_bounds_and_cost_distribution():
    assert [shard_bounds(11, r, 3) for r in range(3)] == [(0, 5), (5, 8), (8, 11)]
    d = fair_distribute_by_cost({"a": 8, "b": 4, "c": 6, "d": 2}, 2)
    assert d == [["a", "d"], ["c", "b"]]


def _write_factors(path, o=3, i=4, ev=False):
    torch.manual_seed(1)
    A = torch.randn(20, i, dtype=torch.float64)
    G = torch.randn(20, o, dtype=torch.float64)
    la, qa = torch.linalg.eigh(A.T @ A / 20)
    lg, qg = torch.linalg.eigh(G.T @ G / 20)
    for sub, t in (("eigen_activation_sharded", qa), ("eigen_gradient_sharded", qg),
                   ("eigenvalue_sharded", torch.outer(lg, la)), ("factor_eig_a", la), ("factor_eig_g", lg)):
        os.makedirs(path / sub, exist_ok=True)
        save_file({"m": t.float().contiguous()}, str(path / sub / "shard_0.safetensors"))
    return qa, qg, la, lg


def test_factored_preconditioner_equals_dense_kronecker(tmp_path):
    qa, qg, la, lg = _write_factors(tmp_path)
    pre = load_preconditioner(tmp_path, inversion_cfg=InversionConfig(damping_factor=0.05))
    assert isinstance(pre, FactoredPreconditioner)
    g = torch.randn(5, 3 * 4)
    out = pre.apply({"m": g, "other": g})["m"].double()
    grid = torch.outer(lg, la)
    m = 1 / (grid + 0.05 * grid.mean())
    H_inv = torch.kron(qg, qa) @ torch.diag(m.flatten()) @ torch.kron(qg, qa).T  # vec is row-major over [O, I]
    torch.testing.assert_close(out, g.double() @ H_inv.T, atol=1e-4, rtol=1e-4)
    assert pre.apply({"other": g})["other"] is g
    ft = load_preconditioner(tmp_path, inversion_cfg=InversionConfig(inversion="factored_tikhonov"))
    assert torch.isfinite(ft.apply({"m": g})["m"]).all()
    custom = FactoredPreconditioner.from_path(tmp_path, apply_fn=lambda lam: torch.ones_like(lam))
    torch.testing.assert_close(custom.apply({"m": g})["m"], g, atol=1e-5, rtol=1e-5)


def test_dense_preconditioner(tmp_path):
    a = torch.randn(8, 8)
    H = a @ a.T
    GradientProcessor(hessians={"m": H}, projection_dim=2).save(tmp_path)
    pre = load_preconditioner(tmp_path, inversion_cfg=InversionConfig(damping_factor=0.1))
    assert isinstance(pre, DensePreconditioner)
    g = torch.randn(3, 8)
    torch.testing.assert_close(pre.apply({"m": g})["m"], g @ invert_psd_matrix(H, damping_factor=0.1), atol=1e-4, rtol=1e-4)


def test_kfac_factors_match_manual_covariances(tmp_path):
    from bergson_b200.config import IndexConfig
    from bergson_b200.data import allocate_batches, pad_and_tensor
    from bergson_b200.hessians.hessian_approximations import collect_hessians

    from .helpers import tiny_dataset, tiny_model

    torch.manual_seed(0)
    model = tiny_model("llama")
    model.requires_grad_(False)
    model.get_input_embeddings().requires_grad_(True)
    ds = tiny_dataset(n=6, length=10)
    cfg = IndexConfig(run_path=str(tmp_path / "run"), token_batch_size=32)
    cfg.partial_run_path.mkdir(parents=True)
    batches = allocate_batches(ds["length"], 32)
    collect_hessians(model, ds, cfg, batches=batches, hessian_cfg=HessianConfig(method="kfac", use_dataset_labels=True))
    A = load_file(str(cfg.partial_run_path / "activation_sharded" / "shard_0.safetensors"))
    S = load_file(str(cfg.partial_run_path / "gradient_sharded" / "shard_0.safetensors"))
    name = "layers.0.mlp.down_proj"
    layer = model.base_model.get_submodule(name)
    acts, grads = [], []
    def grab(m, i, o):
        acts.append(i[0].detach())
        o.register_hook(lambda g: grads.append(g.detach()))

    h1 = layer.register_forward_hook(grab)
    A_ref, S_ref = 0, 0
    for b in batches:
        rows = ds[b]
        x, y, _, mask = pad_and_tensor(rows["input_ids"], sync_max_len=False)
        logits = model(x).logits[:, :-1]
        loss = torch.nn.functional.cross_entropy(logits.reshape(-1, logits.size(-1)), y[:, 1:].reshape(-1), reduction="sum")
        loss.backward()
        a, g = acts.pop()[mask], grads.pop()[mask]
        A_ref, S_ref = A_ref + a.T @ a, S_ref + g.T @ g
    h1.remove()
    assert (A[name] - A_ref).norm() / A_ref.norm() < 1e-4
    assert (S[name] - S_ref).norm() / S_ref.norm() < 1e-4
    total = torch.load(cfg.partial_run_path / "total_processed.pt")
    assert int(total) == sum(l - 1 for l in ds["length"])
    vals_a = compute_eigendecomposition(str(cfg.partial_run_path / "activation_sharded"), total)
    vals_g = compute_eigendecomposition(str(cfg.partial_run_path / "gradient_sharded"), total)
    save_uncorrected_eigenvalues(cfg.partial_run_path, vals_a, vals_g, total, 0, 1)
    qa = load_file(str(cfg.partial_run_path / "eigen_activation_sharded" / "shard_0.safetensors"))[name].double()
    torch.testing.assert_close(qa @ torch.diag(vals_a[name].double()) @ qa.T, (A_ref / total).double(), atol=1e-4, rtol=1e-3)
    grid = load_file(str(cfg.partial_run_path / "eigenvalue_sharded" / "shard_0.safetensors"))[name]
    torch.testing.assert_close(grid, torch.outer(vals_g[name], vals_a[name]) * total, rtol=1e-5, atol=1e-8)


def test_compute_lambda_and_weighted_ce():
    q = {"m": (torch.tensor([4.0, 2.0, 1.0]), torch.eye(3))}
    i = {"m": (torch.tensor([8.0, 6.0, 3.0]), torch.eye(3))}
    assert abs(compute_lambda(q, i, 2) - 6.0 / 8.0) < 1e-9
    assert compute_lambda(q, i, 0) == 1.0 and compute_lambda({}, {}) == 0.99
    torch.manual_seed(0)
    logits, labels = torch.randn(2, 5, 7), torch.randint(0, 7, (2, 5))
    labels[1, 3:] = -100
    plain = weighted_causal_lm_ce(logits, labels)
    ones = weighted_causal_lm_ce(logits, labels, example_weight=torch.ones(2))
    torch.testing.assert_close(plain, ones)
    per_tok = torch.nn.functional.cross_entropy(logits[:, :-1].reshape(-1, 7), labels[:, 1:].reshape(-1), reduction="none",
                                                ignore_index=-100).view(2, 4)
    w = torch.tensor([2.0, 0.5])
    torch.testing.assert_close(weighted_causal_lm_ce(logits, labels, example_weight=w, reduction="sum"), (per_tok * w[:, None]).sum())
    som = (per_tok.sum(1) / torch.tensor([4.0, 2.0])).sum()
    torch.testing.assert_close(weighted_causal_lm_ce(logits, labels, reduction="sum_of_means"), som)


def _gloo_worker(rank, world, port, tmp):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from bergson_b200.hessians.sharded_computation import ShardedMul

        torch.manual_seed(0)
        full = torch.randn(5, 5)
        x = torch.randn(2, 3, 5)
        sm = ShardedMul()
        lo, hi = sm.shard_bounds(5)
        shard = full[lo:hi].contiguous()
        torch.testing.assert_close(sm.gather_rows(shard, 5), full)
        torch.testing.assert_close(sm._matmul(x, shard), x @ full)
        torch.testing.assert_close(sm._transpose_matmul(x, shard), x @ full.T)
        torch.testing.assert_close(sm.global_mean(shard, 25), full.mean())
        grid = torch.randn(5, 4)
        m = torch.ones(2, 5, 4)
        sm.scale_rows_in_place(m, grid[lo:hi].contiguous())
        torch.testing.assert_close(m, grid.expand(2, 5, 4))
        open(os.path.join(tmp, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_sharded_algebra_two_gloo_ranks(tmp_path):
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_gloo_worker, args=(r, 2, port, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()
