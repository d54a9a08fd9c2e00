"""EK-FAC on the GPU kernels (SYRK covariances, fused eigenvalue correction, fp32-accurate
factored apply) against the fp32 CPU path of the same pipeline."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_split_matmul_is_fp32_accurate():
    from bergson_b200.ops.attribution import split_matmul

    torch.manual_seed(0)
    a = torch.randn(300, 520, device="cuda")
    b = torch.randn(520, 264, device="cuda")
    ref = a.double() @ b.double()
    got = split_matmul(a, b)
    err = float((got.double() - ref).abs().max() / ref.abs().max())
    plain = float(((a.bfloat16() @ b.bfloat16()).double() - ref).abs().max() / ref.abs().max())
    assert err < 2e-5 and err < plain / 50, (err, plain)


def test_factored_apply_on_gpu_matches_fp64():
    from bergson_b200.hessians.preconditioner import FactoredPreconditioner

    torch.manual_seed(1)
    o, i, n = 72, 136, 5
    q_a = torch.linalg.qr(torch.randn(i, i, dtype=torch.float64))[0]
    q_g = torch.linalg.qr(torch.randn(o, o, dtype=torch.float64))[0]
    lam = torch.rand(o, i, dtype=torch.float64) + 0.1
    g = torch.randn(n, o * i, dtype=torch.float64)
    fn = lambda s: 1.0 / (s + 0.05)  # noqa: E731
    ref = q_g @ ((q_g.T @ g.view(n, o, i) @ q_a) * fn(lam)) @ q_a.T
    pre = FactoredPreconditioner({"m": q_a.float().cuda()}, {"m": q_g.float().cuda()}, {"m": lam.float().cuda()},
                                 apply_fn=fn)
    got = pre.apply({"m": g.float().cuda()})["m"].double().cpu().view(n, o, i)
    assert float((got - ref).abs().max() / ref.abs().max()) < 5e-5


def test_ekfac_pipeline_on_gpu_tracks_the_cpu_run(tmp_path):
    from bergson_b200.__main__ import main
    from bergson_b200.data import load_scores
    from bergson_b200.hessians.preconditioner import _load_full

    common = ["--model", "native:llama-tiny?hidden_size=128&intermediate_size=256&vocab_size=1024",
              "--index_cfg.data.dataset", "synthetic:zipf?n=24&len=96&vocab=1024&seed=0&min_len=50",
              "--hessian_pipeline_cfg.query.dataset", "synthetic:zipf?n=4&len=96&vocab=1024&seed=1&min_len=50",
              "--method", "kfac", "--hessian_cfg.ev_correction", "true", "--use_dataset_labels", "--token_batch_size", "512",
              "--nproc_per_node", "1"]
    import os

    main(["ekfac", str(tmp_path / "gpu"), "--index_cfg.precision", "bf16", *common])
    os.environ["CUDA_VISIBLE_DEVICES_SAVED"] = os.environ.get("CUDA_VISIBLE_DEVICES", "")
    # the CPU reference run: same weights (seeded init), fp32
    import subprocess
    import sys
    from pathlib import Path

    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    out = subprocess.run([sys.executable, "-m", "bergson_b200", "ekfac", str(tmp_path / "cpu"), "--index_cfg.precision", "fp32", *common],
                         cwd=Path(__file__).resolve().parents[1], env=env, capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stderr[-2000:]
    for sub in ("activation_sharded", "gradient_sharded", "eigenvalue_correction_sharded"):
        a = _load_full(tmp_path / "gpu" / "hessian" / "kfac", sub, "cpu")
        b = _load_full(tmp_path / "cpu" / "hessian" / "kfac", sub, "cpu")
        for k in b:
            rel = float((a[k] - b[k]).norm() / b[k].norm())
            assert rel < (0.08 if sub == "eigenvalue_correction_sharded" else 0.04), (sub, k, rel)
    s_gpu, s_cpu = load_scores(tmp_path / "gpu" / "scores")[:], load_scores(tmp_path / "cpu" / "scores")[:]
    assert np.corrcoef(s_gpu.ravel().astype(np.float64), s_cpu.ravel().astype(np.float64))[0, 1] > 0.98


@pytest.mark.parametrize("drop_scale", [1.0, 30.0])
def test_gram_with_dropped_rows_at_the_fused_path_boundary(drop_scale):
    """The fused covariance path runs the SYRK over all rows and subtracts the Gram of the
    skipped ones; it is taken while at most 1/8 of the rows are skipped.  Exactly at that
    boundary, and with skipped rows far larger than the kept ones (the case where the
    subtraction cancels most of the sum), the result must still match the masked oracle."""
    from types import SimpleNamespace

    from bergson_b200.hessians.kfac import _FactorCollector

    torch.manual_seed(0)
    n, s, d = 8, 64, 256
    x = torch.randn(n, s, d, device="cuda")
    mask = torch.ones(n, s, dtype=torch.bool, device="cuda")
    mask[:, -8:] = False  # 8 of 64 positions per sequence: exactly one eighth
    x[~mask] *= drop_scale
    x = x.to(torch.bfloat16)
    flat = mask.reshape(-1)
    stub = SimpleNamespace(_keep_idx=flat.nonzero(as_tuple=True)[0], _drop_idx=(~flat).nonzero(as_tuple=True)[0],
                           _peer=None, _final_batch=False, _flushed=set(), _flushed_in_gemm=set(),
                           _current_collection_mask=mask, dtype=torch.bfloat16)
    stub._masked = lambda t: _FactorCollector._masked(stub, t)
    acc = torch.zeros(d, d, device="cuda")
    _FactorCollector._gram_into(stub, acc, x)
    assert stub._drop_idx.numel() * 8 == n * s  # the boundary case of the fused path
    kept = x.reshape(-1, d)[flat].double()
    want = kept.T @ kept
    err = (acc.double() - want).abs().max() / want.abs().max()
    # fp32 accumulation of sums that are drop_scale^2 / 7 times larger than the result
    assert err < 1e-5 * max(1.0, drop_scale**2), float(err)
    # One more skipped row takes the compaction path (no subtraction): same oracle.
    mask2 = mask.clone()
    mask2[0, 0] = False
    flat2 = mask2.reshape(-1)
    stub2 = SimpleNamespace(**{**stub.__dict__, "_keep_idx": flat2.nonzero(as_tuple=True)[0],
                               "_drop_idx": (~flat2).nonzero(as_tuple=True)[0], "_current_collection_mask": mask2})
    stub2._masked = lambda t: _FactorCollector._masked(stub2, t)
    acc2 = torch.zeros(d, d, device="cuda")
    _FactorCollector._gram_into(stub2, acc2, x)
    kept2 = x.reshape(-1, d)[flat2].double()
    want2 = kept2.T @ kept2
    assert (acc2.double() - want2).abs().max() / want2.abs().max() < 1e-5 * max(1.0, drop_scale**2)
