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
