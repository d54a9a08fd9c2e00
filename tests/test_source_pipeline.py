"""SOURCE (approximate unrolling) end to end on CPU: four checkpoints of a tiny model in two
segments, plain and optimizer-preconditioned, checked against a dense restatement of the
method's algebra on the stored EK-FAC factors."""

import numpy as np
import torch

from bergson_b200.__main__ import main
from bergson_b200.data import load_gradients, load_scores
from bergson_b200.models import build_model
from bergson_b200.models.registry import PRESETS, args_from_dict

TRAIN = "synthetic:zipf?n=12&len=16&vocab=256&seed=0&min_len=6"
QUERY = "synthetic:zipf?n=4&len=16&vocab=256&seed=1&min_len=8"


def _checkpoints(root, n=4, with_optimizer=False):
    """``checkpoint-<step>`` directories holding a drifting copy of one tiny Llama."""
    args = args_from_dict(dict(PRESETS["llama-tiny"], vocab_size=256))
    model = build_model(args, seed=0)
    g = torch.Generator().manual_seed(7)
    paths = []
    for i in range(n):
        with torch.no_grad():
            for p in model.parameters():
                p.add_(0.01 * torch.randn(p.shape, generator=g))
        d = root / f"checkpoint-{10 * (i + 1)}"
        model.save_pretrained(d)
        if with_optimizer:
            names = [n_ for n_, _ in model.named_parameters()]
            state = {k: {"step": torch.tensor(float(10 * (i + 1))), "exp_avg": torch.zeros_like(p),
                         "exp_avg_sq": torch.rand(p.shape, generator=g) * 1e-2 + 1e-3}
                     for k, (_, p) in enumerate(model.named_parameters())}
            torch.save({"state": state, "param_groups": [{"params": list(range(len(names))), "param_names": names,
                                                          "lr": 1e-2, "betas": (0.9, 0.999), "eps": 1e-8,
                                                          "weight_decay": 0.0}]}, d / "optimizer.pt")
        paths.append(str(d))
    return paths


def _run(tmp_path, name, ckpts, *extra):
    out = tmp_path / name
    main([str(a) for a in (
        "approxunrolling", out, "--model", ckpts[-1], "--index_cfg.data.dataset", TRAIN,
        "--approx_unrolling_cfg.query.dataset", QUERY, "--checkpoints", *ckpts, "--segments", "2",
        "--lr_list", "0.01", "0.02", "--step_size_list", "20", "20", "--nproc_per_node", "1",
        "--token_batch_size", "64", "--ev_correction", "True", "--use_dataset_labels", *extra)])
    return out


def test_source_pipeline_runs_and_matches_dense_algebra(tmp_path):
    ckpts = _checkpoints(tmp_path)
    out = _run(tmp_path, "source", ckpts)
    for d in ("segment_0/kfac/eigenvalue_correction_sharded", "segment_1/kfac/eigen_activation_sharded", "query",
              "segment_0/query_grad_backward", "segment_0/query_grad_segment", "segment_1/query_grad_segment",
              "segment_1/scores_ckpt_1", "scores"):
        assert (out / d).exists(), d
    s = load_scores(out / "scores")[:]
    assert s.shape == (12, 1) and np.isfinite(s).all() and np.abs(s).max() > 0

    # Dense restatement for one module: q_0 = Q exp(-eta K_1 Lam_1) Q^T q_1 and
    # r_l = Q f_s(Lam_l) Q^T q_l with f_s(s) = (1 - exp(-eta K s)) / s, on the saved factors.
    from safetensors.torch import load_file

    def factors(seg):
        base = out / f"segment_{seg}" / "kfac"
        qa = load_file(str(base / "eigen_activation_sharded" / "shard_0.safetensors"))
        qg = load_file(str(base / "eigen_gradient_sharded" / "shard_0.safetensors"))
        lam = load_file(str(base / "eigenvalue_correction_sharded" / "shard_0.safetensors"))
        return qa, qg, lam

    import json

    name = "layers.0.self_attn.q_proj"

    def block(store, O, I):
        """The module's [n, O, I] block of a gradient store (stores order their columns
        by their own info.json)."""
        sizes = json.load(open(store / "info.json"))["grad_sizes"]
        off = 0
        for k, v in sizes.items():
            if k == name:
                break
            off += v
        rows = torch.from_numpy(np.asarray(load_gradients(store), dtype=np.float64))
        return rows[:, off : off + O * I].view(-1, O, I)

    qa1, qg1, lam1 = factors(1)
    O, I = qg1[name].shape[0], qa1[name].shape[0]
    g1 = block(out / "query", O, I)

    def apply(g, qa, qg, lam, fn):
        rot = qg.double().T @ g @ qa.double()
        return qg.double() @ (rot * fn(lam.double())) @ qa.double().T

    k0, k1 = 0.01 * 20, 0.02 * 20
    g0 = apply(g1, qa1[name], qg1[name], lam1[name], lambda s_: torch.exp(-k1 * s_))
    torch.testing.assert_close(block(out / "segment_0" / "query_grad_backward", O, I), g0, rtol=1e-3, atol=1e-6)

    def f_seg(k):
        return lambda s_: torch.where(s_ == 0, torch.full_like(s_, k), -torch.expm1(-k * s_) / s_.masked_fill(s_ == 0, 1))

    qa0, qg0, lam0 = factors(0)
    r0 = apply(g0, qa0[name], qg0[name], lam0[name], f_seg(k0))
    torch.testing.assert_close(block(out / "segment_0" / "query_grad_segment", O, I), r0, rtol=1e-3, atol=1e-6)

    # Final scores: sum over segments of the mean over the segment's checkpoints, written
    # loss-signed (the per-checkpoint inner products are influence-signed).
    total = 0
    for seg in range(2):
        total = total + sum(load_scores(out / f"segment_{seg}" / f"scores_ckpt_{c}")[:] for c in range(2)) / 2
    np.testing.assert_allclose(s, -total, rtol=1e-5, atol=1e-8)


def test_source_pipeline_with_adam_preconditioner(tmp_path):
    ckpts = _checkpoints(tmp_path, with_optimizer=True)
    out = _run(tmp_path, "source_adam", ckpts, "--use_adam_preconditioner")
    assert (out / "segment_0" / "preconditioner.safetensors").exists()
    s = load_scores(out / "scores")[:]
    assert s.shape == (12, 1) and np.isfinite(s).all() and np.abs(s).max() > 0
    # Resuming reuses every finished step and reproduces the scores.
    again = _run(tmp_path, "source_adam", ckpts, "--use_adam_preconditioner")
    np.testing.assert_allclose(load_scores(again / "scores")[:], s)
