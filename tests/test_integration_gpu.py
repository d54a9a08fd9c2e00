"""Fused collection, scoring and querying on a GPU against the torch path."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def setup():
    from bergson_b200.data import allocate_batches, synthetic_dataset
    from bergson_b200.gradients import AdafactorNormalizer
    from bergson_b200.models import build_model
    from bergson_b200.models.registry import PRESETS, args_from_dict

    dev = torch.device("cuda:0")
    args = args_from_dict(dict(PRESETS["llama-tiny"], hidden_size=128, intermediate_size=256, vocab_size=1024))
    model = build_model(args, dtype=torch.bfloat16, device=dev)
    model.requires_grad_(False)
    model.get_input_embeddings().requires_grad_(True)
    ds = synthetic_dataset("synthetic:zipf?n=20&len=150&vocab=1024&seed=0&min_len=70")
    qs = synthetic_dataset("synthetic:zipf?n=6&len=150&vocab=1024&seed=1&min_len=70")
    g = torch.Generator().manual_seed(0)
    norms = {n: AdafactorNormalizer((torch.rand(m.out_features, generator=g) + 0.5).to(dev),
                                    (torch.rand(m.in_features, generator=g) + 0.5).to(dev))
             for n, m in model.base_model.named_modules() if isinstance(m, torch.nn.Linear)}
    return model, ds, qs, norms, allocate_batches


def _build(tmp, name, model, data, norms, allocate_batches, fused, dtype="fp32", unit=False):
    from bergson_b200 import GradientProcessor, IndexConfig, PreprocessConfig, collect_gradients, load_gradients

    cfg = IndexConfig(run_path=str(tmp / name), projection_dim=16, token_batch_size=600, store_dtype=dtype,
                      fused_collection=fused)
    cfg.partial_run_path.mkdir(parents=True)
    c = collect_gradients(model, data, GradientProcessor(norms, projection_dim=16), cfg,
                          batches=allocate_batches(data["length"], 600),
                          preprocess_cfg=PreprocessConfig(unit_normalize=unit))
    assert c._fused_enabled == fused
    torch.cuda.synchronize()
    return cfg.partial_run_path, np.array(load_gradients(cfg.partial_run_path)).astype(np.float32)


@pytest.mark.parametrize("dtype,unit", [("fp32", False), ("fp16", False), ("bf16", True)])
def test_fused_store_matches_torch_path(tmp_path, setup, dtype, unit):
    model, ds, _, norms, alloc = setup
    _, a = _build(tmp_path, "fused", model, ds, norms, alloc, True, dtype, unit)
    _, b = _build(tmp_path, "plain", model, ds, norms, alloc, False, dtype, unit)
    assert np.isfinite(a).all() and np.abs(b).max() > 0
    assert np.abs(a - b).max() / np.abs(b).max() < 3e-2
    cos = (a * b).sum(1) / (np.linalg.norm(a, axis=1) * np.linalg.norm(b, axis=1))
    assert cos.min() > 0.999


def test_fused_scoring_matches_store_products(tmp_path, setup):
    from bergson_b200 import GradientProcessor, IndexConfig, PreprocessConfig, ScoreConfig, collect_gradients
    from bergson_b200.data import load_scores
    from bergson_b200.score.score import create_scorer

    model, ds, qs, norms, alloc = setup
    _, g = _build(tmp_path, "index", model, ds, norms, alloc, True)
    qpath, q = _build(tmp_path, "query", model, qs, norms, alloc, True)
    from bergson_b200.cli.commands import Build
    from bergson_b200.config.config_io import save_run_config

    save_run_config(Build(IndexConfig(run_path=str(qpath)), PreprocessConfig()), qpath)
    for prec, tol in (("bf16", 3e-2), ("fp32", 3e-2)):
        cfg = IndexConfig(run_path=str(tmp_path / f"s_{prec}"), projection_dim=16, token_batch_size=600)
        cfg.partial_run_path.mkdir(parents=True)
        scorer = create_scorer(cfg.partial_run_path, ds, ScoreConfig(query_path=str(qpath), precision=prec),
                               PreprocessConfig(), torch.device("cuda:0"),
                               torch.bfloat16 if prec == "bf16" else torch.float32)
        collect_gradients(model, ds, GradientProcessor(norms, projection_dim=16), cfg,
                          batches=alloc(ds["length"], 600), scorer=scorer)
        scorer.writer.flush()
        s = load_scores(cfg.partial_run_path)[:].astype(np.float32)
        ref = g @ q.T
        assert np.abs(s - ref).max() / np.abs(ref).max() < tol


def test_attributor_topk_on_gpu(tmp_path, setup):
    from bergson_b200 import Attributor

    model, ds, _, norms, alloc = setup
    path, g = _build(tmp_path, "index", model, ds, norms, alloc, True, "fp16")
    for dtype in (torch.float16, torch.float32):
        attr = Attributor(path, device="cuda:0", dtype=dtype, unit_norm=True)
        queries = {n: torch.from_numpy(g[:4, lo:hi]).cuda() for n, (lo, hi) in attr.offsets.items()}
        scores, idx = attr.search(queries, k=3)
        assert idx[:, 0].tolist() == [0, 1, 2, 3] and (scores[:, 0] > 0.99).all()
        low, lidx = attr.search(queries, k=2, reverse=True)
        gn = g / np.linalg.norm(g, axis=1, keepdims=True)
        ref = gn[:4] @ gn.T
        np.testing.assert_allclose(low[:, 0].cpu().numpy(), ref.min(1), atol=2e-2)
