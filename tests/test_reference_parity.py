"""Cross-implementation check: the reference's collector and ours write the same store
for the same model and data.  Skipped when the reference is not installed under
``baseline/_ref``."""

import importlib
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
REF = ROOT / "baseline" / "_ref"
SHIMS = ROOT / "baseline" / "shims"

pytestmark = pytest.mark.skipif(not (REF / "bergson").exists(), reason="reference not installed")


@pytest.fixture(scope="module")
def ref():
    added = [str(SHIMS), str(REF)]
    sys.path[:0] = added
    try:
        yield importlib.import_module("bergson")
    finally:
        for p in added:
            sys.path.remove(p)


@pytest.mark.parametrize("family", ["gpt_neox", "llama"])
@pytest.mark.parametrize("normalizer", [False, True])
def test_store_matches_reference(tmp_path, ref, family, normalizer):
    from bergson_b200 import GradientProcessor, IndexConfig, collect_gradients, load_gradients
    from bergson_b200.data import allocate_batches
    from bergson_b200.gradients import AdafactorNormalizer

    from .helpers import tiny_dataset, tiny_model

    torch.manual_seed(0)
    model = tiny_model(family)
    model.requires_grad_(False)
    model.get_input_embeddings().requires_grad_(True)
    ds = tiny_dataset(n=10, length=14)
    batches = allocate_batches(ds["length"], 40)

    def normalizers(mod):
        if not normalizer:
            return {}
        out = {}
        g = torch.Generator().manual_seed(1)
        for name, m in model.base_model.named_modules():
            if isinstance(m, torch.nn.Linear):
                out[name] = mod.AdafactorNormalizer(torch.rand(m.out_features, generator=g) + 0.1,
                                                    torch.rand(m.in_features, generator=g) + 0.1)
        return out

    import bergson_b200.gradients as ours_grad

    ours_cfg = IndexConfig(run_path=str(tmp_path / "ours"), projection_dim=4, token_batch_size=40)
    ours_cfg.partial_run_path.mkdir(parents=True)
    collect_gradients(model, ds, GradientProcessor(normalizers(ours_grad), projection_dim=4), ours_cfg, batches=batches)

    ref_cfg = ref.IndexConfig(run_path=str(tmp_path / "ref"), projection_dim=4, token_batch_size=40)
    ref_cfg.partial_run_path.mkdir(parents=True)
    ref_grad = importlib.import_module("bergson.gradients")
    ref.collect_gradients(model, ds, ref.GradientProcessor(normalizers(ref_grad), projection_dim=4), ref_cfg,
                          batches=batches)

    a = np.asarray(load_gradients(ours_cfg.partial_run_path))
    b = np.asarray(ref.load_gradients(ref_cfg.partial_run_path))
    assert a.shape == b.shape and a.dtype == b.dtype
    np.testing.assert_allclose(a, b, rtol=2e-4, atol=1e-5)
    # metadata is interchangeable
    import json

    ia = json.load(open(ours_cfg.partial_run_path / "info.json"))
    ib = json.load(open(ref_cfg.partial_run_path / "info.json"))
    assert ia == ib
    assert a.tobytes() == np.asarray(ref.load_gradients(ours_cfg.partial_run_path)).tobytes()
