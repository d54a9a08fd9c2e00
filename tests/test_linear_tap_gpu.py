"""Linear layers on the tcgen05 GEMM and the collector taps that ride on them, against
autograd / the torch collection path."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("layout", ["oi", "io"])
@pytest.mark.parametrize("bias", [False, True])
def test_linear_forward_and_all_gradients(layout, bias):
    from bergson_b200.ops.linear import linear

    torch.manual_seed(0)
    N, S, I, O = 3, 70, 136, 264
    x = torch.randn(N, S, I, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn((O, I) if layout == "oi" else (I, O), device="cuda") / 8).to(torch.bfloat16).requires_grad_(True)
    b = torch.randn(O, device="cuda", dtype=torch.bfloat16, requires_grad=True) if bias else None
    y = linear(x, w, b, layout=layout)
    g = torch.randn_like(y)
    y.backward(g)
    xf, wf = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    bf = b.detach().float().requires_grad_(True) if bias else None
    yf = (xf @ wf.T if layout == "oi" else xf @ wf) + (bf if bias else 0)
    yf.backward(g.float())
    rel = lambda a, r: float((a.float() - r).abs().max() / r.abs().max())  # noqa: E731
    assert rel(y, yf.detach()) < 1e-2
    assert rel(x.grad, xf.grad) < 1e-2
    assert rel(w.grad, wf.grad) < 1e-2
    if bias:
        assert rel(b.grad, bf.grad) < 1e-2


def _collect(tmp, name, family, p, fused, tokens=False, dtype="fp32", bias=False, normalizers=True):
    from bergson_b200 import GradientProcessor, IndexConfig, collect_gradients, load_gradients
    from bergson_b200.data import allocate_batches, synthetic_dataset
    from bergson_b200.gradients import AdafactorNormalizer
    from bergson_b200.models import build_model
    from bergson_b200.models.registry import PRESETS, args_from_dict

    dev = torch.device("cuda:0")
    preset = {"llama": "llama-tiny", "gpt2": "gpt2-tiny", "gpt_neox": "neox-tiny"}[family]
    over = dict(hidden_size=128, intermediate_size=256, vocab_size=1024)
    if family == "gpt2":
        over["max_position_embeddings"] = 512
    model = build_model(args_from_dict(dict(PRESETS[preset], **over)), dtype=torch.bfloat16, device=dev)
    model.requires_grad_(False)
    model.get_input_embeddings().requires_grad_(True)
    ds = synthetic_dataset("synthetic:zipf?n=10&len=150&vocab=1024&seed=0&min_len=70")
    g = torch.Generator().manual_seed(0)
    norms = {}
    for n, m in model.base_model.named_modules():
        if isinstance(m, torch.nn.Linear):
            o, i = m.out_features, m.in_features
        elif type(m).__name__ == "Conv1D":
            o, i = m.nf, m.nx
        else:
            continue
        if not normalizers:
            continue
        norms[n] = AdafactorNormalizer((torch.rand(o, generator=g) + 0.5).to(dev), (torch.rand(i, generator=g) + 0.5).to(dev))
    cfg = IndexConfig(run_path=str(tmp / name), projection_dim=p, token_batch_size=600, store_dtype=dtype,
                      fused_collection=fused, attribute_tokens=tokens)
    cfg.partial_run_path.mkdir(parents=True)
    batches_run = allocate_batches(ds["length"], 600)
    c = collect_gradients(model, ds, GradientProcessor(norms, projection_dim=p, include_bias=bias), cfg,
                          batches=batches_run)
    assert c._fused_enabled == fused
    if fused:
        # every in-tree layer went through its tap (projection side outputs of its own GEMMs)
        assert c._tap_calls == len(batches_run) * len(c.target_info), (c._tap_calls, len(c.target_info))
    torch.cuda.synchronize()
    if tokens:
        from bergson_b200 import TokenGradients

        tg = TokenGradients(cfg.partial_run_path)
        return np.concatenate([np.asarray(tg[i], dtype=np.float32) for i in range(len(ds))])
    return np.array(load_gradients(cfg.partial_run_path)).astype(np.float32)


@pytest.mark.parametrize("family,p", [("llama", 16), ("llama", 8), ("llama", 32), ("gpt2", 16), ("gpt_neox", 16), ("llama", 64)])
def test_tapped_store_matches_torch_path(tmp_path, family, p):
    a = _collect(tmp_path, "fused", family, p, True)
    b = _collect(tmp_path, "plain", family, p, False)
    assert np.isfinite(a).all() and np.abs(b).max() > 0
    assert np.abs(a - b).max() / np.abs(b).max() < 3e-2
    cos = (a * b).sum(1) / (np.linalg.norm(a, axis=1) * np.linalg.norm(b, axis=1))
    assert cos.min() > 0.999


@pytest.mark.parametrize("family", ["gpt2", "gpt_neox"])
def test_tapped_store_with_bias_columns_matches_torch_path(tmp_path, family):
    """``include_bias`` without a normaliser: the bias gradient rides along as a constant vector
    added to the projected activations, so layers with a bias stay on the GEMM taps."""
    a = _collect(tmp_path, "fused", family, 16, True, bias=True, normalizers=False)
    b = _collect(tmp_path, "plain", family, 16, False, bias=True, normalizers=False)
    c = _collect(tmp_path, "nobias", family, 16, False, bias=False, normalizers=False)
    assert np.isfinite(a).all() and np.abs(b).max() > 0
    assert np.abs(a - b).max() / np.abs(b).max() < 3e-2
    cos = (a * b).sum(1) / (np.linalg.norm(a, axis=1) * np.linalg.norm(b, axis=1))
    assert cos.min() > 0.999
    assert np.abs(b - c).max() / np.abs(b).max() > 1e-2  # the bias column does change the rows


def test_tapped_token_rows_match_torch_path(tmp_path):
    a = _collect(tmp_path, "fused", "llama", 16, True, tokens=True)
    b = _collect(tmp_path, "plain", "llama", 16, False, tokens=True)
    assert a.shape == b.shape and np.abs(b).max() > 0
    assert np.abs(a - b).max() / np.abs(b).max() < 3e-2


def test_tapped_store_is_bitwise_repeatable(tmp_path):
    a = _collect(tmp_path, "one", "llama", 16, True)
    b = _collect(tmp_path, "two", "llama", 16, True)
    assert np.array_equal(a, b)
