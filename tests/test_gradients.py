"""Collector output against per-example autograd ground truth."""

import pytest
import torch

from bergson_b200 import GradientCollector, GradientProcessor
from bergson_b200.collector.collector import create_projection_matrix
from bergson_b200.collector.gradient_collectors import TraceCollector
from bergson_b200.gradients import AdafactorNormalizer, AdamNormalizer

from .helpers import TwoLayer


def _per_example_grads(model, x, y, include_bias):
    out = []
    for n in range(x.shape[0]):
        model.zero_grad()
        loss = ((model(x[n : n + 1]) - y[n : n + 1]) ** 2).sum()
        loss.backward()
        row = {}
        for name in ("fc1", "fc2"):
            m = getattr(model, name)
            g = m.weight.grad.clone()
            if include_bias and m.bias is not None:
                g = torch.cat([g, m.bias.grad[:, None]], dim=1)
            row[name] = g
        out.append(row)
    return out


def _collect(model, x, y, processor, **kw):
    c = TraceCollector(model=model, processor=processor, device="cpu", dtype=torch.float32, **kw)
    with c:
        ((model(x) - y) ** 2).sum().backward()
    model.zero_grad()
    return {k: torch.cat(v) for k, v in c.mod_grads.items()}


@pytest.mark.parametrize("include_bias", [False, True])
def test_full_gradients_match_separate_backward(include_bias):
    torch.manual_seed(0)
    model = TwoLayer()
    x, y = torch.randn(4, 6, 5), torch.randn(4, 6, 2)
    truth = _per_example_grads(model, x, y, include_bias)
    got = _collect(model, x, y, GradientProcessor(include_bias=include_bias))
    for n in range(4):
        for name in ("fc1", "fc2"):
            torch.testing.assert_close(got[name][n], truth[n][name].flatten())


@pytest.mark.parametrize("include_bias", [False, True])
@pytest.mark.parametrize("ptype", ["rademacher", "normal"])
def test_projection_is_two_sided(include_bias, ptype):
    torch.manual_seed(1)
    model = TwoLayer()
    x, y = torch.randn(3, 6, 5), torch.randn(3, 6, 2)
    truth = _per_example_grads(model, x, y, include_bias)
    p = 4
    got = _collect(model, x, y, GradientProcessor(projection_dim=p, projection_type=ptype, include_bias=include_bias))
    for name, (o, i) in {"fc1": (3, 5), "fc2": (2, 3)}.items():
        i_eff = i + (1 if include_bias else 0)
        L = create_projection_matrix(f"{name}/left", p, o, torch.float32, torch.device("cpu"), ptype)
        R = create_projection_matrix(f"{name}/right", p, i_eff, torch.float32, torch.device("cpu"), ptype)
        for n in range(3):
            torch.testing.assert_close(got[name][n].view(p, p), L @ truth[n][name] @ R.T, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("kind", ["adam", "adafactor"])
@pytest.mark.parametrize("p", [None, 4])
def test_normalizers(kind, p):
    torch.manual_seed(2)
    model = TwoLayer(bias=False)
    x, y = torch.randn(3, 6, 5), torch.randn(3, 6, 2)
    truth = _per_example_grads(model, x, y, False)
    norms = {}
    for name, (o, i) in {"fc1": (3, 5), "fc2": (2, 3)}.items():
        v = torch.rand(o, i) + 0.1
        norms[name] = AdamNormalizer(v) if kind == "adam" else AdamNormalizer(v).to_adafactor()
    got = _collect(model, x, y, GradientProcessor(normalizers=norms, projection_dim=p))
    for name, (o, i) in {"fc1": (3, 5), "fc2": (2, 3)}.items():
        for n in range(3):
            g = truth[n][name].clone()
            expect = norms[name].normalize_weight(g)
            if p:
                L = create_projection_matrix(f"{name}/left", p, o, torch.float32, torch.device("cpu"), "rademacher")
                R = create_projection_matrix(f"{name}/right", p, i, torch.float32, torch.device("cpu"), "rademacher")
                expect = L @ expect @ R.T
            torch.testing.assert_close(got[name][n], expect.flatten(), atol=1e-3, rtol=1e-3)


def test_token_rows_sum_to_sequence_rows():
    torch.manual_seed(3)
    model = TwoLayer()
    x, y = torch.randn(2, 6, 5), torch.randn(2, 6, 2)
    mask = torch.ones(2, 6, dtype=torch.bool)
    seq = _collect(model, x, y, GradientProcessor(projection_dim=4))
    c = TraceCollector(model=model, processor=GradientProcessor(projection_dim=4), device="cpu",
                       dtype=torch.float32, attribute_tokens=True)
    with c.with_batch(mask):
        ((model(x) - y) ** 2).sum().backward()
    for name in ("fc1", "fc2"):
        tok = torch.cat(c.mod_grads[name]).view(2, 6, -1).sum(1)
        torch.testing.assert_close(tok, seq[name], atol=1e-5, rtol=1e-4)


def test_head_split_matches_row_blocks():
    from bergson_b200.config import AttentionConfig

    torch.manual_seed(4)
    model = TwoLayer(i=5, h=6, o=2, bias=False)
    x, y = torch.randn(3, 4, 5), torch.randn(3, 4, 2)
    full = _collect(model, x, y, GradientProcessor(), target_modules={"fc1"})
    heads = _collect(model, x, y, GradientProcessor(), target_modules={"fc1"},
                     attention_cfgs={"fc1": AttentionConfig(num_heads=3, head_size=2, head_dim=2)})
    whole = full["fc1"].view(3, 6, 5)
    for h in range(3):
        torch.testing.assert_close(heads[f"fc1.head_{h}"].view(3, 2, 5), whole[:, 2 * h : 2 * h + 2])


def test_projection_matrix_is_deterministic_and_scaled():
    a = create_projection_matrix("m/left", 16, 64, torch.float32, torch.device("cpu"), "rademacher")
    b = create_projection_matrix("m/left", 16, 64, torch.float32, torch.device("cpu"), "rademacher")
    c = create_projection_matrix("m/right", 16, 64, torch.float32, torch.device("cpu"), "rademacher")
    assert torch.equal(a, b) and not torch.equal(a, c)
    assert torch.allclose(a.abs(), torch.full_like(a, 0.25))
    n = create_projection_matrix("m/left", 16, 64, torch.float32, torch.device("cpu"), "normal", "row_norm")
    torch.testing.assert_close(n.norm(dim=1), torch.ones(16))


def test_jl_inner_products_are_preserved_in_expectation():
    torch.manual_seed(5)
    g1, g2 = torch.randn(24, 40), torch.randn(24, 40)
    g2 = g2 + 0.5 * g1
    exact = (g1 * g2).sum()
    est = []
    for t in range(300):
        L = create_projection_matrix(f"t{t}/left", 8, 24, torch.float32, torch.device("cpu"), "rademacher")
        R = create_projection_matrix(f"t{t}/right", 8, 40, torch.float32, torch.device("cpu"), "rademacher")
        est.append(((L @ g1 @ R.T) * (L @ g2 @ R.T)).sum())
    assert abs(torch.stack(est).mean() / exact - 1) < 0.15


def _mean_ratio(o, i, p, ptype, trials=200, seed=7):
    g = torch.Generator().manual_seed(seed)
    g1 = torch.randn(o, i, generator=g)
    g2 = g1 + 0.3 * torch.randn(o, i, generator=g)
    true = float((g1 * g2).sum())
    acc = 0.0
    cpu = torch.device("cpu")
    for t in range(trials):
        L = create_projection_matrix(f"s{t}/left", p, o, torch.float32, cpu, ptype)
        R = create_projection_matrix(f"s{t}/right", p, i, torch.float32, cpu, ptype)
        acc += float(((L @ g1 @ R.T) * (L @ g2 @ R.T)).sum())
    return acc / trials / true


@pytest.mark.parametrize("ptype", ["rademacher", "normal"])
def test_projection_scale_is_the_same_for_every_module_shape(ptype):
    """Modules are summed into one score: a shape-dependent scale would reweight attention
    against MLP layers."""
    square, wide = _mean_ratio(32, 32, 16, ptype), _mean_ratio(32, 128, 16, ptype)
    assert square == pytest.approx(1.0, rel=0.15) and wide == pytest.approx(1.0, rel=0.15)
    A = create_projection_matrix("variance", 64, 256, torch.float32, torch.device("cpu"), ptype)
    assert A.pow(2).mean().item() == pytest.approx(1 / 64, rel=0.1)  # entry variance 1 / output dim
    assert (A.T @ A).diagonal().mean().item() == pytest.approx(1.0, rel=0.1)


def test_one_matrix_per_module_summed_is_unbiased():
    """The global projection applies one independent matrix per module and adds the results."""
    dims, p = [64, 256], 32
    g = torch.Generator().manual_seed(11)
    xs = [torch.randn(d, generator=g) for d in dims]
    ys = [x + 0.3 * torch.randn(d, generator=g) for x, d in zip(xs, dims)]
    true = sum(float((x * y).sum()) for x, y in zip(xs, ys))
    acc = 0.0
    for t in range(200):
        for k, d in enumerate(dims):
            R = create_projection_matrix(f"g{k}_{t}", p, d, torch.float32, torch.device("cpu"), "rademacher")
            acc += float(((xs[k] @ R.T) * (ys[k] @ R.T)).sum())
    assert acc / 200 / true == pytest.approx(1.0, rel=0.15)


def test_processor_saved_before_the_scale_option_loads_row_normalised(tmp_path):
    import yaml

    GradientProcessor(projection_dim=8).save(tmp_path)
    cfg = yaml.safe_load((tmp_path / "processor_config.yaml").read_text())
    assert cfg["projection_scale"] == "jl"
    del cfg["projection_scale"]
    (tmp_path / "processor_config.yaml").write_text(yaml.safe_dump(cfg))
    assert GradientProcessor.load(tmp_path).projection_scale == "row_norm"
