"""Bias handling of the gradient collector: module metadata is left as found, models where only
some layers have a bias work under every normaliser, and the factored projection of
bias-augmented gradients equals projecting the full gradient."""

import pytest
import torch
import torch.nn as nn

from bergson_b200 import GradientProcessor
from bergson_b200.collector.collector import create_projection_matrix
from bergson_b200.collector.gradient_collectors import TraceCollector
from bergson_b200.gradients import AdafactorNormalizer, AdamNormalizer

N, S, I, H, O = 3, 5, 4, 6, 3


class Mixed(nn.Module):
    """fc1 has a bias, fc2 has none."""

    def __init__(self):
        super().__init__()
        self.fc1 = nn.Linear(I, H, bias=True)
        self.fc2 = nn.Linear(H, O, bias=False)

    @property
    def device(self):
        return self.fc1.weight.device

    def forward(self, x):
        return self.fc2(torch.relu(self.fc1(x)))


def _collect(model, x, processor):
    c = TraceCollector(model=model, processor=processor, device="cpu", dtype=torch.float32)
    with c:
        (model(x) ** 2).sum().backward()
    model.zero_grad()
    return c, {k: torch.cat(v) for k, v in c.mod_grads.items()}


def _truth(model, x):
    rows = []
    for n in range(x.shape[0]):
        model.zero_grad()
        (model(x[n:n + 1]) ** 2).sum().backward()
        rows.append({"fc1": torch.cat([model.fc1.weight.grad, model.fc1.bias.grad[:, None]], 1).clone(),
                     "fc2": model.fc2.weight.grad.clone()})
    model.zero_grad()
    return rows


def test_module_metadata_is_restored():
    torch.manual_seed(0)
    model = Mixed()
    before = {n: (m.in_features, m.out_features) for n, m in model.named_modules() if isinstance(m, nn.Linear)}
    x = torch.randn(N, S, I)
    for _ in range(3):  # nothing may accumulate over repeated uses either
        _collect(model, x, GradientProcessor(include_bias=True))
    assert {n: (m.in_features, m.out_features) for n, m in model.named_modules() if isinstance(m, nn.Linear)} == before
    assert not hasattr(model.fc1, "_collect_bias") or model.fc1.in_features == I
    out = model(x)  # and the model still runs without hooks
    assert out.shape == (N, S, O)


@pytest.mark.parametrize("kind", ["none", "adam", "adafactor"])
@pytest.mark.parametrize("p", [None, 2])
def test_layers_without_a_bias_under_include_bias(kind, p):
    torch.manual_seed(0)
    model = Mixed()
    norms = {}
    if kind == "adam":
        norms = {"fc1": AdamNormalizer(torch.rand(H, I) + 0.1, bias_avg_sq=torch.rand(H) + 0.1),
                 "fc2": AdamNormalizer(torch.rand(O, H) + 0.1, bias_avg_sq=None)}
    elif kind == "adafactor":
        norms = {"fc1": AdafactorNormalizer(torch.rand(H) + 0.1, torch.rand(I) + 0.1, bias_avg_sq=torch.rand(H) + 0.1),
                 "fc2": AdafactorNormalizer(torch.rand(O) + 0.1, torch.rand(H) + 0.1, bias_avg_sq=None)}
    x = torch.randn(N, S, I)
    c, grads = _collect(model, x, GradientProcessor(normalizers=norms, projection_dim=p, include_bias=True))
    shapes = c.shapes()
    assert set(grads) == {"fc1", "fc2"}
    for name, shape in shapes.items():
        assert grads[name].shape == (N, shape[0] * shape[1]), name
    if p is None:
        assert tuple(shapes["fc1"]) == (H, I + 1) and tuple(shapes["fc2"]) == (O, H)
        if kind == "none":
            truth = _truth(model, x)
            for n in range(N):
                torch.testing.assert_close(grads["fc1"][n].view(H, I + 1), truth[n]["fc1"], atol=1e-5, rtol=1e-5)
                torch.testing.assert_close(grads["fc2"][n].view(O, H), truth[n]["fc2"], atol=1e-5, rtol=1e-5)
        if kind == "adam":
            truth = _truth(model, x)
            w = truth[0]["fc1"][:, :I] / (norms["fc1"].weight_avg_sq.sqrt() + 1e-8)
            torch.testing.assert_close(grads["fc1"][0].view(H, I + 1)[:, :I], w, atol=1e-5, rtol=1e-4)
            b = truth[0]["fc1"][:, I] / (norms["fc1"].bias_avg_sq.sqrt() + 1e-8)
            torch.testing.assert_close(grads["fc1"][0].view(H, I + 1)[:, I], b, atol=1e-5, rtol=1e-4)
    else:
        assert tuple(shapes["fc1"]) == (p, p) and tuple(shapes["fc2"]) == (p, p)


def test_projected_bias_gradients_equal_projecting_the_full_gradient():
    torch.manual_seed(1)
    model = Mixed()
    x = torch.randn(N, S, I)
    p = 2
    _, grads = _collect(model, x, GradientProcessor(projection_dim=p, include_bias=True))
    truth = _truth(model, x)
    cpu = torch.device("cpu")
    for name, (o, i) in {"fc1": (H, I + 1), "fc2": (O, H)}.items():
        L = create_projection_matrix(f"{name}/left", p, o, torch.float32, cpu, "rademacher")
        R = create_projection_matrix(f"{name}/right", p, i, torch.float32, cpu, "rademacher")
        for n in range(N):
            torch.testing.assert_close(grads[name][n].view(p, p), L @ truth[n][name] @ R.T, atol=1e-5, rtol=1e-5)
