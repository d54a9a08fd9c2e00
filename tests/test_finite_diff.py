"""Finite differences along the gradients of a backward pass: exact restoration, double swap,
normalisers, and the effect of one example's gradient step on another example's loss."""

import pytest
import torch
import torch.nn as nn

from bergson_b200 import FiniteDiff
from bergson_b200.gradients import AdamNormalizer
from bergson_b200.utils.gradcheck import compute_effect

from .helpers import tiny_model


def _model():
    return nn.Sequential(nn.Linear(5, 3, bias=False), nn.Linear(3, 4, bias=False))


def _backward(model, n=7):
    model.zero_grad(set_to_none=True)
    (model(torch.randn(n, 5)) ** 2).mean().backward()


@pytest.mark.parametrize("step", [0.05, -0.05])
def test_store_apply_restore(step):
    torch.manual_seed(0)
    model = _model()
    fd = FiniteDiff(model)
    _backward(model)
    grads = {n: p.grad.detach().clone() for n, p in model.named_parameters()}
    orig = {n: p.detach().clone() for n, p in model.named_parameters()}
    fd.store(step)
    for n, p in model.named_parameters():
        assert torch.equal(p, orig[n]) and p.grad is None  # nothing moved yet, gradient buffers were taken over
    with fd.apply():
        for n, p in model.named_parameters():
            torch.testing.assert_close(p, orig[n] + step * grads[n])
    for n, p in model.named_parameters():
        assert torch.equal(p, orig[n])  # bit for bit
    fd.swap()
    fd.swap()
    for n, p in model.named_parameters():
        assert torch.equal(p, orig[n])
    fd.clear()
    assert fd.params == {}


def test_normalisers_are_applied_and_counted():
    torch.manual_seed(1)
    model = _model()
    _backward(model)
    g0 = model[0].weight.grad.detach().clone()
    orig = model[0].weight.detach().clone()
    fd = FiniteDiff(model, normalizers={"0": AdamNormalizer(torch.full((3, 5), 4.0))})
    fd.store(0.1)
    with fd.apply():
        torch.testing.assert_close(model[0].weight, orig + 0.1 * g0 / 2, atol=1e-6, rtol=1e-5)  # sqrt(4) = 2
    _backward(model)
    with pytest.raises(ValueError, match="normalized gradients"):
        FiniteDiff(model, normalizers={"not_a_module": AdamNormalizer(torch.ones(3, 5))}).store(0.1)


def test_effect_of_an_example_on_itself_is_a_descent():
    torch.manual_seed(2)
    model = tiny_model("llama", dtype=torch.float64)
    model.requires_grad_(True)
    before = {n: p.detach().clone() for n, p in model.named_parameters()}
    x = torch.randint(0, 128, (1, 10))
    y = torch.randint(0, 128, (1, 10))
    own = compute_effect(model, x, x, eps=-1e-4)  # a step against the gradient of x lowers the loss on x
    assert float(own) > 0  # (after - before) / eps with eps < 0 and after < before
    other = compute_effect(model, x, y, eps=-1e-4)
    assert abs(float(other)) < abs(float(own))
    for n, p in model.named_parameters():
        assert torch.equal(p, before[n]) and p.grad is None
