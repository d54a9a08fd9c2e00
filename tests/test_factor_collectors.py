"""Kronecker-factor collectors on small modules: bias-augmented activations, GPT-2 style
transposed layers, masked positions, and the row partition used for sharding."""

import math
import os

import pytest
import torch
import torch.nn as nn
from safetensors.torch import save_file

from bergson_b200.collector.collector import HookCollectorBase
from bergson_b200.gradients import GradientProcessor
from bergson_b200.hessians.eigenvectors import LambdaCollector
from bergson_b200.hessians.kfac import CovarianceCollector
from bergson_b200.hessians.sharded_computation import shard_bounds
from bergson_b200.models.common import Conv1D

I, O = 4, 6


class BiasModel(nn.Module):
    def __init__(self):
        super().__init__()
        self.biased = nn.Linear(I, O, bias=True)
        self.unbiased = nn.Linear(O, I, bias=False)

    def forward(self, x):
        return self.unbiased(self.biased(x))


class Conv1DModel(nn.Module):
    def __init__(self):
        super().__init__()
        self.conv = Conv1D(O, I)  # nf = outputs, nx = inputs; weight stored [in, out]
        self.linear = nn.Linear(O, I)

    def forward(self, x):
        return self.linear(self.conv(x))


def _run(collector, model, x, mask):
    with collector:
        with collector.with_batch(mask):
            model(x).sum().backward()


def test_bias_column_enters_the_activation_factor(tmp_path):
    torch.manual_seed(0)
    model = BiasModel()
    c = CovarianceCollector(model=model, dtype=torch.float32, path=str(tmp_path), processor=GradientProcessor(include_bias=True))
    n, s = 2, 3
    x = torch.randn(n, s, I)
    mask = torch.ones(n, s, dtype=torch.bool)
    mask[1, 2] = False  # a position that is not collected
    _run(c, model, x, mask)
    a = x[mask]
    aug = torch.cat([a, a.new_ones(len(a), 1)], dim=1)
    torch.testing.assert_close(c.A_full["biased"], aug.T @ aug)
    assert float(c.A_full["biased"][-1, -1]) == float(mask.sum())  # the bias-bias corner counts positions
    assert c.S_full["biased"].shape == (O, O) and c.A_full["unbiased"].shape == (O, O)
    # the factor sizes multiply to the size of the stored per-layer gradient [O, I + 1]
    assert c.S_full["biased"].shape[1] * c.A_full["biased"].shape[1] == math.prod(c.shapes()["biased"])
    h = model.biased(x)[mask]
    torch.testing.assert_close(c.A_full["unbiased"], h.T @ h, rtol=1e-5, atol=1e-5)


def test_eigenvalue_correction_has_the_stored_gradient_layout(tmp_path):
    model = BiasModel()
    os.makedirs(tmp_path / "eigen_activation_sharded")
    os.makedirs(tmp_path / "eigen_gradient_sharded")
    save_file({"biased": torch.eye(I + 1), "unbiased": torch.eye(O)}, str(tmp_path / "eigen_activation_sharded/shard_0.safetensors"))
    save_file({"biased": torch.eye(O), "unbiased": torch.eye(I)}, str(tmp_path / "eigen_gradient_sharded/shard_0.safetensors"))
    c = LambdaCollector(model=model, path=str(tmp_path), processor=GradientProcessor(include_bias=True))
    x = torch.randn(2, 3, I)
    _run(c, model, x, torch.ones(2, 3, dtype=torch.bool))
    lam = c.eigenvalue_corrections
    assert lam["biased"].shape == (O, I + 1) and lam["unbiased"].shape == (I, O)
    # identity eigenvectors: the correction is the sum over documents of squared per-document gradients
    g_out = model.unbiased.weight.sum(0)  # d(sum of outputs)/d(biased output), the same at every position
    aug = torch.cat([x, x.new_ones(2, 3, 1)], dim=-1)
    per_doc = torch.einsum("o,nsi->noi", g_out, aug)
    torch.testing.assert_close(lam["biased"], per_doc.square().sum(0), rtol=1e-4, atol=1e-5)


def test_transposed_layers_report_and_collect_out_by_in(tmp_path):
    torch.manual_seed(1)
    model = Conv1DModel()
    assert model.conv.weight.shape == (I, O)
    info = HookCollectorBase.discover_targets(model)
    assert info["conv"][1] == torch.Size([O, I]) and info["linear"][1] == torch.Size([I, O])
    c = CovarianceCollector(model=model, dtype=torch.float32, path=str(tmp_path))
    x = torch.randn(2, 3, I)
    mask = torch.ones(2, 3, dtype=torch.bool)
    _run(c, model, x, mask)
    a = x.reshape(-1, I)
    torch.testing.assert_close(c.A_full["conv"], a.T @ a)
    g = model.linear.weight.sum(0).expand(6, O)  # gradient of the sum w.r.t. the conv output, per position
    torch.testing.assert_close(c.S_full["conv"], g.T @ g, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("world", [1, 2, 3, 4, 7])
@pytest.mark.parametrize("dim", [1, 7, 64, 129, 513])
def test_shard_bounds_tile_the_rows(dim, world):
    if dim < world:
        pytest.skip("fewer rows than ranks")
    base, rem = divmod(dim, world)
    end = 0
    for rank in range(world):
        lo, hi = shard_bounds(dim, rank, world)
        assert lo == end and hi - lo == base + (rem if rank == 0 else 0)  # the first rank takes the remainder
        end = hi
    assert end == dim


def _two_batches(model, collector_cls, tmp_path, **kw):
    from safetensors.torch import load_file

    torch.manual_seed(3)
    c = collector_cls(model=model, dtype=torch.float32, path=str(tmp_path), **kw)
    xs = [torch.randn(2, 3, I), torch.randn(1, 4, I)]
    masks = [torch.ones(2, 3, dtype=torch.bool), torch.ones(1, 4, dtype=torch.bool)]
    masks[0][1, 2] = False
    acts, grads = [], []
    with c:
        for x, m in zip(xs, masks):
            with c.with_batch(m):
                model.zero_grad()
                model(x).sum().backward()
            acts.append(x[m])
            # d(sum of outputs)/d(biased output) is the same row at every position
            grads.append(model.unbiased.weight.sum(0).expand(int(m.sum()), O))
        c.teardown()
    A = load_file(str(tmp_path / "activation_sharded" / "shard_0.safetensors"))
    S = load_file(str(tmp_path / "gradient_sharded" / "shard_0.safetensors"))
    return acts, grads, A["biased"], S["biased"]


def test_trace_weighted_factors(tmp_path):
    """TKFAC: each batch's activation Gram is weighted by the trace of its gradient Gram and the
    other way round."""
    from bergson_b200.hessians.tkfac import TraceCovarianceCollector

    acts, grads, A, S = _two_batches(BiasModel(), TraceCovarianceCollector, tmp_path)
    want_a = sum((g * g).sum() * (a.T @ a) for a, g in zip(acts, grads))
    want_s = sum((a * a).sum() * (g.T @ g) for a, g in zip(acts, grads))
    torch.testing.assert_close(A, want_a, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(S, want_s, rtol=1e-4, atol=1e-5)


def test_shampoo_factors_are_built_from_batch_gradients(tmp_path):
    """Shampoo: M = g^T a per batch, A += M^T M, S += M M^T, and A is scaled to unit trace at the end."""
    from bergson_b200.hessians.shampoo import ShampooCollector

    acts, grads, A, S = _two_batches(BiasModel(), ShampooCollector, tmp_path)
    ms = [g.T @ a for a, g in zip(acts, grads)]
    want_a = sum(m.T @ m for m in ms)
    want_s = sum(m @ m.T for m in ms)
    torch.testing.assert_close(A, want_a / want_a.trace(), rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(S, want_s, rtol=1e-4, atol=1e-5)
    assert float(A.trace()) == pytest.approx(1.0, rel=1e-5)
