"""The stand-in packages under ``baseline/shims`` that let the unmodified reference run
offline: the functional optimizers must agree with ``torch.optim`` step for step and stay
differentiable."""

import sys
from pathlib import Path

import pytest
import torch

SHIMS = str(Path(__file__).resolve().parents[1] / "baseline" / "shims")


@pytest.fixture()
def torchopt():
    sys.path.insert(0, SHIMS)
    try:
        import torchopt as mod

        yield mod
    finally:
        sys.path.remove(SHIMS)


def _params():
    torch.manual_seed(0)
    return {"w": torch.randn(4, 3, dtype=torch.float64), "b": torch.randn(3, dtype=torch.float64)}


@pytest.mark.parametrize("inplace", [False, True])
def test_adamw_stand_in_matches_torch_optim(torchopt, inplace):
    p = _params()
    ref = [torch.nn.Parameter(v.clone()) for v in p.values()]
    o = torch.optim.AdamW(ref, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    opt = torchopt.adamw(lambda c: 1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    state = opt.init(p)
    for _ in range(4):
        g = {k: torch.randn_like(v) for k, v in p.items()}
        for r, gg in zip(ref, g.values()):
            r.grad = gg.clone()
        o.step()
        u, state = opt.update(g, state, params=p, inplace=inplace)
        p = torchopt.apply_updates(p, u, inplace=inplace)
    for r, v in zip(ref, p.values()):
        torch.testing.assert_close(v, r.detach(), atol=1e-7, rtol=1e-6)


def test_sgd_stand_in_matches_torch_optim(torchopt):
    p = _params()
    ref = [torch.nn.Parameter(v.clone()) for v in p.values()]
    o = torch.optim.SGD(ref, lr=1e-2, momentum=0.9, weight_decay=0.1)
    opt = torchopt.sgd(1e-2, momentum=0.9, weight_decay=0.1)
    state = opt.init(p)
    for _ in range(4):
        g = {k: torch.randn_like(v) for k, v in p.items()}
        for r, gg in zip(ref, g.values()):
            r.grad = gg.clone()
        o.step()
        u, state = opt.update(g, state, params=p, inplace=False)
        p = torchopt.apply_updates(p, u, inplace=False)
    for r, v in zip(ref, p.values()):
        torch.testing.assert_close(v, r.detach(), atol=1e-12, rtol=1e-10)


def test_update_is_differentiable_and_pytree_paths(torchopt):
    p = {k: v.requires_grad_(True) for k, v in _params().items()}
    opt = torchopt.adamw(1e-2, eps_root=1e-8)
    state = opt.init(p)
    g = {k: (v * v).sum() * torch.ones_like(v) for k, v in p.items()}
    u, state = opt.update(g, state, params=p, inplace=False)
    new = torchopt.apply_updates(p, u, inplace=False)
    (grad,) = torch.autograd.grad(new["w"].sum(), p["w"])
    assert torch.isfinite(grad).all() and grad.abs().sum() > 0
    paths, leaves, _ = torchopt.pytree.tree_flatten_with_path(state)
    assert len(paths) == len(leaves) == len(list(torchopt.pytree.tree_iter(state)))
    assert (0, 0, "b") in paths and (0, 0, "w") in paths  # mu of scale_by_adam, dict keys sorted
    moved = torchopt.pytree.tree_map(lambda t: t.clone(), state)
    assert type(moved[0]).__name__ == "ScaleByAdamState"
