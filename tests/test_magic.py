"""MAGIC trainer: metagradients against finite differences, checkpoint-schedule
invariance, micro-batched VJP == single-shot VJP, optimizers."""

import math
import os

import pytest
import torch

from bergson_b200.magic import optim
from bergson_b200.magic.data_stream import DataStream, pad_dataset_to_batch_size
from bergson_b200.magic.trainer import BackwardState, Trainer, next_save_index

from .helpers import tiny_dataset, tiny_model


def _setup(family="llama", opt="adamw", dtype=torch.float64, n=8, bs=2):
    torch.manual_seed(0)
    model = tiny_model(family, dtype=dtype, num_hidden_layers=1)
    model.requires_grad_(True)
    model.eval()
    ds = tiny_dataset(n=n, length=8, ragged=False)
    data = DataStream(ds, bs)
    data.weights.data = data.weights.data.to(dtype)
    sched = lambda s: 5e-3  # noqa: E731
    make = {"adamw": lambda: optim.adamw(sched, betas=(0.95, 0.975), eps_root=1e-8, weight_decay=0.01),
            "sgd": lambda: optim.sgd(sched, momentum=0.9, weight_decay=0.01),
            "muon": lambda: optim.muon(sched, momentum=0.95, weight_decay=0.0, adamw_betas=(0.95, 0.975), adamw_eps_root=1e-8)}[opt]
    trainer, state = Trainer.initialize(model, make())
    return trainer, state, data, ds


def _query_loss(trainer, state, ds):
    x = torch.tensor(ds["input_ids"][:3])
    return trainer.call_model({k: v for k, v in state.params.items()}, {"input_ids": x, "labels": x}, state.buffers).loss


def _scores(trainer, state0, data, ds, tmp, save_mode="all", **kw):
    final = trainer.train(state0.to("cpu"), data, save_dir=str(tmp), save_mode=save_mode, **{k: v for k, v in kw.items() if k != "double_backward_batch_size"})
    params = {k: v.detach().requires_grad_(True) for k, v in final.params.items()}
    x = torch.tensor(ds["input_ids"][:3])
    loss = trainer.call_model(params, {"input_ids": x, "labels": x}, final.buffers).loss
    g = torch.autograd.grad(loss, list(params.values()))
    n_opt = len(final.differentiable_tensors()) - len(params)
    opt_zero = [torch.zeros_like(t) for t in final.differentiable_tensors()[len(params):]]
    assert len(opt_zero) == n_opt
    bwd = BackwardState(dict(zip(params, g)), opt_zero, torch.zeros_like(data.weights))
    out = trainer.backward(str(tmp), data, bwd, final, save_mode=save_mode, **kw)
    return out.weight_grads.detach().clone(), float(loss)


@pytest.mark.parametrize("opt", ["adamw", "sgd", "muon"])
def test_metagradient_matches_finite_differences(tmp_path, opt):
    trainer, state0, data, ds = _setup(opt=opt)
    scores, base = _scores(trainer, state0, data, ds, tmp_path / "a")
    assert scores.abs().max() > 0
    h = 1e-4
    for i in (0, 3, 6):
        losses = []
        for sign in (+1, -1):
            data.weights.data.fill_(1.0)
            data.weights.data[i] += sign * h
            final = trainer.train(state0.to("cpu"), data)
            losses.append(float(_query_loss(trainer, final, ds)))
        data.weights.data.fill_(1.0)
        fd = (losses[0] - losses[1]) / (2 * h)
        assert math.isclose(fd, float(scores[i]), rel_tol=2e-3, abs_tol=1e-7), (i, fd, float(scores[i]))


def test_save_modes_give_identical_scores(tmp_path):
    trainer, state0, data, ds = _setup(n=18, bs=2)
    ref, _ = _scores(trainer, state0, data, ds, tmp_path / "all", "all")
    for mode in ("sqrt", "log"):
        got, _ = _scores(trainer, state0, data, ds, tmp_path / mode, mode)
        torch.testing.assert_close(got, ref, atol=1e-12, rtol=1e-6)


def test_micro_vjp_equals_single_shot(tmp_path):
    trainer, state0, data, ds = _setup(n=8, bs=4)
    ref, _ = _scores(trainer, state0, data, ds, tmp_path / "one")
    got, _ = _scores(trainer, state0, data, ds, tmp_path / "acc", grad_accum_steps=2)
    torch.testing.assert_close(got, ref, atol=1e-10, rtol=1e-6)
    got2, _ = _scores(trainer, state0, data, ds, tmp_path / "acc2", grad_accum_steps=2, double_backward_batch_size=1)
    torch.testing.assert_close(got2, ref, atol=1e-10, rtol=1e-6)


def test_grad_clipping_is_differentiable(tmp_path):
    trainer, state0, data, ds = _setup()
    scores, _ = _scores(trainer, state0, data, ds, tmp_path / "c", max_grad_norm=0.05)
    h = 1e-4
    losses = []
    for sign in (+1, -1):
        data.weights.data.fill_(1.0)
        data.weights.data[1] += sign * h
        final = trainer.train(state0.to("cpu"), data, max_grad_norm=0.05)
        losses.append(float(_query_loss(trainer, final, ds)))
    data.weights.data.fill_(1.0)
    fd = (losses[0] - losses[1]) / (2 * h)
    assert math.isclose(fd, float(scores[1]), rel_tol=0.05, abs_tol=1e-6)


def test_resume_continues_the_schedule(tmp_path):
    trainer, state0, data, ds = _setup(n=12, bs=2)
    full = trainer.train(state0.to("cpu"), data, save_dir=str(tmp_path / "full"), save_mode="all")
    # interrupted run: only the first 3 checkpoints exist, plus an incomplete one
    part = tmp_path / "part"
    short = DataStream(ds.select(range(8)), 2)
    short.weights.data = short.weights.data.double()
    trainer.train(state0.to("cpu"), short, save_dir=str(part), save_mode="all")
    os.makedirs(part / "step_9.ckpt")
    resumed = trainer.train(state0.to("cpu"), data, save_dir=str(part), save_mode="all", resume=True)
    assert not (part / "step_9.ckpt").exists()  # the checkpoint without a .metadata marker was discarded
    for k in full.params:
        torch.testing.assert_close(resumed.params[k], full.params[k], atol=1e-12, rtol=1e-9)


def test_next_save_index_schedules():
    n = 16
    for mode in ("all", "sqrt", "log"):
        idx, seen = 0, [0]
        while idx < n:
            idx = next_save_index(idx, n, mode)
            assert idx > seen[-1]
            seen.append(idx)
    assert next_save_index(0, 16, "sqrt") == 4 and next_save_index(12, 16, "sqrt") == 13
    assert next_save_index(0, 16, "log") == 8 and next_save_index(8, 16, "log") == 12
    assert next_save_index(0, 16, "interval", 5) == 5
    with pytest.raises(ValueError):
        next_save_index(0, 16, "interval", 0)


def test_muon_matches_torch_optim():
    if not hasattr(torch.optim, "Muon"):
        pytest.skip("torch.optim.Muon unavailable")
    torch.manual_seed(0)
    w = torch.randn(6, 4)
    g = torch.randn(6, 4)
    ref_p = torch.nn.Parameter(w.clone())
    ref = torch.optim.Muon([ref_p], lr=0.1, momentum=0.95, weight_decay=0.0, adjust_lr_fn="match_rms_adamw")
    ours = optim.muon(0.1, momentum=0.95, weight_decay=0.0)
    params = {"w": w.clone()}
    state = ours.init(params)
    for _ in range(3):
        ref_p.grad = g.clone()
        ref.step()
        upd, state = ours.update({"w": g}, state, params=params)
        params = optim.apply_updates(params, upd)
    torch.testing.assert_close(params["w"], ref_p.data, atol=1e-3, rtol=1e-3)


def test_adamw_matches_torch_optim():
    torch.manual_seed(0)
    w, g = torch.randn(5, 3, dtype=torch.float64), torch.randn(5, 3, dtype=torch.float64)
    ref_p = torch.nn.Parameter(w.clone())
    ref = torch.optim.AdamW([ref_p], lr=0.01, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.1)
    ours = optim.adamw(0.01, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.1)
    params = {"w": w.clone()}
    state = ours.init(params)
    for _ in range(4):
        ref_p.grad = g.clone()
        ref.step()
        upd, state = ours.update({"w": g}, state, params=params)
        params = optim.apply_updates(params, upd)
    torch.testing.assert_close(params["w"], ref_p.data, atol=1e-9, rtol=1e-7)


def test_pad_dataset_to_batch_size():
    ds = tiny_dataset(n=5, length=6, ragged=False)
    out, num_docs, pad, wpad = pad_dataset_to_batch_size(ds, 4, 5, "train", 1)
    assert len(out) == 8 and pad == 3 and wpad == 3 and num_docs == 8


def test_lazy_gather_matches_functional_call_to_second_order():
    """Per-module gathering with re-gathering in the backward pass gives the same loss, the
    same gradients and the same gradient-of-gradient as handing the model all parameters."""
    from torch.func import functional_call

    from bergson_b200.magic.fsdp import LazyGather

    torch.manual_seed(0)
    model = tiny_model("gpt2", dtype=torch.float64, num_hidden_layers=2)
    model.eval()
    params = {k: v.detach().clone().requires_grad_(True) for k, v in model.named_parameters()}
    shapes = {k: v.shape for k, v in params.items()}
    x = torch.randint(0, 128, (3, 9))

    def second_order(loss, ps):
        grads = torch.autograd.grad(loss, ps, create_graph=True)
        inner = sum((g * g).sum() for g in grads)
        return grads, torch.autograd.grad(inner, ps, allow_unused=True)

    plist = list(params.values())
    want_loss = functional_call(model, params, args=(), kwargs={"input_ids": x, "labels": x}).loss
    want_g, want_gg = second_order(want_loss, plist)
    with LazyGather(model, params, shapes) as lazy:
        got_loss = model(input_ids=x, labels=x).loss
    assert lazy.packed > 0 and lazy.gathers >= len(shapes)  # tied embeddings are gathered per use
    got_g, got_gg = second_order(got_loss, plist)
    assert lazy.gathers > len(shapes) + 1  # the backward pass gathered again
    torch.testing.assert_close(got_loss, want_loss)
    for a, b in zip(got_g, want_g):
        torch.testing.assert_close(a, b)
    for a, b in zip(got_gg, want_gg):
        if b is None:
            assert a is None
        else:
            torch.testing.assert_close(a, b, rtol=1e-6, atol=1e-9)
    # The module's own parameters are back in place.
    assert all(isinstance(p, torch.nn.Parameter) for p in model.parameters())


def test_state_activation_swaps_parameters_and_random_streams():
    trainer, state, data, ds = _setup(n=4, bs=2)
    model = trainer.model
    own = {k: p.detach().clone() for k, p in model.named_parameters()}
    shifted = state.to("cpu")
    for p in shifted.params.values():
        p.add_(0.5)
    shifted.params = {k: p.requires_grad_(True) for k, p in shifted.params.items()}
    x = torch.tensor(ds["input_ids"][:2])
    before = torch.random.get_rng_state()
    with shifted.activate(model) as params:
        assert set(params) == set(shifted.params)
        loss = model(x, labels=x).loss
        grads = torch.autograd.grad(loss, list(params.values()), allow_unused=True)
        assert any(g is not None and g.abs().sum() > 0 for g in grads)  # gradients reach the state's tensors
        assert torch.equal(torch.random.get_rng_state(), shifted.cpu_rng_state)
        torch.rand(3)  # consuming randomness inside must not leak out
    assert torch.equal(torch.random.get_rng_state(), before)
    for k, p in model.named_parameters():
        assert torch.equal(p, own[k]) and isinstance(p, torch.nn.Parameter)
    plain = model(x, labels=x).loss
    assert not torch.allclose(plain, loss.detach().to(plain.dtype))
    with pytest.raises(KeyError):
        partial = shifted.to("cpu")
        partial.params.pop(next(iter(partial.params)))
        with partial.activate(model):
            pass


def test_muon_argument_checks():
    with pytest.raises(ValueError, match="Nesterov"):
        optim.muon(0.1, momentum=0.0)
    with pytest.raises(ValueError, match="Nesterov"):
        optim.muon(0.1, dampening=0.1)
    with pytest.raises(ValueError, match="weight_decay"):
        optim.muon(0.1, weight_decay=-1.0)
    with pytest.raises(ValueError, match="2 dimensions"):
        optim.muon(0.1).init({"conv": torch.zeros(2, 3, 4)})
    st = optim.muon(0.1, moment_requires_grad=True).init({"w": torch.zeros(3, 2), "b": torch.zeros(3)})
    assert st["trace"]["w"].requires_grad and set(st["mu"]) == {"b"}


@pytest.mark.parametrize("weight_decay", [0.0, 0.1])
@pytest.mark.parametrize("eps_root", [0.0, 1e-6])
def test_muon_updates_vectors_like_adamw(weight_decay, eps_root):
    """Muon orthogonalises matrices only; 1-D parameters take the AdamW step with the same
    hyper-parameters (and torch's AdamW when eps_root is 0)."""
    torch.manual_seed(0)
    b0 = torch.randn(8)
    X, Y = torch.randn(16, 8), torch.randn(16)
    kw = dict(betas=(0.9, 0.999), eps=1e-8, eps_root=eps_root, weight_decay=weight_decay)
    ref_opt = optim.adamw(0.01, **kw)
    mu_opt = optim.muon(0.01, weight_decay=weight_decay, adamw_betas=(0.9, 0.999), adamw_eps=1e-8, adamw_eps_root=eps_root)
    ref, mu = {"b": b0.clone()}, {"b": b0.clone()}
    ref_state, mu_state = ref_opt.init(ref), mu_opt.init(mu)
    torch_b = torch.nn.Parameter(b0.clone())
    torch_opt = torch.optim.AdamW([torch_b], lr=0.01, betas=(0.9, 0.999), eps=1e-8, weight_decay=weight_decay)
    for _ in range(10):
        for params, opt, name in ((ref, ref_opt, "ref"), (mu, mu_opt, "mu")):
            b = params["b"].detach().requires_grad_(True)
            (X @ b - Y).pow(2).mean().backward()
            state = ref_state if name == "ref" else mu_state
            upd, state = opt.update({"b": b.grad}, state, params={"b": b})
            params["b"] = optim.apply_updates({"b": b.detach()}, upd)["b"]
            if name == "ref":
                ref_state = state
            else:
                mu_state = state
        torch_opt.zero_grad()
        (X @ torch_b - Y).pow(2).mean().backward()
        torch_opt.step()
    torch.testing.assert_close(mu["b"], ref["b"], atol=1e-6, rtol=0)
    if eps_root == 0.0:
        torch.testing.assert_close(mu["b"], torch_b.data, atol=1e-5, rtol=0)


def test_muon_mixed_shapes():
    torch.manual_seed(1)
    params = {"W": torch.randn(4, 4), "b": torch.randn(4)}
    opt = optim.muon(0.01)
    state = opt.init(params)
    upd, state = opt.update({k: torch.randn_like(v) for k, v in params.items()}, state, params=params)
    assert upd["W"].shape == (4, 4) and upd["b"].shape == (4,) and int(state["count"]) == 1
    # the matrix update has (nearly) orthonormal direction: equal singular values
    sv = torch.linalg.svdvals(upd["W"] + 0.01 * 0.1 * params["W"])  # take the weight-decay term back out
    assert float(sv.max() / sv.min()) < 2.5
