"""MAGIC's in-place training step on the GPU: the multi-tensor AdamW kernel and the fused
global-norm clipping coefficient against fp32 PyTorch, and the trainer taking that path; the traced step and its VJP kernel."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def native():
    from bergson_b200.ops import native

    assert native.available()
    return native


def _adamw_reference(p, m, v, g, lr, b1, b2, eps, eps_root, wd, step, coef=1.0):
    g = g.float() * coef
    m = b1 * m + (1 - b1) * g
    v = b2 * v + (1 - b2) * g * g
    upd = (m / (1 - b1**step)) / ((v / (1 - b2**step) + eps_root).sqrt() + eps) + wd * p.float()
    return p.float() - lr * upd, m, v


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_adamw_multi_matches_fp32_reference(native, dtype):
    torch.manual_seed(0)
    # Aligned and ragged sizes, a scalar-like tensor, and an offset view whose address is not
    # a multiple of 16 bytes (all in one launch).
    sizes = [4096 * 33, 1000, 7, 1, 128 * 1024 + 4]
    ps = [torch.randn(n, device="cuda").to(dtype) for n in sizes]
    base = torch.randn(1025, device="cuda").to(dtype)
    ps.append(base[1:])
    first = base[0].clone()
    gs = [torch.randn_like(p) for p in ps[:-1]] + [torch.randn(1025, device="cuda").to(dtype)[1:]]
    ms = [torch.randn(p.numel(), device="cuda") * 0.1 for p in ps]
    vs = [torch.rand(p.numel(), device="cuda") * 0.1 for p in ps]
    coef = torch.tensor([0.37], device="cuda")
    hp = dict(lr=1e-2, b1=0.9, b2=0.95, eps=1e-8, eps_root=1e-12, wd=0.1)
    for step in (1, 2):
        want = [_adamw_reference(p, m, v, g, step=step, coef=0.37, **hp) for p, m, v, g in zip(ps, ms, vs, gs)]
        native.adamw_multi(ps, ms, vs, gs, hp["lr"], hp["b1"], hp["b2"], hp["eps"], hp["eps_root"], hp["wd"], step,
                           1.0, coef)
        for (p_ref, m_ref, v_ref), p, m, v in zip(want, ps, ms, vs):
            torch.testing.assert_close(m, m_ref, atol=1e-6, rtol=1e-5)
            torch.testing.assert_close(v, v_ref, atol=1e-6, rtol=1e-5)
            if dtype == torch.float32:
                torch.testing.assert_close(p, p_ref, atol=1e-6, rtol=1e-5)
            else:  # one rounding of the fp32 result to the 16-bit type
                torch.testing.assert_close(p, p_ref.to(dtype), atol=1e-6, rtol=2**-7)
    assert torch.equal(base[0], first)  # the element before the offset view is left alone


def test_multi_sumsq_and_clip_coefficient(native):
    torch.manual_seed(1)
    xs = [torch.randn(n, device="cuda", dtype=torch.bfloat16) for n in (5, 4096 * 17, 1, 333)]
    out = torch.zeros(2, device="cuda")
    native.multi_sumsq(xs, out, False, 1.5)
    sq = sum(x.float().pow(2).sum() for x in xs)
    torch.testing.assert_close(out[0], sq, rtol=1e-5, atol=0)
    torch.testing.assert_close(out[1], (1.5 / (sq.sqrt() + 1e-6)).clamp(max=1.0), rtol=1e-5, atol=0)
    again = torch.zeros(2, device="cuda")
    native.multi_sumsq(xs, again, False, 1.5)
    assert torch.equal(out, again)  # fixed summation order
    native.multi_sumsq(xs, again, True, 0.0)
    torch.testing.assert_close(again[0], 2 * sq, rtol=1e-5, atol=0)
    small = [torch.full((4,), 0.1, device="cuda")]
    native.multi_sumsq(small, out, False, 10.0)
    assert out[1].item() == 1.0  # no clipping below the threshold


def _tiny_trainer(max_grad_norm):
    from bergson_b200.magic import optim
    from bergson_b200.magic.data_stream import DataStream
    from bergson_b200.magic.trainer import Trainer

    from .helpers import tiny_dataset, tiny_model

    torch.manual_seed(0)
    model = tiny_model("llama", dtype=torch.float32, num_hidden_layers=2).to("cuda")
    model.requires_grad_(True)
    model.eval()
    opt = optim.adamw(lambda i: 1e-3 * (1 + i), betas=(0.9, 0.95), weight_decay=0.01)
    trainer, state = Trainer.initialize(model, opt)
    data = DataStream(tiny_dataset(n=8, length=16, ragged=False), 4, device="cuda")
    with torch.no_grad():
        batch = {k: (v.detach() if isinstance(v, torch.Tensor) else v) for k, v in data[0].items()}
    return trainer, state, batch, max_grad_norm


@pytest.mark.parametrize("max_grad_norm", [None, 0.05])
def test_trainer_inplace_step_uses_the_fused_kernel_and_matches_functional(monkeypatch, native, max_grad_norm):
    from bergson_b200.magic import optim

    trainer, state, batch, clip = _tiny_trainer(max_grad_norm)
    want = state.to("cuda")
    calls = []
    real = native.adamw_multi
    monkeypatch.setattr(native, "adamw_multi", lambda *a, **k: (calls.append(len(a[0])), real(*a, **k))[1])
    for _ in range(3):
        state = trainer.step(state, batch, inplace=True, max_grad_norm=clip)
        want = trainer.step(want, batch, inplace=False, max_grad_norm=clip)
    assert len(calls) == 3 and calls[0] == len(state.params)
    assert int(state.opt_state["count"]) == 3 and state.opt_state["count"].device.type == "cpu"
    for k in state.params:
        torch.testing.assert_close(state.params[k], want.params[k], atol=2e-6, rtol=1e-4)
        torch.testing.assert_close(state.opt_state["nu"][k], want.opt_state["nu"][k], atol=1e-10, rtol=1e-4)
    assert optim.global_norm_coef([torch.ones(3)], 1.0) is None  # CPU tensors: not eligible


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_traced_adamw_step_and_its_vjp_match_autograd(native, dtype):
    """The one-launch traced step and its hand-written VJP against the same update written
    with differentiable torch operations (fp64 autograd)."""
    from bergson_b200.magic import optim

    torch.manual_seed(0)
    shapes = {"a": (33, 17), "b": (129,), "c": (4, 4, 8)}
    params = {k: torch.randn(s, device="cuda").to(dtype) for k, s in shapes.items()}
    grads = {k: (torch.randn(s, device="cuda") * 0.1).to(dtype) for k, s in shapes.items()}
    opt = optim.adamw(lambda i: 1e-2, betas=(0.9, 0.95), eps=1e-8, eps_root=1e-8, weight_decay=0.1)
    state = opt.init(params)
    for k in shapes:  # non-trivial moments, third step
        state["mu"][k] = torch.randn(shapes[k], device="cuda") * 0.05
        state["nu"][k] = torch.rand(shapes[k], device="cuda") * 0.01
    state["count"] = torch.tensor(2)

    def run(ps, gs, mus, nus, fused):
        st = {"mu": mus, "nu": nus, "count": state["count"]}
        if fused:
            new_p, new_s = opt.step_traced(gs, st, ps)
        else:
            upd, new_s = opt.update(gs, st, params=ps, inplace=False)
            new_p = optim.apply_updates(ps, upd)
        return new_p, new_s

    leaves = [{k: v.clone().requires_grad_(True) for k, v in d.items()} for d in (params, grads, state["mu"], state["nu"])]
    new_p, new_s = run(*leaves, fused=True)
    assert new_p["a"].grad_fn is not None and type(new_p["a"].grad_fn).__name__.startswith("_AdamWStepFn")
    ref_leaves = [{k: v.double().requires_grad_(True) for k, v in d.items()} for d in (params, grads, state["mu"], state["nu"])]
    ref_p, ref_s = run(*ref_leaves, fused=False)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    for k in shapes:
        torch.testing.assert_close(new_p[k].double(), ref_p[k], atol=tol, rtol=tol)
        torch.testing.assert_close(new_s["nu"][k].double(), ref_s["nu"][k], atol=1e-6, rtol=1e-5)

    def vjp(new_p, new_s, leaves, cast):
        outs = [new_p[k] for k in shapes] + [new_s["mu"][k] for k in shapes] + [new_s["nu"][k] for k in shapes]
        gen = torch.Generator(device="cuda").manual_seed(1)
        cots = [torch.randn(o.shape, device="cuda", generator=gen).to(cast(o)) for o in outs]
        ins = [d[k] for d in leaves for k in shapes]
        return torch.autograd.grad(outs, ins, grad_outputs=cots)

    got = vjp(new_p, new_s, leaves, lambda o: o.dtype)
    want = vjp(ref_p, ref_s, ref_leaves, lambda o: torch.float64)
    for g, w in zip(got, want):
        scale = w.abs().max().item() + 1e-12
        assert (g.double() - w).abs().max().item() <= (1e-4 if dtype == torch.float32 else 3e-2) * scale


@pytest.mark.parametrize("shape", [(256, 96), (64, 320)])
def test_newton_schulz_on_the_gemm_kernel_matches_torch(native, shape):
    from bergson_b200.magic import optim

    torch.manual_seed(0)
    g = torch.randn(shape, device="cuda").to(torch.bfloat16).requires_grad_(True)
    out = optim.zeropower_via_newtonschulz(g)
    assert out.shape == g.shape and type(out.grad_fn).__name__ != "AddmmBackward0"
    g64 = g.detach().double().requires_grad_(True)
    ref = optim.zeropower_via_newtonschulz(g64)  # CPU-style path in fp64 (dtype not 16-bit)
    assert (out.double() - ref).abs().max() <= 6e-2 * ref.abs().max()
    # Singular values are pushed towards 1 (the iteration's purpose).
    sv = torch.linalg.svdvals(out.float())
    assert sv.min() > 0.3 and sv.max() < 1.6
    # First derivative through the kernel path.
    probe = torch.randn(shape, device="cuda")
    (gg,) = torch.autograd.grad((out.float() * probe).sum(), g)
    (gr,) = torch.autograd.grad((ref * probe.double()).sum(), g64)
    assert torch.nn.functional.cosine_similarity(gg.double().flatten(), gr.flatten(), dim=0) > 0.98


@pytest.mark.parametrize("family", ["gpt2", "llama"])
def test_meta_step_on_kernels_matches_cpu_fp64(native, family):
    """One traced step plus its VJP (the metagradient building block) on the GPU in fp32, where
    GEMMs, LayerNorm, GELU, softmax, cross-entropy and AdamW run on kernels to second order,
    against the same computation on the CPU in fp64."""
    from bergson_b200.magic import optim
    from bergson_b200.magic.data_stream import DataStream
    from bergson_b200.magic.trainer import Trainer

    from .helpers import tiny_dataset, tiny_model

    def run(device, dtype):
        torch.manual_seed(0)
        model = tiny_model(family, dtype=dtype, num_hidden_layers=2, hidden_size=64, intermediate_size=128,
                           num_attention_heads=4, vocab_size=128).to(device)
        model.requires_grad_(True)
        model.eval()
        opt = optim.adamw(lambda i: 1e-2, betas=(0.9, 0.95), eps_root=1e-8, weight_decay=0.01)
        trainer, state = Trainer.initialize(model, opt)
        data = DataStream(tiny_dataset(n=8, length=16, ragged=False), 4, device=device)
        data.weights.data = data.weights.data.to(dtype)
        state = trainer.step(state, data[0], inplace=False)  # non-trivial moments
        state.detach_()
        state.requires_grad = True
        data.requires_grad = True
        before = state.differentiable_tensors()
        after = trainer.step(state, data[1], trace=True).differentiable_tensors()
        gen = torch.Generator().manual_seed(1)
        cot = [torch.randn(t.shape, generator=gen).to(device, t.dtype) * 1e-2 for t in after]
        grads = torch.autograd.grad(after, before + [data.weights], grad_outputs=cot, allow_unused=True)
        return [None if g is None else g.detach().double().cpu() for g in grads]

    got = run("cuda", torch.float32)
    want = run("cpu", torch.float64)
    assert len(got) == len(want)
    for g, w in zip(got, want):
        assert (g is None) == (w is None)
        if w is not None and w.abs().max() > 0:
            assert (g - w).abs().max() <= 2e-3 * w.abs().max() + 1e-9
    assert want[-1].abs().max() > 0  # the data-weight gradient is not trivially zero


def test_padded_vocabulary_head_loss_matches_plain_path(native):
    """A vocabulary that is not a multiple of 8: the head's GEMM and the loss run on the padded
    width; loss, logits and gradients must equal the unpadded torch computation."""
    from .helpers import tiny_model

    torch.manual_seed(0)
    model = tiny_model("gpt2", dtype=torch.bfloat16, num_hidden_layers=1, vocab_size=131).to("cuda")
    model.eval()
    x = torch.randint(0, 131, (3, 24), device="cuda")
    w = torch.rand(3, device="cuda")
    out = model(input_ids=x, labels=x, example_weight=w)
    assert out.logits.shape == (3, 24, 131) and out.logits.stride(-2) == 136  # view of the padded rows
    h = model.hidden(x)
    logits = (h.float() @ model.get_output_embeddings().weight.float().T)
    tok = torch.nn.functional.cross_entropy(logits[:, :-1].reshape(-1, 131), x[:, 1:].reshape(-1), reduction="none")
    want = (tok.view(3, 23) * w[:, None]).sum() / (3 * 23)
    torch.testing.assert_close(out.loss.float(), want, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(out.logits.float(), logits, rtol=5e-2, atol=5e-2)
    (g,) = torch.autograd.grad(out.loss, model.get_output_embeddings().weight)
    (g_ref,) = torch.autograd.grad(want, model.get_output_embeddings().weight)
    assert g.shape == g_ref.shape
    assert torch.nn.functional.cosine_similarity(g.float().flatten(), g_ref.float().flatten(), dim=0) > 0.99
