"""Each sm_100a kernel against a plain PyTorch fp32 expression of the same op."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def native():
    from bergson_b200.ops import native as n

    assert n.available()
    return n


def _status_ok(native):
    torch.cuda.synchronize()
    assert int(native.kernel_status(0).item()) == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("T,K", [(128, 64), (300, 136), (1024, 768), (4099, 4096)])
def test_proj_right(native, dtype, T, K):
    torch.manual_seed(0)
    a = torch.randn(T, K, device="cuda", dtype=dtype)
    p = (torch.randn(16, K, device="cuda") / 4).to(dtype)
    out = native.proj_right(a, p)
    ref = a.float() @ p.float().T
    _status_ok(native)
    torch.testing.assert_close(out, ref, atol=2e-2 * (K / 64) ** 0.5, rtol=1e-2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("N,S,K", [(1, 128, 64), (3, 77, 72), (2, 300, 512), (4, 1024, 3072)])
def test_proj_left_outer(native, dtype, N, S, K):
    torch.manual_seed(1)
    g = torch.randn(N, S, K, device="cuda", dtype=dtype)
    p = (torch.randn(16, K, device="cuda") / 4).to(dtype)
    a_proj = torch.randn(N * S, 16, device="cuda")
    acc = torch.zeros(N, 3 * 256, device="cuda")
    native.proj_left_outer(g, p, a_proj, acc, 256)
    gp = g.float() @ p.float().T  # [N, S, 16]
    ref = torch.einsum("nsi,nsj->nij", gp, a_proj.view(N, S, 16)).reshape(N, 256)
    _status_ok(native)
    scale = ref.abs().max().item()
    torch.testing.assert_close(acc[:, 256:512], ref, atol=2e-3 * scale, rtol=1e-2)
    assert acc[:, :256].abs().max().item() == 0 and acc[:, 512:].abs().max().item() == 0


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (200, 72, 264), (1000, 1024, 4096)])
def test_tn_gemm(native, M, N, K):
    torch.manual_seed(2)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    c = native.tn_gemm(a, b)
    ref = a.float() @ b.float().T
    _status_ok(native)
    torch.testing.assert_close(c, ref, atol=1e-3 * K**0.5 + 1e-2, rtol=1e-2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_rmsnorm(native, dtype):
    from bergson_b200.ops import functional as F

    torch.manual_seed(3)
    x = torch.randn(37, 512, device="cuda", dtype=dtype, requires_grad=True)
    w = (1 + 0.1 * torch.randn(512, device="cuda")).to(dtype).requires_grad_()
    y = F.rms_norm(x, w, 1e-5)
    gy = torch.randn_like(y)
    y.backward(gy)
    x2 = x.detach().float().requires_grad_()
    w2 = w.detach().float().requires_grad_()
    y2 = F.rms_norm_ref(x2, w2, 1e-5)
    y2.backward(gy.float())
    tol = dict(atol=3e-2, rtol=3e-2) if dtype == torch.bfloat16 else dict(atol=1e-5, rtol=1e-4)
    torch.testing.assert_close(y.float(), y2, **tol)
    torch.testing.assert_close(x.grad.float(), x2.grad, **tol)
    torch.testing.assert_close(w.grad.float(), w2.grad, atol=tol["atol"] * 10, rtol=tol["rtol"])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_layernorm(native, dtype):
    from bergson_b200.ops import functional as F

    torch.manual_seed(4)
    x = torch.randn(29, 768, device="cuda", dtype=dtype, requires_grad=True)
    w = (1 + 0.1 * torch.randn(768, device="cuda")).to(dtype).requires_grad_()
    b = (0.1 * torch.randn(768, device="cuda")).to(dtype).requires_grad_()
    y = F.layer_norm(x, w, b, 1e-5)
    gy = torch.randn_like(y)
    y.backward(gy)
    x2, w2, b2 = (t.detach().float().requires_grad_() for t in (x, w, b))
    y2 = F.layer_norm_ref(x2, w2, b2, 1e-5)
    y2.backward(gy.float())
    tol = dict(atol=3e-2, rtol=3e-2) if dtype == torch.bfloat16 else dict(atol=1e-5, rtol=1e-4)
    torch.testing.assert_close(y.float(), y2, **tol)
    torch.testing.assert_close(x.grad.float(), x2.grad, **tol)
    torch.testing.assert_close(w.grad.float(), w2.grad, atol=tol["atol"] * 10, rtol=tol["rtol"])
    torch.testing.assert_close(b.grad.float(), b2.grad, atol=tol["atol"] * 10, rtol=tol["rtol"])


@pytest.mark.parametrize("rot", [8, 32])
def test_rotary(native, rot):
    from bergson_b200.ops import functional as F

    x = torch.randn(2, 19, 4, 32, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    cos, sin = F.rotary_tables(19, rot, 10000.0, x.device)
    y = F.rotary(x, cos, sin, rot)
    gy = torch.randn_like(y)
    y.backward(gy)
    x2 = x.detach().float().requires_grad_()
    y2 = F.rotary_ref(x2, cos, sin, rot)
    y2.backward(gy.float())
    torch.testing.assert_close(y.float(), y2, atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(x.grad.float(), x2.grad, atol=2e-2, rtol=2e-2)


def test_swiglu_gelu(native):
    from bergson_b200.ops import functional as F

    g = torch.randn(64, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    u = torch.randn(64, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = F.swiglu(g, u)
    gy = torch.randn_like(y)
    y.backward(gy)
    g2, u2 = g.detach().float().requires_grad_(), u.detach().float().requires_grad_()
    y2 = F.swiglu_ref(g2, u2)
    y2.backward(gy.float())
    torch.testing.assert_close(y.float(), y2, atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(g.grad.float(), g2.grad, atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(u.grad.float(), u2.grad, atol=3e-2, rtol=3e-2)
    for approx in ("none", "tanh"):
        x = torch.randn(64, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        y = F.gelu(x, approx)
        y.backward(gy)
        x2 = x.detach().float().requires_grad_()
        y2 = F.gelu_ref(x2, approx)
        y2.backward(gy.float())
        torch.testing.assert_close(y.float(), y2, atol=3e-2, rtol=3e-2)
        torch.testing.assert_close(x.grad.float(), x2.grad, atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("V", [1000, 50304])
def test_cross_entropy(native, V):
    from bergson_b200.ops import functional as F

    torch.manual_seed(5)
    z = (3 * torch.randn(33, V, device="cuda")).to(torch.bfloat16).requires_grad_()
    t = torch.randint(0, V, (33,), device="cuda")
    t[5] = -100
    loss = F.token_cross_entropy(z, t)
    w = torch.rand(33, device="cuda")
    (loss * w).sum().backward()
    z2 = z.detach().float().requires_grad_()
    loss2 = F.token_cross_entropy_ref(z2, t)
    (loss2 * w).sum().backward()
    torch.testing.assert_close(loss, loss2, atol=1e-3, rtol=1e-3)
    torch.testing.assert_close(z.grad.float(), z2.grad, atol=5e-3, rtol=2e-2)


def test_finalize_rows(native):
    acc = torch.randn(5, 512, device="cuda") * 1e5
    out = torch.zeros(9, 512, device="cuda", dtype=torch.float16)
    idx = torch.tensor([8, 0, 3, 4, 6], device="cuda")
    native.finalize_rows(acc, out, idx, -65504.0, 65504.0, False)
    ref = acc.clamp(-65504.0, 65504.0).half()
    torch.testing.assert_close(out[idx], ref)
    assert out[1].abs().max() == 0
    out2 = torch.zeros(5, 512, device="cuda", dtype=torch.float16)
    native.finalize_rows(acc / 1e5, out2, None, -65504.0, 65504.0, True)
    r = (acc / 1e5).half().float()
    ref2 = (r / r.norm(dim=1, keepdim=True)).half()
    torch.testing.assert_close(out2, ref2, atol=1e-3, rtol=1e-2)


@pytest.mark.parametrize("T,D", [(64, 128), (1000, 200), (4096, 768), (5000, 1032)])
def test_cov_syrk(native, T, D):
    torch.manual_seed(6)
    x = torch.randn(T, D, device="cuda", dtype=torch.bfloat16)
    c = torch.zeros(D, D, device="cuda")
    native.cov_syrk(x, [c.data_ptr()], [0, D], None)
    native.cov_syrk(x, [c.data_ptr()], [0, D], None)  # accumulates
    _status_ok(native)
    full = torch.triu(c) + torch.triu(c, 1).T
    ref = 2 * (x.float().T @ x.float())
    torch.testing.assert_close(full, ref, atol=1e-3 * T**0.5 + 1e-2, rtol=1e-3)


def test_cov_syrk_row_shards_and_fold(native):
    """Two "ranks" emulated on one GPU as two destination buffers; the fold step adds a
    local accumulator into the same adds."""
    torch.manual_seed(7)
    T, D = 2048, 392
    x = torch.randn(T, D, device="cuda", dtype=torch.bfloat16)
    local = torch.randn(D, D, device="cuda")
    r0, r1 = torch.zeros(200, D, device="cuda"), torch.zeros(D - 200, D, device="cuda")
    native.cov_syrk(x, [r0.data_ptr(), r1.data_ptr()], [0, 200, D], local)
    _status_ok(native)
    got = torch.cat([r0, r1])
    ref = x.float().T @ x.float() + local
    # only 128 x 256 tiles touching the upper triangle are produced
    mask = torch.zeros(D, D, dtype=torch.bool, device="cuda")
    for i in range(0, D, 128):
        mask[i : i + 128, (i // 256) * 256 :] = True
    torch.testing.assert_close(got[mask], ref[mask], atol=0.2, rtol=1e-3)
    assert got[~mask].abs().max() == 0


def test_tn_gemm_gathered_two_buffers(native):
    """All-gather fused into the operand loads: two "ranks" emulated as two buffers."""
    torch.manual_seed(8)
    M, K, N = 300, 520, 200
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b0 = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    b1 = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    c = native.tn_gemm_gathered(a, [b0.data_ptr(), b1.data_ptr()], N)
    _status_ok(native)
    ref = a.float() @ torch.cat([b0, b1]).float().T
    torch.testing.assert_close(c, ref, atol=1e-3 * K**0.5 + 1e-2, rtol=1e-2)


def test_cov_syrk_full_tiles_push(native):
    """Pure push of a local accumulator into two row-shard destinations (T = 0)."""
    D = 392
    local = torch.randn(D, D, device="cuda")
    r0, r1 = torch.zeros(196, D, device="cuda"), torch.zeros(D - 196, D, device="cuda")
    x = torch.zeros(64, D, device="cuda", dtype=torch.bfloat16)
    native.cov_syrk(x, [r0.data_ptr(), r1.data_ptr()], [0, 196, D], local, True, 0)
    _status_ok(native)
    torch.testing.assert_close(torch.cat([r0, r1]), local)
    xs = torch.randn(1000, D, device="cuda", dtype=torch.bfloat16)
    r0.zero_(), r1.zero_()
    native.cov_syrk(xs, [r0.data_ptr(), r1.data_ptr()], [0, 196, D], local, True, -1)
    _status_ok(native)
    torch.testing.assert_close(torch.cat([r0, r1]), local + xs.float().T @ xs.float(), atol=0.2, rtol=1e-3)


def test_adamw_step_and_row_sumsq(native):
    torch.manual_seed(9)
    n = 10007
    p = torch.randn(n, device="cuda")
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    g = torch.randn(n, device="cuda").to(torch.bfloat16)
    pm = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    ref_p = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.1)
    for step in (1, 2, 3):
        native.adamw_step(p, m, v, g, pm, 1e-2, 0.9, 0.99, 1e-8, 0.0, 0.1, step, 1.0)
        ref_p.grad = g.float()
        opt.step()
    torch.testing.assert_close(p, ref_p.data, atol=1e-5, rtol=1e-4)
    torch.testing.assert_close(pm.float(), p, atol=1e-2, rtol=1e-2)
    x = torch.randn(33, 1000, device="cuda", dtype=torch.float16)
    out = torch.ones(33, device="cuda")
    native.row_sumsq(x, out)
    torch.testing.assert_close(out, 1 + x.float().pow(2).sum(1), rtol=1e-4, atol=1e-3)


def test_rotation_hi_lo_is_fp32_accurate(native):
    from bergson_b200.ops import attribution

    torch.manual_seed(10)
    x = torch.randn(3, 700, 768, device="cuda", dtype=torch.bfloat16)
    q = torch.linalg.qr(torch.randn(768, 768, device="cuda", dtype=torch.float64))[0].float()
    got = attribution.rotate(x, q)
    ref = (x.double() @ q.double()).float()
    _status_ok(native)
    assert got.dtype == torch.float32 and got.shape == ref.shape
    assert (got - ref).abs().max() / ref.abs().max() < 2e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layer_norm_and_gelu_second_order_match_torch(native, dtype):
    """Value, gradients and a gradient of the gradients (what a traced training step needs) of the
    kernel-backed LayerNorm and GELU against torch's own formulas in fp64."""
    from bergson_b200 import ops

    torch.manual_seed(0)
    rows, d = 96, 256
    x = torch.randn(rows, d, device="cuda").to(dtype).requires_grad_(True)
    w = (1 + 0.1 * torch.randn(d, device="cuda")).to(dtype).requires_grad_(True)
    b = (0.1 * torch.randn(d, device="cuda")).to(dtype).requires_grad_(True)
    cot = torch.randn(rows, d, device="cuda")
    probe = torch.randn(rows, d, device="cuda")

    def chain(fn, x, w, b, cast):
        y = fn(x, w, b)
        gx, gw, gb = torch.autograd.grad((y * cot.to(cast)).sum(), (x, w, b), create_graph=True)
        inner = (gx * probe.to(cast)).sum() + gw.pow(2).sum() + gb.pow(2).sum()
        ggx, ggw = torch.autograd.grad(inner, (x, w))
        return y, gx, gw, gb, ggx, ggw

    for approx in ("tanh", "none"):
        ours = lambda x, w, b: ops.gelu(ops.layer_norm(x, w, b, 1e-5), approximate=approx)  # noqa: E731
        ref = lambda x, w, b: torch.nn.functional.gelu(  # noqa: E731
            torch.nn.functional.layer_norm(x, (d,), w, b, 1e-5), approximate=approx)
        with ops.composable():  # the kernels must be the path taken for graphs that are differentiated again
            got = chain(ours, x, w, b, dtype)
        assert "LayerNormBwdFn" in type(got[1].grad_fn).__name__ or got[1].grad_fn is not None
        want = chain(ref, *(t.detach().double().requires_grad_(True) for t in (x, w, b)), torch.float64)
        tol = 2e-4 if dtype == torch.float32 else 4e-2
        for g, r in zip(got, want):
            assert (g.double() - r).abs().max() <= tol * (r.abs().max() + 1e-6), approx


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_softmax_second_order_matches_torch(native, dtype):
    """The explicit attention path (scores, softmax, values) differentiated twice: the softmax's
    backward of the backward runs on the kernel; compared with torch in fp64."""
    from bergson_b200 import ops

    torch.manual_seed(0)
    B, H, S, D = 2, 3, 64, 16
    q, k, v = ((torch.randn(B, H, S, D, device="cuda") * 0.5).to(dtype).requires_grad_(True) for _ in range(3))
    cot, probe = torch.randn(B, H, S, D, device="cuda"), torch.randn(B, H, S, D, device="cuda")

    def chain(fn, q, k, v, cast):
        o = fn(q, k, v)
        gq, gk, gv = torch.autograd.grad((o * cot.to(cast)).sum(), (q, k, v), create_graph=True)
        inner = (gq * probe.to(cast)).sum() + (gk * gk).sum() + (gv * probe.to(cast)).sum()
        return (o, gq, gk, gv) + torch.autograd.grad(inner, (q, k, v))

    def ref(q, k, v):
        att = (q @ k.transpose(-1, -2)) / D**0.5
        att = att.masked_fill(~torch.ones(S, S, dtype=torch.bool, device="cuda").tril(), float("-inf"))
        return torch.softmax(att, -1) @ v

    with ops.composable():
        got = chain(ops.causal_attention, q, k, v, dtype)
    want = chain(ref, *(t.detach().double().requires_grad_(True) for t in (q, k, v)), torch.float64)
    tol = 1e-4 if dtype == torch.float32 else 5e-2
    for g, r in zip(got, want):
        assert torch.isfinite(g).all()
        assert (g.double() - r).abs().max() <= tol * (r.abs().max() + 1e-6)


@pytest.mark.parametrize("dtype,V", [(torch.float32, 1000), (torch.bfloat16, 1003)])
def test_token_cross_entropy_second_order_matches_torch(native, dtype, V):
    """Per-token CE on the kernels, differentiated twice (odd vocabulary sizes take the scalar
    loops), with ignored rows, against torch in fp64."""
    from bergson_b200 import ops

    torch.manual_seed(0)
    T = 37
    z = (torch.randn(T, V, device="cuda") * 2).to(dtype).requires_grad_(True)
    w = torch.rand(T, device="cuda").requires_grad_(True)
    tgt = torch.randint(0, V, (T,), device="cuda")
    tgt[::5] = -100
    probe = torch.randn(T, V, device="cuda")

    def chain(ce, z, w, cast):
        loss = (ce(z) * w.to(cast)).sum()
        (gz,) = torch.autograd.grad(loss, z, create_graph=True)
        ggz, ggw = torch.autograd.grad((gz * probe.to(cast)).sum(), (z, w))
        return loss, gz, ggz, ggw

    with ops.composable():
        got = chain(lambda z: ops.token_cross_entropy(z, tgt), z, w, torch.float32)
    z64, w64 = z.detach().double().requires_grad_(True), w.detach().double().requires_grad_(True)
    want = chain(lambda z: torch.nn.functional.cross_entropy(z, tgt, reduction="none", ignore_index=-100), z64, w64,
                 torch.float64)
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    for g, r in zip(got, want):
        assert (g.double() - r).abs().max() <= tol * (r.abs().max() + 1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rms_norm_and_swiglu_second_order_match_torch(native, dtype):
    from bergson_b200 import ops

    torch.manual_seed(0)
    rows, d = 80, 256
    x = torch.randn(rows, d, device="cuda").to(dtype).requires_grad_(True)
    w = (1 + 0.1 * torch.randn(d, device="cuda")).to(dtype).requires_grad_(True)
    u = torch.randn(rows, d, device="cuda").to(dtype).requires_grad_(True)
    cot, probe = torch.randn(rows, d, device="cuda"), torch.randn(rows, d, device="cuda")

    def chain(fn, x, w, u, cast):
        y = fn(x, w, u)
        gx, gw, gu = torch.autograd.grad((y * cot.to(cast)).sum(), (x, w, u), create_graph=True)
        inner = (gx * probe.to(cast)).sum() + gw.pow(2).sum() + (gu * probe.to(cast)).sum()
        return (y, gx, gw, gu) + torch.autograd.grad(inner, (x, w, u))

    def ref(x, w, u):
        n = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * w
        return torch.nn.functional.silu(n) * u

    with ops.composable():
        got = chain(lambda x, w, u: ops.swiglu(ops.rms_norm(x, w, 1e-5), u), x, w, u, dtype)
    want = chain(ref, *(t.detach().double().requires_grad_(True) for t in (x, w, u)), torch.float64)
    tol = 2e-4 if dtype == torch.float32 else 5e-2
    for g, r in zip(got, want):
        assert (g.double() - r).abs().max() <= tol * (r.abs().max() + 1e-6)
