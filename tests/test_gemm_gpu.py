"""Persistent tcgen05 GEMM against fp32 torch products: every operand layout, single-CTA and
CTA-pair forms, ragged shapes, bias, accumulation, the projection side output, the batched
sum-of-squares form, and a bounded wait that is made to run out."""

import pytest
import torch

pytestmark = pytest.mark.gpu

WAIT = 400_000_000  # cycles; keeps a protocol error from costing more than a fraction of a second


def _operands(M, N, K, a_mn, b_mn, dtype=torch.bfloat16, batch=None):
    lead = () if batch is None else (batch,)
    a = torch.randn(*lead, *((K, M) if a_mn else (M, K)), device="cuda", dtype=dtype)
    b = torch.randn(*lead, *((K, N) if b_mn else (N, K)), device="cuda", dtype=dtype)
    af = a.float().transpose(-1, -2) if a_mn else a.float()
    bf = b.float() if b_mn else b.float().transpose(-1, -2)
    return a, b, af @ bf


def _status():
    return torch.zeros(1, dtype=torch.int32, device="cuda")


MODES = {"single": dict(cta_group=1), "pair": dict(cta_group=2), "wide": dict(cta_group=2, wide=True)}


def _gemm(mode, a, b, a_mn, b_mn, out, out_f32, bias, accumulate, aux, sq, st):
    from bergson_b200.ops import native

    return native.gemm(a, b, a_mn, b_mn, out, out_f32, bias, accumulate, aux, sq_accumulate=sq, wait_cycles=WAIT,
                       status=st, **MODES[mode])


@pytest.mark.parametrize("cg", ["single", "pair", "wide"])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (300, 520, 200), (1000, 776, 328), (129, 8, 72), (2048, 1280, 1024)])
def test_gemm_layouts_and_ragged_shapes(cg, a_mn, b_mn, M, N, K):
    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("MN-major operands need a row stride that is a multiple of 8 elements")
    torch.manual_seed(M + N + K)
    a, b, ref = _operands(M, N, K, a_mn, b_mn)
    st = _status()
    d32, _ = _gemm(cg, a, b, a_mn, b_mn, None, True, None, False, None, False, st)
    d16, _ = _gemm(cg, a, b, a_mn, b_mn, None, False, None, False, None, False, st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    scale = ref.abs().max()
    assert float((d32 - ref).abs().max() / scale) < 1e-5
    assert float((d16.float() - ref).abs().max() / scale) < 1e-2


@pytest.mark.parametrize("cg", ["single", "pair", "wide"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gemm_bias_accumulate_and_aux_output(cg, dtype):
    torch.manual_seed(1)
    M, N, K = 1111, 1024, 520
    a, b, ref = _operands(M, N, K, False, True, dtype)
    bias = torch.randn(N, device="cuda", dtype=dtype)
    p = (torch.randn(32, K, device="cuda") / 4).to(dtype)
    st = _status()
    d, aux = _gemm(cg, a, b, False, True, None, True, bias, False, p, False, st)
    ref_b = ref + bias.float()
    assert float((d - ref_b).abs().max() / ref_b.abs().max()) < 1e-5
    ref_aux = a.float() @ p.float().T
    assert aux.shape == (M, 32) and float((aux - ref_aux).abs().max() / ref_aux.abs().max()) < 1e-5
    # accumulate into an existing output, in the 16-bit type as well
    _gemm(cg, a, b, False, True, d, True, None, True, None, False, st)
    assert float((d - (ref_b + ref)).abs().max() / ref.abs().max()) < 1e-5
    d16 = torch.ones(M, N, device="cuda", dtype=dtype)
    _gemm(cg, a, b, False, True, d16, False, None, True, None, False, st)
    assert float((d16.float() - (ref + 1)).abs().max() / ref.abs().max()) < 2e-2
    assert int(st.item()) == 0


@pytest.mark.parametrize("cg", ["single", "pair", "wide"])
def test_gemm_batched_and_sum_of_squares(cg):
    torch.manual_seed(2)
    nb, M, N, K = 5, 200, 264, 136
    a, b, ref = _operands(M, N, K, True, True, batch=nb)
    st = _status()
    d, _ = _gemm(cg, a, b, True, True, None, True, None, False, None, False, st)
    assert d.shape == (nb, M, N) and float((d - ref).abs().max() / ref.abs().max()) < 1e-5
    sq = torch.zeros(M, N, device="cuda")
    _gemm(cg, a, b, True, True, sq, True, None, False, None, True, st)
    want = ref.pow(2).sum(0)
    assert float((sq - want).abs().max() / want.abs().max()) < 1e-5
    assert int(st.item()) == 0


def test_gemm_is_bitwise_repeatable():
    from bergson_b200.ops import native

    torch.manual_seed(3)
    a, b, _ = _operands(3000, 1536, 2048, False, False)
    outs = [_gemm("wide", a, b, False, False, None, False, None, False, None, False, _status())[0] for _ in range(3)]
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


def test_wait_probe_times_out_and_returns():
    """A barrier that nothing arrives on: the bounded wait gives up after its budget, the
    kernel records the status and returns; the context stays usable."""
    from bergson_b200.ops import native

    st = _status()
    waited = native.wait_probe(100_000, st)
    torch.cuda.synchronize()
    assert int(st.item()) == 4  # kStatusTimeoutFlag
    assert 100_000 <= int(waited.item()) < 50_000_000
    x = torch.ones(8, device="cuda")
    assert float(x.sum()) == 8.0


def _second_order(fn, a, b, probe_a):
    """Value, first derivatives and a second derivative (d/da, d/db of <dL/db, probe>) of
    ``L = sum(fn(a, b) * cot)``: enough to exercise the backward of the backward."""
    y = fn(a, b)
    cot = torch.linspace(-1, 1, y.numel(), device=y.device, dtype=y.dtype).view_as(y)
    ga, gb = torch.autograd.grad((y * cot).sum(), (a, b), create_graph=True)
    inner = (ga * probe_a).sum() + (gb * gb).sum() * 1e-3
    gga, ggb = torch.autograd.grad(inner, (a, b))
    return y, ga, gb, gga, ggb


@pytest.mark.parametrize("a_mn", [False, True])
@pytest.mark.parametrize("b_mn", [False, True])
def test_gemm_function_is_closed_under_differentiation(a_mn, b_mn):
    from bergson_b200.ops.linear import _GemmFn

    torch.manual_seed(0)
    M, N, K = 264, 136, 200
    a = (torch.randn((K, M) if a_mn else (M, K), device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
    b = (torch.randn((K, N) if b_mn else (N, K), device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
    probe = torch.randn_like(a)

    def ours(a, b):
        return _GemmFn.apply(a, b, a_mn, b_mn, None)

    def ref(a, b):
        A = a.T if a_mn else a
        B = b if b_mn else b.T
        return A @ B

    got = _second_order(ours, a, b, probe)
    a64, b64 = a.detach().double().requires_grad_(True), b.detach().double().requires_grad_(True)
    want = _second_order(ref, a64, b64, probe.double())
    for g, w in zip(got, want):
        scale = w.abs().max().item() + 1e-6
        assert (g.double() - w).abs().max().item() <= 2e-2 * scale


def test_linear_pads_odd_output_sizes_and_stays_twice_differentiable():
    from bergson_b200 import ops
    from bergson_b200.ops.linear import linear

    torch.manual_seed(0)
    x = (torch.randn(4, 40, 64, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(1003, 64, device="cuda") * 0.2).to(torch.bfloat16).requires_grad_(True)  # 1003 % 8 != 0
    y = linear(x, w)
    assert y.shape == (4, 40, 1003)
    torch.testing.assert_close(y.float(), x.float() @ w.float().T, atol=3e-2, rtol=3e-2)
    with ops.composable():
        y2 = linear(x, w)
        (gx,) = torch.autograd.grad(y2.float().pow(2).sum(), x, create_graph=True)
        (gw,) = torch.autograd.grad(gx.float().pow(2).sum(), w)
    x64, w64 = x.detach().double().requires_grad_(True), w.detach().double().requires_grad_(True)
    (gx64,) = torch.autograd.grad((x64 @ w64.T).pow(2).sum(), x64, create_graph=True)
    (gw64,) = torch.autograd.grad(gx64.pow(2).sum(), w64)
    assert (gx.double() - gx64).abs().max() <= 3e-2 * gx64.abs().max()
    assert (gw.double() - gw64).abs().max() <= 5e-2 * gw64.abs().max()


def test_gather_with_copy_and_scatter_forms_on_one_gpu():
    """The peer forms of the wide GEMM with both "ranks" on this GPU (every table entry is a
    local buffer): the copier warps fill the other rank's rows of A while the own rows' tiles
    run, and the epilogue scatters row blocks into the owners' slots."""
    from bergson_b200.ops import native

    torch.manual_seed(0)
    world, rows, K, N = 2, 512, 384, 320
    shards = [torch.randn(rows, K, device="cuda").to(torch.bfloat16) for _ in range(world)]
    w = (torch.randn(N, K, device="cuda") * 0.1).to(torch.bfloat16)
    want = torch.cat(shards).float() @ w.float().T
    for rank in range(world):
        full = torch.zeros(world * rows, K, device="cuda", dtype=torch.bfloat16)
        full[rank * rows : (rank + 1) * rows] = shards[rank]
        done = torch.zeros(8, dtype=torch.int32, device="cuda")
        y, _ = native.gemm(full, w, False, False, None, False, None, False, None, cta_group=2, wide=True,
                           a_peer_ptrs=[s.data_ptr() for s in shards], gather_done=done, gather_rank=rank)
        torch.cuda.synchronize()
        assert torch.equal(full, torch.cat(shards))  # the copiers delivered the other rank's rows
        assert int(done[1 - rank]) > 0 and int(done[rank]) == 0
        assert (y.float() - want).abs().max() <= 2e-2 * want.abs().max()
    # Scatter: rank `slot` pushes row block o of its product into owner o's [world, rows, N] region.
    x = torch.cat(shards)
    regions = [torch.full((world, rows, N), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    for slot in range(world):
        native.gemm(x, w, False, False, None, False, None, False, None, cta_group=2, wide=True,
                    d_peer_ptrs=[r.data_ptr() for r in regions], d_rows_per_rank=rows, d_slot=slot)
    torch.cuda.synchronize()
    for owner in range(world):
        block = want[owner * rows : (owner + 1) * rows]
        for slot in range(world):
            got = regions[owner][slot].float()
            assert torch.isfinite(got).all()
            assert (got - block).abs().max() <= 2e-2 * want.abs().max()
        summed = native.slot_reduce(regions[owner], shards[owner][:, :N].contiguous())
        ref = shards[owner][:, :N].float() + 2 * block
        assert (summed.float() - ref).abs().max() <= 3e-2 * ref.abs().max()
    assert int(native.kernel_status(0).item()) == 0


def test_peer_barrier_passes_when_signalled_and_gives_up_when_not():
    """The cross-rank flag barrier with both ranks' flag words on this GPU: it returns cleanly
    when the other rank's arrival is already recorded, and when it never comes the bounded
    wait runs out, the status word says so, and the context stays usable."""
    from bergson_b200.ops import native

    flags = [torch.zeros(8, dtype=torch.int32, device="cuda") for _ in range(2)]
    ptrs = [f.data_ptr() for f in flags]
    st = _status()
    flags[0][1] = 1  # rank 1 "arrived" at epoch 1
    native.peer_barrier(ptrs, 0, 1, 2_000_000, st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert int(flags[0][0]) == 1 and int(flags[1][0]) == 1  # rank 0 signalled both ranks
    native.peer_barrier(ptrs, 0, 2, 200_000, st)  # nobody raises rank 1's word to 2
    torch.cuda.synchronize()
    assert int(st.item()) == 4  # kStatusTimeoutFlag
    assert float(torch.ones(8, device="cuda").sum()) == 8.0
