"""Micro-benchmarks of the attribution kernels against their rooflines.

    python benchmarks/bench_kernels.py [--kernel NAME] [--small] [--iters N]

Each kernel is timed with CUDA events after warm-up, on inputs larger than L2, and
reported as achieved bandwidth / throughput and as a fraction of the measured peaks in
``MEASURED_PEAKS.json`` at the repository root (copy bandwidth and cuBLAS bf16 GEMM).
The torch composition of the same op (cuBLAS / ATen) is timed alongside.  ``--small``
selects shapes of a few hundred MB for profiler captures.
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

import sys

sys.path.insert(0, str(Path(__file__).resolve().parent))
from common import ROOT  # noqa: E402,F401  (puts the repository root on sys.path)


def _peaks() -> dict:
    p = Path(__file__).resolve().parents[1] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "tflops": d["bf16_tflops"], "src": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "src": "fallback"}


def _time(fn, iters: int, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(iters):
        fn()
    t1.record()
    torch.cuda.synchronize()
    return t0.elapsed_time(t1) / iters


def bench_proj_right(small: bool, iters: int):
    from bergson_b200.ops import native

    T, K = (16384, 4096) if small else (65536, 4096)
    a = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    p = (torch.randn(16, K, device="cuda") / 4).to(torch.bfloat16)
    ms = _time(lambda: native.proj_right(a, p), iters)
    ref = _time(lambda: a @ p.T, iters)
    return dict(kernel="proj_right", shape=[T, K], ms=ms, torch_ms=ref, bytes=T * K * 2 + T * 64, flops=2 * T * K * 16)


def bench_proj_left_outer(small: bool, iters: int):
    from bergson_b200.ops import native

    N, S, K = (8, 2048, 4096) if small else (32, 2048, 4096)
    g = torch.randn(N, S, K, device="cuda", dtype=torch.bfloat16)
    p = (torch.randn(16, K, device="cuda") / 4).to(torch.bfloat16)
    ap = torch.randn(N * S, 16, device="cuda")
    acc = torch.zeros(N, 256, device="cuda")
    ms = _time(lambda: native.proj_left_outer(g, p, ap, acc, 0), iters)
    apb = ap.view(N, S, 16).to(torch.bfloat16)
    ref = _time(lambda: (g @ p.T).mT @ apb, iters)
    return dict(kernel="proj_left_outer", shape=[N, S, K], ms=ms, torch_ms=ref,
                bytes=N * S * K * 2 + N * S * 64, flops=2 * N * S * K * 16 + 2 * N * S * 256)


def bench_cov_syrk(small: bool, iters: int):
    from bergson_b200.ops import native

    T, D = (16384, 3072) if small else (65536, 4096)
    x = torch.randn(T, D, device="cuda", dtype=torch.bfloat16)
    c = torch.zeros(D, D, device="cuda")
    ms = _time(lambda: native.cov_syrk(x, [c.data_ptr()], [0, D], None), iters)
    xf = None
    ref = _time(lambda: torch.addmm(c, x.T, x.to(torch.bfloat16), out=None) if False else x.T @ x, iters)
    del xf
    # only tiles on or above the block diagonal are computed
    nt = -(-D // 128)
    frac = (nt * (nt + 1) / 2) / (nt * nt)
    return dict(kernel="cov_syrk", shape=[T, D], ms=ms, torch_ms=ref, bytes=T * D * 2 + D * D * 4,
                flops=2 * T * D * D * frac, note="flops count the computed (upper) tiles; torch_ms is the full bf16 GEMM")


def bench_tn_gemm(small: bool, iters: int):
    from bergson_b200.ops import native

    M, N, K = (8192, 1024, 8192) if small else (32768, 1024, 57344)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    ms = _time(lambda: native.tn_gemm(a, b), iters)
    ref = _time(lambda: a @ b.T, iters)
    return dict(kernel="tn_gemm(score)", shape=[M, N, K], ms=ms, torch_ms=ref, bytes=(M + N) * K * 2 + M * N * 4,
                flops=2 * M * N * K)


def bench_ce(small: bool, iters: int):
    from bergson_b200.ops import native

    T, V = (4096, 128256) if small else (16384, 128256)
    z = torch.randn(T, V, device="cuda", dtype=torch.bfloat16)
    t = torch.randint(0, V, (T,), device="cuda")
    ms = _time(lambda: native.ce_fwd(z, t, -100), iters)
    ref = _time(lambda: torch.nn.functional.cross_entropy(z, t, reduction="none"), iters)
    return dict(kernel="ce_fwd", shape=[T, V], ms=ms, torch_ms=ref, bytes=T * V * 2, flops=0)


def bench_rmsnorm(small: bool, iters: int):
    from bergson_b200.ops import native

    T, D = (32768, 4096) if small else (131072, 4096)
    x = torch.randn(T, D, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(D, device="cuda", dtype=torch.bfloat16)
    ms = _time(lambda: native.rmsnorm_fwd(x, w, 1e-5), iters)
    from bergson_b200.ops.functional import rms_norm_ref

    ref = _time(lambda: rms_norm_ref(x, w, 1e-5), iters)
    return dict(kernel="rmsnorm_fwd", shape=[T, D], ms=ms, torch_ms=ref, bytes=2 * T * D * 2, flops=0)


def _time_interleaved(fns: dict, rounds: int = 6, inner: int = 5) -> dict:
    """Median milliseconds per call of each function, the functions taking turns in short
    bursts so that clock and temperature drift hits all of them alike."""
    import statistics

    for fn in fns.values():
        for _ in range(3):
            fn()
    torch.cuda.synchronize()
    samples = {k: [] for k in fns}
    for _ in range(rounds):
        for k, fn in fns.items():
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(inner):
                fn()
            t1.record()
            torch.cuda.synchronize()
            samples[k].append(t0.elapsed_time(t1) / inner)
    return {k: statistics.median(v) for k, v in samples.items()}


def bench_linear_gemm(small: bool, iters: int):
    """The Linear-layer products of the 32-layer d4096 model (16384 tokens per step) on the
    persistent tcgen05 GEMM (CTA-pair form, with and without the projection side output, and
    the single-CTA form) against torch (cuBLAS), interleaved in time."""
    from bergson_b200.ops import native

    T = 4096 if small else 16384
    shapes = [("fwd q/o", T, 4096, 4096, False), ("fwd k/v", T, 1024, 4096, False), ("fwd gate/up", T, 14336, 4096, False),
              ("fwd down", T, 4096, 14336, False), ("dgrad q/o", T, 4096, 4096, True), ("dgrad k/v", T, 4096, 1024, True),
              ("dgrad gate/up", T, 4096, 14336, True), ("dgrad down", T, 14336, 4096, True)]
    out = []
    for name, M, N, K, b_mn in shapes:
        a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        b = torch.randn((K, N) if b_mn else (N, K), device="cuda", dtype=torch.bfloat16)
        d = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        p = (torch.randn(16, K, device="cuda") / 4).to(torch.bfloat16)
        ms = _time_interleaved({
            "pair": lambda: native.gemm(a, b, False, b_mn, d, False, None, False, None, 2),
            "pair_proj": lambda: native.gemm(a, b, False, b_mn, d, False, None, False, p, 2),
            "wide": lambda: native.gemm(a, b, False, b_mn, d, False, None, False, None, 2, wide=True),
            "wide_proj": lambda: native.gemm(a, b, False, b_mn, d, False, None, False, p, 2, wide=True),
            "single": lambda: native.gemm(a, b, False, b_mn, d, False, None, False, None, 1),
            "torch": (lambda: torch.matmul(a, b, out=d)) if b_mn else (lambda: torch.matmul(a, b.T, out=d)),
        })
        out.append(dict(kernel=f"gemm {name}", shape=[M, N, K], ms=ms["wide"], ms_with_projection=ms["wide_proj"],
                        ms_pair=ms["pair"], ms_pair_with_projection=ms["pair_proj"], ms_single_cta=ms["single"],
                        torch_ms=ms["torch"],
                        bytes=(M * K + N * K + M * N) * 2, flops=2 * M * N * K))
    return out


def bench_ce_bwd(small: bool, iters: int):
    from bergson_b200.ops import native

    T, V = (4096, 128256) if small else (16384, 128256)
    z = torch.randn(T, V, device="cuda", dtype=torch.bfloat16)
    t = torch.randint(0, V, (T,), device="cuda")
    _, lse = native.ce_fwd(z, t, -100)
    dl = torch.ones(T, device="cuda")
    ms = _time(lambda: native.ce_bwd(z, t, lse, dl, -100), iters)
    zr = z.clone().requires_grad_(True)

    def ref():
        zr.grad = None
        torch.nn.functional.cross_entropy(zr, t, reduction="sum").backward()

    return dict(kernel="ce_bwd", shape=[T, V], ms=ms, torch_ms=_time(ref, iters), bytes=2 * T * V * 2, flops=0)


def bench_rmsnorm_bwd(small: bool, iters: int):
    from bergson_b200.ops import native
    from bergson_b200.ops.functional import rms_norm_ref

    T, D = (32768, 4096) if small else (131072, 4096)
    x = torch.randn(T, D, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(D, device="cuda", dtype=torch.bfloat16)
    dy = torch.randn_like(x)
    _, rstd = native.rmsnorm_fwd(x, w, 1e-5)
    ms = _time(lambda: native.rmsnorm_bwd(dy, x, w, rstd, False), iters)
    xr = x.clone().requires_grad_(True)

    def ref():
        xr.grad = None
        rms_norm_ref(xr, w, 1e-5).backward(dy)

    return dict(kernel="rmsnorm_bwd", shape=[T, D], ms=ms, torch_ms=_time(ref, iters), bytes=3 * T * D * 2, flops=0)


def bench_adamw(small: bool, iters: int):
    from bergson_b200.ops import native

    n = (64 if small else 256) * 1024 * 1024
    p, m, v = (torch.zeros(n, device="cuda") for _ in range(3))
    g = torch.randn(n, device="cuda", dtype=torch.bfloat16)
    pm = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    ms = _time(lambda: native.adamw_step(p, m, v, g, pm, 3e-4, 0.9, 0.999, 1e-8, 0.0, 0.01, 1, 1.0), iters)
    opt = torch.optim.AdamW([torch.nn.Parameter(torch.zeros(n, device="cuda"))], lr=3e-4, fused=True)
    opt.param_groups[0]["params"][0].grad = g.float()
    return dict(kernel="adamw_step", shape=[n], ms=ms, torch_ms=_time(opt.step, iters), bytes=n * (6 * 4 + 2 + 2), flops=0)


def _param_list(small: bool, dtype):
    """A parameter list shaped like a transformer's: a few large matrices, many small vectors."""
    big = 8 if small else 24
    shapes = [(4096, 4096)] * big + [(4096,)] * (4 * big) + [(32768, 1024)]
    return [torch.randn(s, device="cuda").to(dtype) for s in shapes]


def bench_adamw_multi(small: bool, iters: int):
    """Multi-tensor AdamW (in-place step) and the traced step + VJP pair of MAGIC, one launch each,
    against torch's fused multi-tensor AdamW on the same list."""
    from bergson_b200.ops import native

    ps = _param_list(small, torch.bfloat16)
    gs = [torch.randn_like(p) for p in ps]
    ms, vs = [torch.zeros(p.shape, device="cuda") for p in ps], [torch.zeros(p.shape, device="cuda") for p in ps]
    n = sum(p.numel() for p in ps)
    hp = (3e-4, 0.9, 0.999, 1e-8, 1e-8, 0.01)
    coef = torch.ones(1, device="cuda")
    t_step = _time(lambda: native.adamw_multi(ps, ms, vs, gs, *hp, 1, 1.0, coef), iters)
    ref_p = [torch.nn.Parameter(p.float()) for p in ps]
    opt = torch.optim.AdamW(ref_p, lr=3e-4, fused=True)
    for p, g in zip(ref_p, gs):
        p.grad = g.float()
    t_torch = _time(opt.step, iters)
    out = [dict(kernel="adamw_multi (bf16 params, fp32 moments, in place)", shape=[len(ps), n], ms=t_step, torch_ms=t_torch,
                bytes=n * (2 + 2 + 2 + 4 * 4), flops=0)]
    t_fwd = _time(lambda: native.adamw_traced_fwd(ps, gs, ms, vs, *hp, 1), iters)
    cps, cms, cvs = [torch.randn_like(p) for p in ps], [torch.randn_like(m) for m in ms], [None] * len(ps)
    t_bwd = _time(lambda: native.adamw_traced_bwd(gs, ms, vs, cps, cms, cvs, *hp, 1), iters)
    out.append(dict(kernel="adamw_traced_fwd (out of place)", shape=[len(ps), n], ms=t_fwd, torch_ms=t_torch,
                    bytes=n * (2 + 2 + 4 + 4 + 2 + 4 + 4), flops=0))
    out.append(dict(kernel="adamw_traced_bwd (VJP)", shape=[len(ps), n], ms=t_bwd, torch_ms=t_torch,
                    bytes=n * (2 + 4 + 4 + 2 + 4 + 2 + 2 + 4 + 4), flops=0))
    acc = torch.zeros(2, device="cuda")
    t_norm = _time(lambda: native.multi_sumsq(gs, acc, False, 1.0), iters)
    t_norm_torch = _time(lambda: torch.nn.utils.get_total_norm(gs), iters)
    out.append(dict(kernel="multi_sumsq (clipping coefficient)", shape=[len(ps), n], ms=t_norm, torch_ms=t_norm_torch,
                    bytes=n * 2, flops=0))
    return out


def bench_second_order(small: bool, iters: int):
    """Backward-of-backward kernels of the traced (MAGIC) path on GPT-2-sized tensors, against the
    same quantity from torch's own double-backward formulas."""
    from bergson_b200.ops import native

    rows, d, ff = (8192, 768, 3072) if small else (32768, 768, 3072)
    bf = torch.bfloat16
    out = []

    def torch_ms(fn, inputs, cots):
        """Time of autograd evaluating the backward of fn's backward."""
        leaves = [t.detach().requires_grad_(True) for t in inputs]
        y = fn(*leaves)
        grads = torch.autograd.grad(y, leaves, torch.ones_like(y), create_graph=True)
        keep = [(g, c) for g, c in zip(grads, cots) if g is not None and g.requires_grad]
        gs, cs = [g for g, _ in keep], [c for _, c in keep]
        return _time(lambda: torch.autograd.grad(gs, leaves, cs, retain_graph=True, allow_unused=True), iters)

    x = torch.randn(rows, d, device="cuda").to(bf)
    w, b = torch.ones(d, device="cuda", dtype=bf), torch.zeros(d, device="cuda", dtype=bf)
    dy, cu = torch.randn_like(x), torch.randn_like(x)
    _, mean, rstd = native.layernorm_fwd(x, w, b, 1e-5)
    ms = _time(lambda: native.layernorm_bwd_bwd(cu, w, b, dy, x, w, mean, rstd), iters)
    ref = torch_ms(lambda x, w, b: torch.nn.functional.layer_norm(x, (d,), w, b, 1e-5), [x, w, b], [cu, w.float().to(bf), b])
    out.append(dict(kernel="layernorm_bwd_bwd", shape=[rows, d], ms=ms, torch_ms=ref, bytes=rows * d * 2 * 5, flops=0))

    h = torch.randn(rows, ff, device="cuda").to(bf)
    dyh, ch = torch.randn_like(h), torch.randn_like(h)
    ms = _time(lambda: native.gelu_bwd_bwd(ch, dyh, h, True), iters)
    ref = torch_ms(lambda h: torch.nn.functional.gelu(h, approximate="tanh"), [h], [ch])
    out.append(dict(kernel="gelu_bwd_bwd", shape=[rows, ff], ms=ms, torch_ms=ref, bytes=rows * ff * 2 * 5, flops=0))

    s_rows, s_len = (rows // 512) * 12 * 512, 512  # [B * H * S, S] attention rows
    y = torch.softmax(torch.randn(s_rows, s_len, device="cuda"), -1).to(bf)
    dys, cs = torch.randn_like(y), torch.randn_like(y)
    ms = _time(lambda: native.softmax_bwd_bwd(cs, dys, y), iters)
    z = torch.randn(s_rows, s_len, device="cuda").to(bf)
    ref = torch_ms(lambda z: torch.softmax(z, -1), [z], [cs])
    out.append(dict(kernel="softmax_bwd_bwd", shape=[s_rows, s_len], ms=ms, torch_ms=ref, bytes=s_rows * s_len * 2 * 5, flops=0))

    T, V = (4096, 50264) if small else (16384, 50264)
    logits = torch.randn(T, V, device="cuda").to(bf)
    tgt = torch.randint(0, 50257, (T,), device="cuda")
    _, lse = native.ce_fwd(logits, tgt, -100)
    dloss, c = torch.rand(T, device="cuda"), torch.randn(T, V, device="cuda").to(bf)
    ms = _time(lambda: native.ce_bwd_bwd(c, logits, tgt, lse, dloss, -100), iters)
    ref = torch_ms(lambda z: torch.nn.functional.cross_entropy(z.float(), tgt, reduction="none"), [logits], [c])
    out.append(dict(kernel="ce_bwd_bwd", shape=[T, V], ms=ms, torch_ms=ref, bytes=T * V * 2 * 5, flops=0))
    return out


def bench_slot_reduce(small: bool, iters: int):
    """Owner-side sum of reduce-scatter slots (+ residual), 8 slots of [2048, 8192] bf16."""
    from bergson_b200.ops import native

    w, rows, d = (2, 8192, 4096) if small else (8, 2048, 8192)
    slots = torch.randn(w, rows, d, device="cuda").to(torch.bfloat16)
    res = torch.randn(rows, d, device="cuda").to(torch.bfloat16)
    out = torch.empty_like(res)
    ms = _time(lambda: native.slot_reduce(slots, res, out), iters)
    ref = _time(lambda: torch.add(res.float(), slots.float().sum(0)).to(torch.bfloat16), iters)
    return dict(kernel="slot_reduce", shape=[w, rows, d], ms=ms, torch_ms=ref, bytes=(w + 2) * rows * d * 2, flops=0)


def bench_contract(small: bool, iters: int):
    """Per-example 16 x S x 16 contraction of the projected operands (deterministic order)."""
    from bergson_b200.ops import native

    N, S = (8, 2048) if small else (32, 2048)
    gp = torch.randn(N * S, 16, device="cuda")
    ap = torch.randn(N * S, 16, device="cuda")
    acc = torch.zeros(N, 256, device="cuda")
    ms = _time(lambda: native.proj_contract(gp, ap, acc, N, S, 16, 0), iters)
    ref = _time(lambda: torch.bmm(gp.view(N, S, 16).mT, ap.view(N, S, 16)), iters)
    return dict(kernel="proj_contract", shape=[N, S, 16], ms=ms, torch_ms=ref, bytes=2 * N * S * 16 * 4, flops=2 * N * S * 256)


def bench_rotary(small: bool, iters: int):
    from bergson_b200.ops import native
    from bergson_b200.ops.functional import rotary_ref, rotary_tables

    B, S, H, D = (4, 2048, 32, 128) if small else (8, 2048, 32, 128)
    x = torch.randn(B, S, H, D, device="cuda", dtype=torch.bfloat16)
    cos, sin = rotary_tables(S, D, 500000.0, x.device)
    ms = _time(lambda: native.rotary(x, cos, sin, D, False), iters)
    return dict(kernel="rotary", shape=[B, S, H, D], ms=ms, torch_ms=_time(lambda: rotary_ref(x, cos, sin, D), iters),
                bytes=2 * x.numel() * 2, flops=0)


def bench_swiglu(small: bool, iters: int):
    from bergson_b200.ops import native

    T, F_ = (4096, 14336) if small else (16384, 14336)
    g = torch.randn(T, F_, device="cuda", dtype=torch.bfloat16)
    u = torch.randn_like(g)
    dy = torch.randn_like(g)
    ms = _time(lambda: native.swiglu_bwd(dy, g, u), iters)
    ref = _time(lambda: torch.nn.functional.silu(g) * u, iters)
    return dict(kernel="swiglu_bwd", shape=[T, F_], ms=ms, torch_ms=ref, bytes=5 * T * F_ * 2, flops=0,
                note="torch_ms is the forward silu(g) * u composition (3 tensor passes), for scale only")


def bench_gemm_case(small: bool, iters: int):
    """One Linear forward and one input-gradient product on the wide GEMM (profiling case)."""
    from bergson_b200.ops import native

    M, N, K = (8192, 4096, 4096) if small else (16384, 4096, 4096)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    bk = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    bm = torch.randn(K, N, device="cuda", dtype=torch.bfloat16)
    d = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    ms = _time(lambda: native.gemm(a, bk, False, False, d, False, None, False, None, 2, wide=True), iters)
    ms2 = _time(lambda: native.gemm(a, bm, False, True, d, False, None, False, None, 2, wide=True), iters)
    ref = _time(lambda: torch.matmul(a, bk.T, out=d), iters)
    return dict(kernel="gemm_wide", shape=[M, N, K], ms=ms, ms_dgrad=ms2, torch_ms=ref, bytes=(M * K + N * K + M * N) * 2,
                flops=2 * M * N * K)


BENCHES = {"proj_right": bench_proj_right, "proj_left_outer": bench_proj_left_outer, "cov_syrk": bench_cov_syrk,
           "tn_gemm": bench_tn_gemm, "ce_fwd": bench_ce, "rmsnorm_fwd": bench_rmsnorm, "linear_gemm": bench_linear_gemm, "ce_bwd": bench_ce_bwd,
           "rmsnorm_bwd": bench_rmsnorm_bwd, "adamw": bench_adamw, "proj_contract": bench_contract, "rotary": bench_rotary,
           "swiglu_bwd": bench_swiglu, "gemm_case": bench_gemm_case, "adamw_multi": bench_adamw_multi, "second_order": bench_second_order,
           "slot_reduce": bench_slot_reduce}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", choices=sorted(BENCHES), default=None)
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    from clocks import ClockSampler

    peaks = _peaks()
    for name, fn in BENCHES.items():
        if args.kernel and name != args.kernel:
            continue
        with ClockSampler(torch.cuda.current_device(), period_ms=100) as sampler:
            res = fn(args.small, args.iters)
        clocks = sampler.result
        for r in res if isinstance(res, list) else [res]:
            gbs = r["bytes"] / r["ms"] / 1e6
            tf = r["flops"] / r["ms"] / 1e9
            r.update(gbs=round(gbs, 1), tflops=round(tf, 1), frac_hbm=round(gbs / peaks["hbm_gbs"], 3),
                     frac_tc=round(tf / peaks["tflops"], 3), speedup_vs_torch=round(r["torch_ms"] / r["ms"], 2),
                     peaks=peaks["src"], clocks=clocks,
                     ms_x_mhz=round(r["ms"] * clocks["sm_mhz"], 1) if clocks.get("sm_mhz") else None)
            print(json.dumps(r), flush=True)
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
