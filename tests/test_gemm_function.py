"""Layout algebra of the twice-differentiable GEMM function, checked on CPU with a torch
stand-in for the kernel: first and second derivatives for all four storage layouts."""

import sys

import pytest
import torch

import bergson_b200.ops  # noqa: F401 - registers the submodule below
from bergson_b200.ops import native


@pytest.mark.parametrize("a_mn", [False, True])
@pytest.mark.parametrize("b_mn", [False, True])
def test_gemm_function_gradients_all_layouts(monkeypatch, a_mn, b_mn):
    mod = sys.modules["bergson_b200.ops.linear"]

    def fake_gemm(a, b, a_mn, b_mn, out, out_f32, bias, accumulate, aux, **form):
        d = (a.T if a_mn else a) @ (b if b_mn else b.T)
        return (d if bias is None else d + bias), None

    monkeypatch.setattr(native, "gemm", fake_gemm, raising=False)
    monkeypatch.setattr(mod, "_operand_ok", lambda t: True)
    M, N, K = 5, 7, 3
    a = torch.randn((K, M) if a_mn else (M, K), dtype=torch.float64, requires_grad=True)
    b = torch.randn((K, N) if b_mn else (N, K), dtype=torch.float64, requires_grad=True)
    bias = torch.randn(N, dtype=torch.float64, requires_grad=True)
    fn = lambda a, b, bias: mod._GemmFn.apply(a, b, a_mn, b_mn, bias)  # noqa: E731
    assert torch.autograd.gradcheck(fn, (a, b, bias))
    assert torch.autograd.gradgradcheck(fn, (a, b, bias))
