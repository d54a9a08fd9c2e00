"""The allocation-free RMSNorm backward, called through its exported C symbol.

Some hosts of these kernels may not allocate device memory while they run (a fixed memory
plan, a C caller that only owns its inputs and outputs).  For them the library carries its
own scratch.  The tests call the symbol with ctypes, several times in a row on the same
scratch, compare with the op written out in fp32 PyTorch, and check that neither torch's
allocator nor the device's free memory moved across the calls."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

_TYPE_CODE = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}


def _lib():
    from bergson_b200.ops import native

    assert native.available()
    lib = ctypes.CDLL(str(native.extension_path()))
    fn = lib.bgn_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_long, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.bgn_noalloc_last_error.restype = ctypes.c_char_p
    return lib


def _call(lib, dy, x, w, rstd, dx, dw, type_code=None):
    stream = torch.cuda.current_stream().cuda_stream
    code = _TYPE_CODE[x.dtype] if type_code is None else type_code
    return lib.bgn_rmsnorm_bwd_noalloc(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                       dw.data_ptr(), x.shape[0], x.shape[1], code, stream)


def _reference(dy, x, w, eps):
    """RMSNorm backward in fp32: y = x * rstd * w with rstd = (mean(x^2) + eps)^-1/2."""
    dy, x, w = dy.float(), x.float(), w.float()
    rstd = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    xhat = x * rstd
    gw = dy * w
    dx = rstd * (gw - xhat * (gw * xhat).mean(-1, keepdim=True))
    dw = (dy * xhat).sum(0)
    return dx, dw, rstd.squeeze(-1)


# Rows below, at and above the number of partial-sum slots (296); hidden sizes up to the
# scratch's limit (8192); every element type.  Later cases reuse scratch left by earlier ones.
CASES = [
    (700, 1024, torch.bfloat16),
    (37, 4096, torch.bfloat16),
    (296, 2048, torch.float16),
    (5, 8192, torch.bfloat16),
    (1000, 8192, torch.float32),
    (1, 64, torch.float32),
]


def test_noalloc_rmsnorm_backward_matches_fp32_reference():
    lib = _lib()
    torch.manual_seed(0)
    eps = 1e-5
    inputs = []
    for rows, d, dtype in CASES:
        x = torch.randn(rows, d, device="cuda").to(dtype)
        w = (1 + 0.1 * torch.randn(d, device="cuda")).to(dtype)
        dy = torch.randn(rows, d, device="cuda").to(dtype)
        dx_ref, dw_ref, rstd = _reference(dy, x, w, eps)
        inputs.append((dy, x, w, rstd.contiguous(), torch.empty_like(x), torch.empty(d, device="cuda"), dx_ref, dw_ref))
    # One call first: it resolves the scratch's device address (no allocation either, but the
    # free-memory reading below should bracket steady-state calls only).
    assert _call(lib, *inputs[0][:6]) == 0, lib.bgn_noalloc_last_error().decode()
    torch.cuda.synchronize()
    allocated, reserved = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(2):  # every case twice in a row
        for dy, x, w, rstd, dx, dw, _, _ in inputs:
            rc = _call(lib, dy, x, w, rstd, dx, dw)
            assert rc == 0, lib.bgn_noalloc_last_error().decode()
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert torch.cuda.memory_allocated() == allocated and torch.cuda.memory_reserved() == reserved
    assert free_after == free_before
    for (rows, d, dtype), (dy, x, w, rstd, dx, dw, dx_ref, dw_ref) in zip(CASES, inputs):
        tol = 1e-4 if dtype == torch.float32 else 2e-2  # dx is rounded to the 16-bit type
        torch.testing.assert_close(dx.float(), dx_ref, atol=tol, rtol=tol)
        # dw accumulates in fp32 from the stored inputs: only the summation order differs.
        torch.testing.assert_close(dw, dw_ref, atol=1e-3 * rows**0.5, rtol=1e-4)


def test_noalloc_rejects_sizes_beyond_the_scratch():
    lib = _lib()
    d = 8192 + 8
    x = torch.zeros(4, d, device="cuda", dtype=torch.bfloat16)
    rstd = torch.ones(4, device="cuda")
    dw = torch.empty(d, device="cuda")
    rc = _call(lib, x, x, x[0].contiguous(), rstd, torch.empty_like(x), dw)
    assert rc != 0 and b"exceeds" in lib.bgn_noalloc_last_error()


def test_noalloc_names_the_rejected_argument():
    lib = _lib()
    x = torch.zeros(4, 1028, device="cuda", dtype=torch.bfloat16)  # 1028 % 8 != 0
    rstd = torch.ones(4, device="cuda")
    dw = torch.empty(1028, device="cuda")
    args = (x, x, x[0].contiguous(), rstd, torch.empty_like(x), dw)
    assert _call(lib, *args) != 0
    assert b"16-byte packet" in lib.bgn_noalloc_last_error()
    assert _call(lib, *args, type_code=7) != 0
    assert b"element type" in lib.bgn_noalloc_last_error()
    ok = torch.zeros(4, 1024, device="cuda", dtype=torch.bfloat16)
    assert _call(lib, ok, ok, ok[0].contiguous(), rstd, torch.empty_like(ok), dw) == 0
    assert lib.bgn_noalloc_last_error() == b""
