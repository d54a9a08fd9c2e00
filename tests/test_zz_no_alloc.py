"""The allocation-free RMSNorm backward, called through its exported C symbol.

Some hosts of these kernels may not allocate device memory while they run (a fixed memory
plan, a region that will be captured, a C caller that only owns its inputs and outputs).
For them the library carries its own scratch.  The test calls the symbol with ctypes, twice
in a row on the same buffers' worth of scratch, and compares with the regular entry point,
which takes caller-allocated scratch."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from bergson_b200.ops import native

    assert native.available()
    lib = ctypes.CDLL(str(native.extension_path()))
    fn = lib.bgn_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_long, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.bgn_noalloc_last_error.restype = ctypes.c_char_p
    return lib


def _call(lib, dy, x, w, rstd, dx, dw):
    stream = torch.cuda.current_stream().cuda_stream
    return lib.bgn_rmsnorm_bwd_noalloc(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                       dw.data_ptr(), x.shape[0], x.shape[1], 1, stream)


def test_noalloc_rmsnorm_backward_matches_regular_entry_point():
    from bergson_b200.ops import native

    lib = _lib()
    torch.manual_seed(0)
    for rows, d in ((700, 1024), (37, 4096)):  # second call reuses scratch left by the first
        x = torch.randn(rows, d, device="cuda", dtype=torch.bfloat16)
        w = (1 + 0.1 * torch.randn(d, device="cuda")).to(torch.bfloat16)
        dy = torch.randn_like(x)
        _, rstd = native.rmsnorm_fwd(x, w, 1e-5)
        dx_ref, dw_ref = native.rmsnorm_bwd(dy, x, w, rstd, True)
        dx = torch.empty_like(x)
        dw = torch.empty(d, device="cuda", dtype=torch.float32)
        before = torch.cuda.memory_allocated()
        rc = _call(lib, dy, x, w, rstd, dx, dw)
        assert rc == 0, lib.bgn_noalloc_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        torch.testing.assert_close(dx.float(), dx_ref.float(), atol=3e-2, rtol=3e-2)
        torch.testing.assert_close(dw, dw_ref.float(), atol=0.3, rtol=3e-2)


def test_noalloc_rejects_sizes_beyond_the_scratch():
    lib = _lib()
    d = 8192 + 8
    x = torch.zeros(4, d, device="cuda", dtype=torch.bfloat16)
    rstd = torch.ones(4, device="cuda")
    dw = torch.empty(d, device="cuda")
    rc = _call(lib, x, x, x[0].contiguous(), rstd, torch.empty_like(x), dw)
    assert rc != 0 and b"exceeds" in lib.bgn_noalloc_last_error()
