// RMSNorm backward for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference implementation.  It exists for
// hosts that drive the kernels from a context where cudaMalloc / cudaFree (or torch's
// caching allocator) must not run: under a memory budget fixed at start-up, or from a
// thin C caller that owns only its input and output buffers.  The weight-gradient partial sums that `bgn_rmsnorm_bwd` expects the caller to
// provide as scratch live here in a fixed device array that belongs to the library.
#pragma once

#include <cuda_runtime.h>

extern "C" {

// Limits of the built-in scratch: hidden sizes up to kBgnNoAllocMaxD, any number of rows.
// The array occupies kBgnNoAllocPartials * kBgnNoAllocMaxD * 4 bytes (about 9.7 MB) on every
// GPU that loads the library, for the life of the process.
enum { kBgnNoAllocMaxD = 8192, kBgnNoAllocPartials = 296 };

// dx[rows, d] (type code as in kernels.h) and dw[d] (fp32, overwritten) of
// y = rmsnorm(x) * w given dy.  Same math as bgn_rmsnorm_bwd followed by a column sum of
// its partials.  Returns 0 on success, a cudaError_t value on a CUDA failure, and
// cudaErrorInvalidValue when d exceeds kBgnNoAllocMaxD, d is not a multiple of the 16-byte
// packet (8 elements for 16-bit types, 4 for fp32), type is not 0..2, rows is not positive or a
// pointer is null; bgn_noalloc_last_error() then names which, or gives the CUDA error's text.
//
// * Allocates nothing: no cudaMalloc, cudaFree or allocating library call.
// * Every pointer and the stream must belong to the device that is current at the call: the
//   scratch of that device is used, and nothing checks where the buffers live.
// * The first call on each device resolves the device address of the scratch array
//   (cudaGetSymbolAddress with that device current); later calls only launch kernels.
// * All calls on a device share the scratch, which keeps the previous call's contents;
//   every call rewrites the part it reads, so nothing needs clearing between calls, but
//   two calls that overlap on the GPU (different streams) race on it.  Serialise them.
int bgn_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                            float* dw, long rows, int d, int type, cudaStream_t stream);

// Text of the most recent failure of bgn_rmsnorm_bwd_noalloc on the calling thread ("" if none).
const char* bgn_noalloc_last_error(void);
}
