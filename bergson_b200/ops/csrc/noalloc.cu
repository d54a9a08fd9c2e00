// Allocation-free RMSNorm backward; see noalloc.h for the contract.
#include "noalloc.h"

#include <cstdio>
#include <mutex>

#include "kernels.h"

namespace {

// Scratch for the per-block partial sums of dL/dw.  In host code this name is only a handle
// for cudaGetSymbolAddress; the device address is looked up once per device below.
static __device__ __align__(256) float g_dw_partials[kBgnNoAllocPartials * kBgnNoAllocMaxD];

constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {nullptr};
std::mutex g_setup_mutex;
thread_local char g_error[256] = "";

int fail(int code, const char* fmt, long a = 0, long b = 0) {
  std::snprintf(g_error, sizeof(g_error), fmt, a, b);
  return code;
}

// Records "<what>: <CUDA error name> (<code>): <CUDA error text>".
int fail_cuda(int code, const char* what) {
  std::snprintf(g_error, sizeof(g_error), "%s: %s (%d): %s", what, cudaGetErrorName(cudaError_t(code)), code,
                cudaGetErrorString(cudaError_t(code)));
  return code;
}

__global__ void sum_partials_kernel(const float* __restrict__ partials, int n_partial, int d,
                                    float* __restrict__ dw) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= d) return;
  float s = 0.f;
  for (int r = 0; r < n_partial; ++r) s += partials[long(r) * d + c];
  dw[c] = s;
}

// Device address of the scratch array on the current device (resolved on first use).
int scratch_for_current_device(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(int(e), "cudaGetDevice failed (%ld)", long(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(int(cudaErrorInvalidDevice), "device index %ld out of range", dev);
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_dw_partials);
    if (e != cudaSuccess || ptr == nullptr)
      return fail(int(e == cudaSuccess ? cudaErrorInvalidSymbol : e), "cudaGetSymbolAddress failed (%ld)", long(e));
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return 0;
}

}  // namespace

extern "C" const char* bgn_noalloc_last_error(void) { return g_error; }

extern "C" int bgn_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd,
                                       void* dx, float* dw, long rows, int d, int type, cudaStream_t stream) {
  g_error[0] = 0;
  if (!dy || !x || !w || !rstd || !dx || !dw)
    return fail(int(cudaErrorInvalidValue), "null pointer argument");
  if (d <= 0 || d > kBgnNoAllocMaxD)
    return fail(int(cudaErrorInvalidValue), "hidden size %ld exceeds the built-in scratch (max %ld)", d,
                long(kBgnNoAllocMaxD));
  if (rows <= 0) return fail(int(cudaErrorInvalidValue), "rows must be positive (got %ld)", rows);
  if (type < 0 || type > 2)
    return fail(int(cudaErrorInvalidValue), "element type %ld is not one of 0 (fp16), 1 (bf16), 2 (fp32)", type);
  const int vec = type == 2 ? 4 : 8;  // elements per 16-byte packet
  if (d % vec)
    return fail(int(cudaErrorInvalidValue), "hidden size %ld is not a multiple of the 16-byte packet (%ld elements)", d, vec);
  float* scratch = nullptr;
  if (int rc = scratch_for_current_device(&scratch)) return rc;
  const int n_partial = int(rows < kBgnNoAllocPartials ? rows : kBgnNoAllocPartials);
  int rc = bgn_rmsnorm_bwd(dy, x, w, rstd, dx, scratch, n_partial, rows, d, type, stream);
  if (rc != 0) return fail_cuda(rc, "rmsnorm backward launch failed");
  sum_partials_kernel<<<(d + 255) / 256, 256, 0, stream>>>(scratch, n_partial, d, dw);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail_cuda(int(e), "partial-sum launch failed");
  return 0;
}
