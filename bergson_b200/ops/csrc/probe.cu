// A kernel whose only job is to wait, with a budget, on an mbarrier that nothing arrives on.
// It exercises the give-up path that every pipelined kernel of this library shares: the wait
// returns false once the cycle budget is spent, the status word is set, and the kernel returns
// normally, leaving the context usable.  Nothing here faults, traps or spins without a limit.
#include "gemm.cuh"
#include "kernels_gemm.h"

namespace bgn {

__global__ void wait_probe_kernel(long long budget, int* status, long long* waited) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const long long start = clock64();
    const bool ok = mbar_wait_budget(&bar, 0, budget);  // phase 0 never completes
    *waited = clock64() - start;
    if (!ok) atomicCAS(status, kStatusOk, kStatusTimeoutFlag);
  }
}

}  // namespace bgn

extern "C" int bgn_wait_probe(long long budget_cycles, int* status, long long* waited, cudaStream_t stream) {
  if (budget_cycles <= 0 || budget_cycles > (1ll << 31)) return int(cudaErrorInvalidValue);
  bgn::wait_probe_kernel<<<1, 32, 0, stream>>>(budget_cycles, status, waited);
  return int(cudaGetLastError());
}
