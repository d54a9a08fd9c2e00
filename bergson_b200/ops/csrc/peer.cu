// Cross-rank building blocks over peer memory (one process per GPU, buffers mapped on every
// rank): a bounded flag barrier, the owner-side sum of reduce-scatter slots, and a push of
// row blocks into the owners' slots.  See kernels_peer.h for the contracts.
#include "kernels_peer.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace bgn {

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Thread t < world: tell rank t that this rank reached `epoch`, then wait until rank t's
// arrival shows up in this rank's own flag array.  Everything this rank's earlier kernels on
// the stream wrote (to any rank's memory) is ordered before the signal by the system fence.
__global__ void peer_barrier_kernel(PeerFlagTable table, int rank, int world, unsigned epoch, long long budget,
                                    int* status) {
  const int t = threadIdx.x;
  if (t >= world) return;
  __threadfence_system();
  st_release_sys(table.flags[t] + rank, epoch);
  const unsigned* mine = table.flags[rank] + t;
  const long long start = clock64();
  bool seen = false;
  // Epochs only grow (wrap-around compared as a signed distance).
  while (!(seen = int(ld_acquire_sys(mine) - epoch) >= 0)) {
    if (clock64() - start > budget) break;
    __nanosleep(64);
  }
  if (!seen) atomicCAS(status, kStatusOk, kStatusTimeoutFlag);
  __threadfence_system();
}

template <typename T>
__global__ void slot_reduce_kernel(const T* __restrict__ slots, int world, long slot_elems, const T* __restrict__ residual,
                                   T* __restrict__ out) {
  constexpr int V = 16 / sizeof(T);
  const long n_vec = slot_elems / V;
  for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < n_vec; i += long(gridDim.x) * blockDim.x) {
    float acc[V];
#pragma unroll
    for (int k = 0; k < V; ++k) acc[k] = 0.f;
    if (residual != nullptr) {
      union { uint4 u; T h[V]; } r;
      r.u = reinterpret_cast<const uint4*>(residual)[i];
#pragma unroll
      for (int k = 0; k < V; ++k) acc[k] = float(r.h[k]);
    }
    for (int w = 0; w < world; ++w) {  // fixed order: the sum does not depend on arrival order
      union { uint4 u; T h[V]; } s;
      s.u = reinterpret_cast<const uint4*>(slots + w * slot_elems)[i];
#pragma unroll
      for (int k = 0; k < V; ++k) acc[k] += float(s.h[k]);
    }
    union { uint4 u; T h[V]; } o;
#pragma unroll
    for (int k = 0; k < V; ++k) o.h[k] = T(acc[k]);
    reinterpret_cast<uint4*>(out)[i] = o.u;
  }
}

// src [world * rows, cols] (row stride ld_src) -> block o goes to dst.ptrs[o] + slot * rows * cols.
__global__ void peer_push_kernel(const uint4* __restrict__ src, long ld_src_vec, PeerPtrTable dst, int slot, long rows,
                                 long cols_vec, int world) {
  const long per_block = rows * cols_vec;
  const long total = per_block * world;
  for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < total; i += long(gridDim.x) * blockDim.x) {
    const int o = int(i / per_block);
    const long rem = i - o * per_block;
    const long r = rem / cols_vec, c = rem - r * cols_vec;
    uint4* d = reinterpret_cast<uint4*>(dst.ptrs[o]) + (long(slot) * rows + r) * cols_vec + c;
    *d = src[(long(o) * rows + r) * ld_src_vec + c];
  }
}

}  // namespace bgn

using namespace bgn;

extern "C" int bgn_peer_barrier(const PeerFlagTable* table, int rank, int world, unsigned epoch, long long budget_cycles,
                                int* status, cudaStream_t stream) {
  if (!table || world < 1 || world > kPeerMax || rank < 0 || rank >= world || !status) return int(cudaErrorInvalidValue);
  if (budget_cycles <= 0) budget_cycles = 1ll << 32;  // about two seconds
  peer_barrier_kernel<<<1, 32, 0, stream>>>(*table, rank, world, epoch, budget_cycles, status);
  return int(cudaGetLastError());
}

extern "C" int bgn_slot_reduce(const void* slots, int world, long slot_elems, const void* residual, void* out, int type,
                               cudaStream_t stream) {
  if (world < 1 || slot_elems <= 0 || slot_elems % 8) return int(cudaErrorInvalidValue);
  long blocks = (slot_elems / 8 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (type == 1)
    slot_reduce_kernel<__nv_bfloat16><<<int(blocks), 256, 0, stream>>>(
        (const __nv_bfloat16*)slots, world, slot_elems, (const __nv_bfloat16*)residual, (__nv_bfloat16*)out);
  else if (type == 0)
    slot_reduce_kernel<__half><<<int(blocks), 256, 0, stream>>>((const __half*)slots, world, slot_elems,
                                                                 (const __half*)residual, (__half*)out);
  else
    return int(cudaErrorInvalidValue);
  return int(cudaGetLastError());
}

extern "C" int bgn_peer_push(const void* src, long ld_src, const PeerPtrTable* dst, int slot, long rows, long cols,
                             int world, cudaStream_t stream) {
  if (!dst || world < 1 || world > kPeerMax || cols % 8 || ld_src % 8 || rows <= 0) return int(cudaErrorInvalidValue);
  const long total = rows * (cols / 8) * world;
  long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  peer_push_kernel<<<int(blocks), 256, 0, stream>>>((const uint4*)src, ld_src / 8, *dst, slot, rows, cols / 8, world);
  return int(cudaGetLastError());
}
