// C launch interface of the persistent tcgen05 GEMM; see gemm.cuh for the kernel.
#pragma once

#include <cuda_runtime.h>

extern "C" {

// d[M, N] (+)= A * B over K, 16-bit inputs (fmt 0 = fp16, 1 = bf16), fp32 accumulation.
//   a_mn == 0: `a` is [M, K] row-major with row stride lda;  a_mn == 1: `a` is [K, M], stride lda.
//   b_mn == 0: `b` is [N, K] row-major with row stride ldb;  b_mn == 1: `b` is [K, N], stride ldb.
// Strides are in elements and must be multiples of 8; base pointers 16-byte aligned.
// Output `d` has the input type, or fp32 when out_f32; `bias` ([N], input type or fp32) is
// added per column; `accumulate` adds into d.  aux_n > 0 additionally writes
// aux_out[M, aux_n] (fp32) = A * aux_p^T with aux_p [aux_n, K] (K-major, input type).
// batch > 1 runs the same product for every batch item (strides in elements); with
// sq_accumulate the squares of every item's product are summed into one fp32 d
// (d_batch_stride 0), which must be zero-initialised by the caller.
// cta_group 2 runs pairs of CTAs on one 256-row tile (cluster launch); 1 is the single-CTA form.
// wait_cycles <= 0 selects the default budget of the bounded waits.
struct BgnGemmArgs {
  const void* a;
  const void* b;
  void* d;
  int M, N, K;
  long lda, ldb, ldd;
  int a_mn, b_mn, fmt, out_f32;
  const void* bias;
  int bias_f32;
  int accumulate;
  const void* aux_p;
  int aux_n;
  float* aux_out;
  int batch;
  long a_batch_stride, b_batch_stride, d_batch_stride;
  int sq_accumulate;
  int cta_group;
  int wide;  // with cta_group 2: 512 x 256 tiles per CTA pair (two row blocks per CTA, one accumulator stage)
  int sm_count;
  int panel;  // tile columns per rasterisation panel; <= 0 picks one from K
  long long wait_cycles;
  int no_tma_store;  // 1: write 16-bit outputs from registers instead of through TMA stores
  long long* trace;  // optional device buffer for per-tile timestamps of the first CTA group (debugging aid)
  // Peer-memory forms (pair / single-CTA kernel; K-major A, 16-bit output, batch 1).
  // gather_world > 0: A is the concatenation over ranks of [gather_rows, K] blocks at a_peers[r]
  //   (row stride lda; gather_rows a multiple of 128; M must equal gather_world * gather_rows);
  //   every rank's block is read through its own tensor map with plain (non-multicast) TMA loads.
  // scatter_world > 0: output rows [o * scatter_rows, (o + 1) * scatter_rows) are stored into
  //   d_peers[o] at row scatter_slot * scatter_rows + local row (row stride ldd); `d` is unused.
  //   The stores are complete on the peers only after a cross-rank barrier that follows the kernel.
  // gather_copy (with gather_world > 0; wide kernel): `a` is a local [M, K] buffer (lda == K)
  //   whose rows of rank gather_rank are already in place; one copier warp per CTA pulls the other
  //   ranks' blocks from a_peers[r] into it while the local rows' tiles run, and tiles of remote
  //   rows start once gather_done[r] (device ints, zero before the launch) shows that every CTA
  //   delivered its slice.  gather_rows must be a multiple of 512.
  int gather_world, gather_rows;
  int gather_copy, gather_rank;
  int* gather_done;
  const void* a_peers[8];
  int scatter_world, scatter_rows, scatter_slot;
  void* d_peers[8];
};

int bgn_gemm(const BgnGemmArgs* args, int* status, cudaStream_t stream);

// Waits up to `budget_cycles` SM cycles (at most 2^31) on a barrier that is never signalled, then
// sets *status to the flag-timeout code and stores the cycles spent in *waited.
int bgn_wait_probe(long long budget_cycles, int* status, long long* waited, cudaStream_t stream);
}
