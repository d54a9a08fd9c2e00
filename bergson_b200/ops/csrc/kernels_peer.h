// C launch interface of the peer-memory helpers (peer.cu).  Every pointer table holds device
// addresses that are valid on the calling GPU: this rank's own buffer and its mappings of
// the other ranks' buffers (one process per GPU).
#pragma once

#include <cuda_runtime.h>

extern "C" {

enum { kPeerMax = 8 };

struct PeerFlagTable {
  unsigned* flags[kPeerMax];  // flags[r]: rank r's array of kPeerMax 32-bit words, zero at start
};

struct PeerPtrTable {
  void* ptrs[kPeerMax];
};

// Barrier over `world` ranks on the stream: orders everything this rank's earlier kernels on
// the stream stored (into any rank's memory) before every other rank's later kernels.
// Each rank calls it with the same, strictly growing `epoch` (start at 1).  The wait is
// bounded: after `budget_cycles` SM cycles (<= 0: about two seconds) the kernel records the
// flag-timeout code in *status and returns, so a missing peer never hangs the GPU; the caller
// must then treat the data as incomplete.  Ranks must run on different GPUs.
int bgn_peer_barrier(const PeerFlagTable* table, int rank, int world, unsigned epoch, long long budget_cycles,
                     int* status, cudaStream_t stream);

// out[i] = (residual ? residual[i] : 0) + sum_w slots[w * slot_elems + i], accumulated in fp32 in
// rank order and rounded once (type 0 = fp16, 1 = bf16; slot_elems a multiple of 8, 16-byte
// aligned pointers): the owner's half of a reduce-scatter whose other half are peer stores.
int bgn_slot_reduce(const void* slots, int world, long slot_elems, const void* residual, void* out, int type,
                    cudaStream_t stream);

// Row block o of src [world * rows, cols] (16-bit elements, row stride ld_src) is copied into
// dst->ptrs[o] at element offset slot * rows * cols: the push half of a reduce-scatter for data
// that is not produced by a GEMM epilogue.
int bgn_peer_push(const void* src, long ld_src, const PeerPtrTable* dst, int slot, long rows, long cols, int world,
                  cudaStream_t stream);
}
