// TMA-fed tcgen05 "TN" GEMM skeleton: D[rows, BLOCK_N] = A[rows, K] * B[BLOCK_N, K]^T with
// both operands K-major (K contiguous) bf16/fp16 and an fp32 accumulator in TMEM.
//
// One CTA computes one 128 x BLOCK_N tile.  Warp 0 lane 0 is the TMA producer, warp 1 owns
// TMEM and issues the MMAs (lane 0), warps 2..5 are the epilogue (each reads the 32-lane
// TMEM quadrant `warp_id % 4`).  A is addressed through a 3-D tensor map (K, rows, batch) so
// that a tile never straddles two batch items and rows past the end are zero-filled by TMA.
// The epilogue is a functor invoked per thread with its accumulator row.
#pragma once

#include "common.cuh"

namespace bgn {

constexpr int kBlockM = 128;
constexpr int kBlockK = 64;  // 64 two-byte elements = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kGemmThreads = 192;

struct TnGemmShape {
  int rows;            // rows of A per batch item
  int k;               // reduction length
  int n_total;         // rows of B (per source when B is gathered from several buffers)
  int tiles_per_src;   // 0: one B buffer; else n-tiles per source buffer (gridDim.y = sources * this)
};

// B operand maps: index 0 for an ordinary GEMM; one map per rank when the rows of B are
// spread over the ranks' buffers (plain, non-multicast TMA loads, also from peer memory).
struct TmapSet {
  CUtensorMap m[8];
};

template <int BLOCK_N>
struct TnGemmSmem {
  static constexpr int kABytes = kBlockM * kBlockK * 2;
  static constexpr int kBBytes = BLOCK_N * kBlockK * 2;
  // B tiles must keep 1024-byte alignment for the 128B swizzle pattern.
  static constexpr int kBBytesPadded = (kBBytes + 1023) / 1024 * 1024;
  static constexpr int kStageBytes = kABytes + kBBytesPadded;
  // Skinny tiles (BLOCK_N <= 32) are bandwidth bound: two CTAs per SM with six stages each
  // keep more loads in flight and halve the tail of the last wave.
  static constexpr int kCtasPerSm = BLOCK_N <= 32 ? 2 : 1;
  static constexpr int stages(int extra_bytes) {
    int avail = (227 * 1024) / kCtasPerSm - 1024 /*align slack*/ - 256 /*barriers*/ - extra_bytes;
    int s = avail / kStageBytes;
    return s > 8 ? 8 : s;
  }
};

// Epilogue contract:  void operator()(int quad_row /*0..127*/, int c /*chunk start in tile*/,
//                                     const float (&acc)[16], int tile_m, int out_col0 /*global
//                                     column of the tile's first column*/, int n_valid /*valid
//                                     columns in the tile*/, int batch, void* epi_smem)
// called once per 16-column chunk by each of the 128 epilogue threads, followed by
// `finish(...)` after all chunks (all 128 epilogue threads call it).

template <int BLOCK_N, int FMT, class Epilogue>
__global__ void __launch_bounds__(kGemmThreads, TnGemmSmem<BLOCK_N>::kCtasPerSm)
tn_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ TmapSet tmaps_b,
               TnGemmShape shape, int stages, Epilogue epi, int* status) {
  using S = TnGemmSmem<BLOCK_N>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* tiles = smem;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(tiles + stages * S::kStageBytes);
  uint64_t* empty_bar = full_bar + stages;
  uint64_t* tmem_full_bar = empty_bar + stages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_full_bar + 1);
  // Barriers and the TMEM slot live in a fixed 256-byte block; the epilogue scratch that
  // follows is therefore 256-byte aligned (it holds float4 data).
  uint8_t* epi_smem = reinterpret_cast<uint8_t*>(full_bar) + 256;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tile_m = blockIdx.x, tile_n = blockIdx.y, batch = blockIdx.z;
  const int num_kb = (shape.k + kBlockK - 1) / kBlockK;
  constexpr uint32_t kTmemCols = BLOCK_N < 32 ? 32 : BLOCK_N;
  // Which B buffer this n-tile reads, the row coordinate inside it and the output column.
  const int src = shape.tiles_per_src > 0 ? tile_n / shape.tiles_per_src : 0;
  const int n_coord = (shape.tiles_per_src > 0 ? tile_n % shape.tiles_per_src : tile_n) * BLOCK_N;
  const int out_col0 = src * shape.n_total + n_coord;
  const int n_valid = shape.n_total - n_coord < BLOCK_N ? shape.n_total - n_coord : BLOCK_N;
  const CUtensorMap* tmap_b = &tmaps_b.m[src];

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(tmem_full_bar, 1);
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int issued = 0;
      bool ok = true;
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % stages;
        const uint32_t parity = ((kb / stages) & 1) ^ 1;
        if (!mbar_wait_bounded(&empty_bar[s], parity)) {
          atomicCAS(status, kStatusOk, kStatusTimeoutProducer);
          ok = false;
          break;
        }
        uint8_t* a_dst = tiles + s * S::kStageBytes;
        uint8_t* b_dst = a_dst + S::kABytes;
        mbar_expect_tx(&full_bar[s], S::kABytes + S::kBBytes);
        tma_load_3d(a_dst, &tmap_a, &full_bar[s], kb * kBlockK, tile_m * kBlockM, batch);
        tma_load_2d(b_dst, tmap_b, &full_bar[s], kb * kBlockK, n_coord);
        issued = kb + 1;
      }
      if (!ok) {
        // Drain: give copies already issued a bounded chance to land before the CTA exits.
        for (int kb = issued > stages ? issued - stages : 0; kb < issued; ++kb) {
          mbar_wait_bounded(&full_bar[kb % stages], (kb / stages) & 1);
        }
      }
    }
  } else if (warp == 1) {
    constexpr uint32_t idesc = make_idesc_f16(kBlockM, BLOCK_N, FMT);
    bool ok = true;
    for (int kb = 0; kb < num_kb && ok; ++kb) {
      const int s = kb % stages;
      const uint32_t parity = (kb / stages) & 1;
      ok = mbar_wait_bounded(&full_bar[s], parity);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) atomicCAS(status, kStatusOk, kStatusTimeoutMma);
        break;
      }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t a_addr = smem_u32(tiles + s * S::kStageBytes);
        const uint32_t b_addr = a_addr + S::kABytes;
#pragma unroll
        for (int k = 0; k < kBlockK / kUmmaK; ++k) {
          const uint64_t da = make_kmajor_sw128_desc(a_addr + k * kUmmaK * 2);
          const uint64_t db = make_kmajor_sw128_desc(b_addr + k * kUmmaK * 2);
          umma_f16(tmem_base, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
        }
        umma_commit(&empty_bar[s]);
      }
      __syncwarp();
    }
    if (lane == 0) umma_commit(tmem_full_bar);  // fires when every MMA above has retired
    __syncwarp();
  } else {
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    bool ok = mbar_wait_bounded(tmem_full_bar, 0);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) {
      if (lane == 0) atomicCAS(status, kStatusOk, kStatusTimeoutEpilogue);
    }
    tc_fence_after();
    const int row = quad * 32 + lane;
    if (ok) {
#pragma unroll
      for (int c = 0; c < BLOCK_N; c += 16) {
        float acc[16];
        tmem_ld_32x16(tmem_base + (uint32_t(quad * 32) << 16) + c, acc);
        epi(row, c, acc, tile_m, out_col0, n_valid, batch, epi_smem);
      }
    }
    // finish() contains a named barrier over the 128 epilogue threads, so every one of
    // them calls it on both the normal and the give-up path.
    epi.finish(row, tile_m, out_col0, batch, epi_smem, ok);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace bgn
