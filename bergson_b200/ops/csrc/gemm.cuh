// Persistent tcgen05 GEMM:  D[M, N] (+)= A * B  with 16-bit inputs and fp32 accumulation in TMEM.
//
// Either operand may be stored "K-major" (the reduction axis is contiguous: A as [M, K],
// B as [N, K] row-major) or "MN-major" (the M / N axis is contiguous: A as [K, M], B as
// [K, N] row-major), which covers the forward (x W^T), input-gradient (g W) and
// weight-gradient (g^T x) products of a Linear layer without any transposed copy.
//
// Structure (one CTA, or a pair of CTAs on neighbouring SMs when CG == 2):
//   * warps 0 and 6, one lane each: TMA producers of the A and of the B operand; a ring of
//     shared-memory stages, each holding a 128-row slab of A and (256 / CG) rows of B, 64
//     reduction elements deep (one TMA instruction per operand and stage);
//   * warp 1, one lane of the leader CTA: issues tcgen05.mma (cta_group::CG); with CG == 2
//     the instruction spans both CTAs (M = 256: 128 accumulator rows in each CTA's TMEM,
//     each CTA supplies half of B), which halves the shared-memory traffic per flop;
//   * warps 2..5: epilogue; they drain one of two TMEM accumulator stages (256 columns
//     each) while the tensor cores fill the other for the CTA's next tile.
// CTAs are persistent: tile indices are dealt round-robin over the grid, rasterised in
// panels of a few tile columns so that a wave of CTAs shares its A and B slabs through L2.
//
// Optional extra output ("aux tile"): one more tile column per tile row whose B operand is a
// small matrix P [aux_n, K] (aux_n <= 64), written as fp32 [M, aux_n].  The Linear layers use it
// to get A P_in^T (forward) and G P_out^T (input-gradient pass) from the same pass over A.
//
// No load carries a multicast qualifier.  With CG == 2 each CTA loads its own halves with
// plain TMA loads that signal the leader CTA's barrier.  Every wait is bounded by a cycle
// budget passed at launch; a wait that runs out records a status word, the role stops issuing
// work, and the CTA still reaches the final barrier and frees its TMEM.
#pragma once

#include "common.cuh"

namespace bgn {

constexpr int kGemmBlockK = 64;
constexpr int kGemmTileN = 256;
constexpr int kGemmThreadsV2 = 224;

constexpr int kGemmMaxPeers = 8;

struct GemmParams {
  int M, N, K;
  int a_mn, b_mn;      // 1: operand stored MN-major
  void* d;             // [M, ldd] output (16-bit type of the inputs, or fp32 when OUT32)
  long ldd;
  const void* bias;    // optional [N], same 16-bit type as the inputs (or fp32 when bias_f32)
  int bias_f32;
  int accumulate;      // 1: d += result
  int aux_n;           // 0, or rows of the aux operand P (multiple of 16, <= 64)
  float* aux_out;      // [M, aux_ld] fp32
  long aux_ld;
  int batch;           // >= 1; batched operands use the third coordinate of the tensor maps
  long d_batch_stride; // elements between consecutive batch items of d (0: all batches add
                       // into the same matrix, see sq_accumulate)
  int sq_accumulate;   // 1: d (fp32) += result^2 with vector reductions (batched sum of squares)
  int panel;           // tile columns per rasterisation panel
  int a_blocked;       // MN-major A addressed through a (64, K, M/64[, batch]) map: one load per stage
  int b_blocked;       // likewise for an MN-major B
  int tma_store;       // 16-bit output written through shared-memory staging and TMA stores
  long long wait_cycles;
  long long* trace;    // optional: per-tile timestamps of CTA group 0 (8 values per tile); null in production
  // Peer-memory forms (pair / single-CTA kernel only).
  int a_gather_rows;   // > 0: rows [r * a_gather_rows, (r + 1) * a_gather_rows) of A live in rank r's
                       // buffer and are loaded through that rank's tensor map (all-gather -> GEMM)
  int d_scatter_rows;  // > 0: output rows [o * d_scatter_rows, ...) are stored into rank o's buffer
                       // d_peers[o], at row d_slot * d_scatter_rows + local row (GEMM -> the push
                       // half of a reduce-scatter; the owner adds the slots afterwards)
  int d_slot;
  void* d_peers[kGemmMaxPeers];
  // Gather-with-copy form (wide kernel only): A is the local [M, K] buffer; the row blocks of
  // the other ranks are pulled into it by one copier warp per CTA while the tiles of this
  // rank's own rows are computed, so every remote byte crosses NVLink once.  Tiles are visited
  // starting at this rank's rows (tm_shift); a producer waits (bounded) for gather_done[src] to
  // reach the number of CTAs before it loads rows that came from rank src.
  int gather_copy;
  int gather_rank, gather_world;
  int tm_shift;
  const void* gather_src[kGemmMaxPeers];
  void* d_gather_dst;  // the local [M, K] buffer that tmap_a describes
  int* gather_done;
};

// One tensor map per rank for a row-gathered A operand.
struct GemmPeerMaps {
  CUtensorMap a[kGemmMaxPeers];
};

template <int CG>
struct GemmSmemV2 {
  static constexpr int kABytes = 128 * kGemmBlockK * 2;                 // 16 KB
  static constexpr int kBRows = kGemmTileN / CG;                        // rows of B per CTA
  static constexpr int kBBytes = kBRows * kGemmBlockK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  // Output staging for the TMA-store epilogue: 128 rows x 256 columns of a 16-bit type.
  static constexpr int kStagingBytes = 128 * kGemmTileN * 2;            // 64 KB
  static constexpr int kStages = (227 * 1024 - 2048 - kStagingBytes) / kStageBytes;  // 3 (CG 1) or 5 (CG 2)
  static constexpr int kBytes = kStages * kStageBytes + kStagingBytes + 1024 + 512;
};

// ---- cluster helpers ------------------------------------------------------------------------

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Address of `smem_addr` (a shared::cta address of this CTA) in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// One tiled TMA load of rank 2..4 into this CTA's shared memory.  With CG == 2 the barrier
// address may belong to the leader CTA (pair form of the instruction); no multicast.
template <int CG>
__device__ __forceinline__ void tma_load_nd(uint32_t dst, const CUtensorMap* m, uint32_t bar, int rank, int c0, int c1,
                                            int c2, int c3) {
  const uint64_t map = reinterpret_cast<uint64_t>(m);
  if constexpr (CG == 1) {
    if (rank == 2) {
      asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                   ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
    } else if (rank == 3) {
      asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                   ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
    } else {
      asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                   ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
    }
  } else {
    if (rank == 2) {
      asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                   ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
    } else if (rank == 3) {
      asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                   ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
    } else {
      asm volatile("cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                   ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
    }
  }
}

// Load `rows` rows (a multiple of 64 when MN-major) x 64 reduction elements of one operand.
//   K-major:            box (64 k, rows)            at (k0, row0[, batch])
//   MN-major, blocked:  box (64 mn, 64 k, rows/64)  at (0, k0, row0 / 64[, batch])
//   MN-major, plain:    rows/64 boxes (64 mn, 64 k) at (row0 + 64 b, k0[, batch])
template <int CG>
__device__ __forceinline__ void load_operand(uint32_t dst, const CUtensorMap* m, uint32_t bar, bool mn, bool blocked,
                                             int rows, int row0, int k0, int batch, bool batched) {
  if (!mn) {
    tma_load_nd<CG>(dst, m, bar, batched ? 3 : 2, k0, row0, batch, 0);
  } else if (blocked) {
    tma_load_nd<CG>(dst, m, bar, batched ? 4 : 3, 0, k0, row0 >> 6, batch);
  } else {
    for (int b = 0; b < (rows >> 6); ++b)
      tma_load_nd<CG>(dst + b * 8192, m, bar, batched ? 3 : 2, row0 + b * 64, k0, batch, 0);
  }
}

template <int CG>
__device__ __forceinline__ void umma_f16_cg(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
  if constexpr (CG == 1) {
    umma_f16(tmem_d, da, db, idesc, acc);
  } else {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}" ::"r"(tmem_d),
        "l"(da), "l"(db), "r"(idesc), "r"(acc)
        : "memory");
  }
}

// Arrive on `bar` (same offset in every CTA of the pair) once all MMAs issued so far retire.
template <int CG>
__device__ __forceinline__ void umma_commit_cg(uint64_t* bar) {
  if constexpr (CG == 1) {
    umma_commit(bar);
  } else {
    const uint16_t mask = 3;
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
            smem_u32(bar)),
        "h"(mask)
        : "memory");
  }
}

template <int CG>
__device__ __forceinline__ void tmem_alloc_cg(uint32_t* slot, uint32_t ncols) {
  if constexpr (CG == 1) {
    tmem_alloc(slot, ncols);
    tmem_relinquish();
  } else {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
}

template <int CG>
__device__ __forceinline__ void tmem_dealloc_cg(uint32_t taddr, uint32_t ncols) {
  if constexpr (CG == 1) {
    tmem_dealloc(taddr, ncols);
  } else {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
  }
}

__device__ __forceinline__ bool mbar_wait_budget(uint64_t* bar, uint32_t parity, long long budget) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  while (clock64() - start < budget) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  return false;
}

// 32 lanes x 32 consecutive fp32 columns.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, float* v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

struct GemmTile {
  int tm, tn, batch;
  bool aux;
};

// Tile `t` of the flattened (batch, panel, row, column) order; tiles_nt counts the aux column.
__device__ __forceinline__ GemmTile gemm_tile(long t, int tiles_m, int tiles_n, int tiles_nt, int panel_w) {
  GemmTile r;
  const long per_batch = long(tiles_m) * tiles_nt;
  r.batch = int(t / per_batch);
  const int u = int(t - r.batch * per_batch);
  const int per_panel = panel_w * tiles_m;
  const int panel = u / per_panel;
  const int rem = u - panel * per_panel;
  const int left = tiles_nt - panel * panel_w;
  const int width = left < panel_w ? left : panel_w;
  r.tm = rem / width;
  r.tn = panel * panel_w + rem % width;
  r.aux = r.tn >= tiles_n;
  return r;
}

template <int CG, int FMT, bool OUT32>
__global__ void __launch_bounds__(kGemmThreadsV2, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            const __grid_constant__ CUtensorMap tmap_p, const __grid_constant__ CUtensorMap tmap_d,
            const __grid_constant__ GemmPeerMaps peers, GemmParams p, int* status) {
  using S = GemmSmemV2<CG>;
  using InT = typename std::conditional<FMT == 1, __nv_bfloat16, __half>::type;
  constexpr int kStages = S::kStages;
  constexpr int kTileM = 128 * CG;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = tiles + kStages * S::kStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(staging + S::kStagingBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full_bar = empty_bar + kStages;   // [2]
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;    // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta_rank = CG == 1 ? 0u : cluster_ctarank();
  const bool leader = cta_rank == 0;
  const int group = blockIdx.x / CG, num_groups = gridDim.x / CG;

  const int tiles_m = (p.M + kTileM - 1) / kTileM;
  const int tiles_n = (p.N + kGemmTileN - 1) / kGemmTileN;
  const int tiles_nt = tiles_n + (p.aux_n > 0 ? 1 : 0);
  const long num_tiles = long(tiles_m) * tiles_nt * p.batch;
  const int num_kb = (p.K + kGemmBlockK - 1) / kGemmBlockK;
  const bool three_d = p.batch > 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full_bar[a], 1);
      mbar_init(&tmem_empty_bar[a], 4 * CG);  // one arrival per epilogue warp of every CTA
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    if (p.aux_n > 0) tma_prefetch_desc(&tmap_p);
    if (p.tma_store) tma_prefetch_desc(&tmap_d);
  }
  if (warp == 1) tmem_alloc_cg<CG>(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  if constexpr (CG == 2) cluster_sync_all();  // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0 || warp == 6) {
    if (lane == 0) {
      // ---------------- producers: warp 0 loads this CTA's slab of A, warp 6 its rows of B ----------------
      const bool is_a = warp == 0;
      uint32_t stage = 0, phase = 0;
      long issued = 0;
      bool ok = true;
      for (long t = group; t < num_tiles && ok; t += num_groups) {
        const GemmTile tile = gemm_tile(t, tiles_m, tiles_n, tiles_nt, p.panel);
        const int m0 = tile.tm * kTileM + int(cta_rank) * 128;
        const int b_rows = tile.aux ? p.aux_n / CG : S::kBRows;
        const int n0 = tile.aux ? int(cta_rank) * b_rows : tile.tn * kGemmTileN + int(cta_rank) * b_rows;
        const CUtensorMap* mb = tile.aux ? &tmap_p : &tmap_b;
        const bool b_mn = tile.aux ? false : p.b_mn != 0;
        const uint32_t stage_tx = uint32_t(CG) * uint32_t(S::kABytes + b_rows * kGemmBlockK * 2);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_budget(&empty_bar[stage], phase ^ 1u, p.wait_cycles)) {
            atomicCAS(status, kStatusOk, kStatusTimeoutProducer);
            ok = false;
            break;
          }
          const uint32_t a_dst = smem_u32(tiles + stage * S::kStageBytes);
          uint32_t bar = smem_u32(&full_bar[stage]);
          if (is_a && leader) mbar_expect_tx(&full_bar[stage], stage_tx);
          if constexpr (CG == 2) bar = map_to_cta(bar, 0);
          const int k0 = kb * kGemmBlockK;
          if (is_a) {
            const CUtensorMap* ma = &tmap_a;
            int m_src = m0;
            if (p.a_gather_rows > 0) {  // this CTA's 128 rows sit in one rank's buffer
              const int src = m0 / p.a_gather_rows;
              ma = &peers.a[src];
              m_src = m0 - src * p.a_gather_rows;
            }
            load_operand<CG>(a_dst, ma, bar, p.a_mn != 0, p.a_blocked != 0, 128, m_src, k0, tile.batch, three_d);
          } else {
            load_operand<CG>(a_dst + S::kABytes, mb, bar, b_mn, p.b_blocked != 0, b_rows, n0, k0, tile.batch,
                             three_d && !tile.aux);
          }
          ++issued;
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        // Give-up path: loads already issued may still be landing in this CTA's shared memory.
        // Wait out a fixed interval far above a TMA round trip before heading for the exit.
        const long long start = clock64();
        while (clock64() - start < 400000) {
        }
      }
      (void)issued;
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (leader) {
      uint32_t stage = 0, phase = 0;
      long local_tile = 0;
      bool ok = true;
      long long g_start = 0, g_wait = 0;
      if (p.trace != nullptr && lane == 0) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g_start));
      for (long t = group; t < num_tiles && ok; t += num_groups, ++local_tile) {
        const GemmTile tile = gemm_tile(t, tiles_m, tiles_n, tiles_nt, p.panel);
        const int as = int(local_tile & 1);
        const uint32_t use = uint32_t(local_tile >> 1);
        // Wait until the epilogue has drained this accumulator stage (first use: free).
        const bool tracing = p.trace != nullptr && lane == 0 && group == 0;
        const bool tracing_all = p.trace != nullptr && lane == 0;
        const long long t_begin = tracing ? clock64() : 0;
        long long full_wait = 0;
        ok = mbar_wait_budget(&tmem_empty_bar[as], (use & 1u) ^ 1u, p.wait_cycles);
        const long long t_acc_free = tracing ? clock64() : 0;
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) atomicCAS(status, kStatusOk, kStatusTimeoutMma);
          break;
        }
        tc_fence_after();
        const bool b_mn = tile.aux ? false : p.b_mn != 0;
        const int n_inst = tile.aux ? p.aux_n : kGemmTileN;
        const uint32_t idesc = make_idesc_f16(kTileM, n_inst, FMT, p.a_mn, b_mn ? 1 : 0);
        const uint32_t d_addr = tmem_base + uint32_t(as) * kGemmTileN;
        const uint32_t a_step = p.a_mn ? 2048u : 32u, b_step = b_mn ? 2048u : 32u;
        for (int kb = 0; kb < num_kb; ++kb) {
          const long long w0 = tracing_all ? clock64() : 0;
          ok = mbar_wait_budget(&full_bar[stage], phase, p.wait_cycles);
          if (tracing_all) full_wait += clock64() - w0;
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) {
            if (lane == 0) atomicCAS(status, kStatusOk, kStatusTimeoutMma);
            break;
          }
          tc_fence_after();
          if (lane == 0) {
            const uint32_t a_addr = smem_u32(tiles + stage * S::kStageBytes);
            const uint32_t b_addr = a_addr + S::kABytes;
            const uint64_t da0 = p.a_mn ? make_mnmajor_sw128_desc(a_addr, 8192) : make_kmajor_sw128_desc(a_addr);
            const uint64_t db0 = b_mn ? make_mnmajor_sw128_desc(b_addr, 8192) : make_kmajor_sw128_desc(b_addr);
#pragma unroll
            for (int k = 0; k < kGemmBlockK / 16; ++k) {
              // The start-address field counts 16-byte units; the steps keep it inside the stage.
              umma_f16_cg<CG>(d_addr, da0 + uint64_t((a_step * k) >> 4), db0 + uint64_t((b_step * k) >> 4), idesc,
                              (kb | k) != 0 ? 1u : 0u);
            }
            umma_commit_cg<CG>(&empty_bar[stage]);
          }
          __syncwarp();
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok && lane == 0) umma_commit_cg<CG>(&tmem_full_bar[as]);
        if (tracing) {
          long long* tr = p.trace + local_tile * 8;
          tr[0] = t_begin;
          tr[1] = t_acc_free;
          tr[2] = clock64();
          tr[3] = full_wait;
        }
        g_wait += full_wait;
        __syncwarp();
      }
      if (p.trace != nullptr && lane == 0) {
        long long g_end;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g_end));
        long long* tr = p.trace + 512 + group * 4;
        tr[0] = g_start;
        tr[1] = g_end;
        tr[2] = local_tile;
        tr[3] = g_wait;
      }
    }
  } else if (warp < 6) {
    // ---------------- epilogue ----------------
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    long local_tile = 0;
    bool ok = true;
    uint32_t empty_addr[2];
#pragma unroll
    for (int a = 0; a < 2; ++a) {
      empty_addr[a] = smem_u32(&tmem_empty_bar[a]);
      if constexpr (CG == 2) empty_addr[a] = map_to_cta(empty_addr[a], 0);
    }
    for (long t = group; t < num_tiles && ok; t += num_groups, ++local_tile) {
      const GemmTile tile = gemm_tile(t, tiles_m, tiles_n, tiles_nt, p.panel);
      const int as = int(local_tile & 1);
      const uint32_t use = uint32_t(local_tile >> 1);
      const bool tracing = p.trace != nullptr && group == 0 && leader && warp == 2 && lane == 0;
      const long long e0 = tracing ? clock64() : 0;
      ok = mbar_wait_budget(&tmem_full_bar[as], use & 1u, p.wait_cycles);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) atomicCAS(status, kStatusOk, kStatusTimeoutEpilogue);
        break;
      }
      const long long e1 = tracing ? clock64() : 0;
      tc_fence_after();
      const long row = long(tile.tm) * kTileM + long(cta_rank) * 128 + row_in_tile;
      const bool row_ok = row < p.M;
      const uint32_t t_addr = tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(as) * kGemmTileN;
      if (tile.aux) {
        float* dst = p.aux_out + (long(tile.batch) * p.M + row) * p.aux_ld;
        for (int c = 0; c < p.aux_n; c += 16) {
          float v[16];
          tmem_ld_32x16(t_addr + c, v);
          if (row_ok) {
#pragma unroll
            for (int i = 0; i < 16; i += 4)
              *reinterpret_cast<float4*>(dst + c + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
          }
        }
      } else if (!OUT32 && p.tma_store) {
        // Stage this warp's 32 rows x 256 columns in shared memory (four 64-column slabs in the
        // 128-byte swizzle) and hand them to TMA stores, which clip at the matrix edges.
        const int col0 = tile.tn * kGemmTileN;
        const int n_valid = p.N - col0 < kGemmTileN ? p.N - col0 : kGemmTileN;
        uint8_t* stg = staging + quad * 16384;
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // previous tile's stores
        __syncwarp();
        const uint32_t stg_row = smem_u32(stg) + uint32_t(lane) * 128u;
#pragma unroll 1
        for (int c = 0; c < kGemmTileN; c += 32) {
          if (c >= n_valid) break;  // uniform over the CTA
          float v[32];
          tmem_ld_32x32(t_addr + c, v);
          if (p.bias != nullptr) {
            const int nv = n_valid - c < 32 ? n_valid - c : 32;
            if (p.bias_f32) {
              const float* b = reinterpret_cast<const float*>(p.bias) + col0 + c;
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (i < nv) v[i] += __ldg(b + i);
            } else {
              const InT* b = reinterpret_cast<const InT*>(p.bias) + col0 + c;
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (i < nv) v[i] += to_float<InT>(b[i]);
            }
          }
          const uint32_t slab = stg_row + uint32_t(c >> 6) * 4096u;
          const uint32_t chunk0 = uint32_t(c & 63) >> 3;  // 16-byte chunk of the 128-byte row: 0 or 4
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            union { uint4 u; InT h[8]; } o;
#pragma unroll
            for (int e = 0; e < 8; ++e) o.h[e] = from_float<InT>(v[j * 8 + e]);
            const uint32_t addr = slab + (((chunk0 + j) ^ (uint32_t(lane) & 7u)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(o.u.x), "r"(o.u.y), "r"(o.u.z),
                         "r"(o.u.w)
                         : "memory");
          }
        }
        fence_proxy_async();
        __syncwarp();
        const int row0 = tile.tm * kTileM + int(cta_rank) * 128 + quad * 32;
        if (lane == 0 && row0 < p.M) {
          for (int b = 0; b < 4; ++b) {
            if (b * 64 >= n_valid) break;
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                             reinterpret_cast<uint64_t>(&tmap_d)),
                         "r"(smem_u32(stg) + uint32_t(b) * 4096u), "r"(col0 + b * 64), "r"(row0)
                         : "memory");
          }
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      } else {
        const int col0 = tile.tn * kGemmTileN;
        const int n_valid = p.N - col0 < kGemmTileN ? p.N - col0 : kGemmTileN;
        long d_row_off = long(tile.batch) * p.d_batch_stride + row * p.ldd + col0;
        void* d_base = p.d;
        if (p.d_scatter_rows > 0 && row_ok) {
          const int owner = int(row / p.d_scatter_rows);
          d_base = p.d_peers[owner];
          d_row_off = (long(p.d_slot) * p.d_scatter_rows + (row - long(owner) * p.d_scatter_rows)) * p.ldd + col0;
        }
#pragma unroll 1
        for (int c = 0; c < kGemmTileN; c += 32) {
          if (c >= n_valid) break;  // uniform over the CTA
          float v[32];
          tmem_ld_32x32(t_addr + c, v);
          if (!row_ok) continue;
          const int nv = n_valid - c < 32 ? n_valid - c : 32;
          if (p.bias != nullptr) {
            if (p.bias_f32) {
              const float* b = reinterpret_cast<const float*>(p.bias) + col0 + c;
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (i < nv) v[i] += __ldg(b + i);
            } else {
              const InT* b = reinterpret_cast<const InT*>(p.bias) + col0 + c;
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (i < nv) v[i] += to_float<InT>(b[i]);
            }
          }
          if constexpr (OUT32) {
            float* dst = reinterpret_cast<float*>(d_base) + d_row_off + c;
            if (p.sq_accumulate) {
              if (nv == 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
                for (int i = 0; i < 32; i += 4)
                  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + i), "f"(v[i] * v[i]),
                               "f"(v[i + 1] * v[i + 1]), "f"(v[i + 2] * v[i + 2]), "f"(v[i + 3] * v[i + 3])
                               : "memory");
              } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                  if (i < nv) atomicAdd(dst + i, v[i] * v[i]);
              }
            } else if (nv == 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
              for (int i = 0; i < 32; i += 4) {
                float4 o = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                if (p.accumulate) {
                  const float4 old = *reinterpret_cast<const float4*>(dst + i);
                  o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                *reinterpret_cast<float4*>(dst + i) = o;
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (i < nv) dst[i] = p.accumulate ? dst[i] + v[i] : v[i];
            }
          } else {
            InT* dst = reinterpret_cast<InT*>(d_base) + d_row_off + c;
            if (nv == 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                union { uint4 u; InT h[8]; } o;
                if (p.accumulate) {
                  o.u = *reinterpret_cast<const uint4*>(dst + i);
#pragma unroll
                  for (int j = 0; j < 8; ++j) o.h[j] = from_float<InT>(to_float<InT>(o.h[j]) + v[i + j]);
                } else {
#pragma unroll
                  for (int j = 0; j < 8; ++j) o.h[j] = from_float<InT>(v[i + j]);
                }
                *reinterpret_cast<uint4*>(dst + i) = o.u;
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (i < nv) dst[i] = from_float<InT>(p.accumulate ? to_float<InT>(dst[i]) + v[i] : v[i]);
            }
          }
        }
      }
      if (tracing) {
        long long* tr = p.trace + local_tile * 8;
        tr[4] = e0;
        tr[5] = e1;
        tr[6] = clock64();
      }
      // All reads of this accumulator stage by this warp are complete (tcgen05.wait::ld).
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if constexpr (CG == 2) mbar_arrive_cluster(empty_addr[as]);
        else mbar_arrive(&tmem_empty_bar[as]);
      }
    }
  }

  if (warp >= 2 && warp < 6 && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  if constexpr (CG == 2) cluster_sync_all();  // the peer may still be reading this CTA's operands
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_cg<CG>(tmem_base, 512);
  }
}

}  // namespace bgn
