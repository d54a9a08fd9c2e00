// Wide form of the persistent tcgen05 GEMM: a CTA pair owns a 512 x 256 output tile.
//
// Each CTA holds two 128-row blocks of A per stage (rows r and r + 256 of the tile, r being the
// CTA's 128-row share of a 256-row MMA) and its 128-row half of B, so that every B slab in
// shared memory feeds two cta_group::2 MMAs (M = 256, N = 256) instead of one.  Per flop that
// is a quarter less shared-memory fill traffic than the 256 x 256 pair tile of gemm.cuh, which
// is what limits that kernel's tensor-pipe utilisation.  The price is TMEM: the two 128 x 256
// fp32 accumulators fill all 512 columns, so there is one accumulator stage and the epilogue of
// a tile overlaps only the first k-block of the next one.  Eight epilogue warps (two per TMEM
// lane quadrant, each taking half of the columns) keep the drain short: for plain 16-bit outputs
// they move their accumulator slice through registers into a shared-memory staging slab, hand
// the row block back to the MMA warp at once, and let TMA stores write the slab to memory while
// the next tile's MMAs already run.  Other outputs (fp32, accumulate, batched) are stored from
// registers with 32-byte stores.  The two row blocks are released separately.
//
// Warp roles: 0 = A producer, 1 = MMA issuer (leader CTA), 2..9 = epilogue, 10 = B producer,
// 11 = copier (gather-with-copy form only: pulls the other ranks' row blocks of A into local
// memory over NVLink while the tiles of the local rows run; see GemmParams::gather_copy).
// Operand layouts, the aux (projection) tile column, bias, accumulation, the batched
// sum-of-squares form and the bounded waits are those of gemm.cuh.
#pragma once

#include "gemm.cuh"

namespace bgn {

constexpr int kWideThreads = 384;
constexpr int kWideTileM = 512;     // rows per CTA pair
constexpr int kWideABytes = 2 * 128 * kGemmBlockK * 2;   // two row blocks
constexpr int kWideBBytes = 128 * kGemmBlockK * 2;
constexpr int kWideStageBytes = kWideABytes + kWideBBytes;  // 48 KB
constexpr int kWideStages = 3;
// Output staging: each of the eight epilogue warps owns 32 rows x 128 columns of a 16-bit type.
constexpr int kWideStagingBytes = 8 * 32 * 128 * 2;  // 64 KB
constexpr int kWideSmemBytes = kWideStages * kWideStageBytes + kWideStagingBytes + 1024 + 512;

// 32 bytes per thread in one instruction: a full sector per row.
__device__ __forceinline__ void st_global_v8(void* ptr, const uint32_t (&r)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(ptr), "r"(r[0]), "r"(r[1]), "r"(r[2]),
               "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}

__device__ __forceinline__ uint4 ld_volatile_v4(const uint4* ptr) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr));
  return v;
}

__device__ __forceinline__ int ld_acquire_gpu(const int* ptr) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
  return v;
}

// Visit order of the row tiles: rotated so that a rank starts with its own rows.
__device__ __forceinline__ void rotate_tile(GemmTile& tile, const GemmParams& p, int tiles_m) {
  if (p.tm_shift > 0) {
    tile.tm += p.tm_shift;
    if (tile.tm >= tiles_m) tile.tm -= tiles_m;
  }
}

template <int FMT, bool OUT32>
__global__ void __launch_bounds__(kWideThreads, 1)
gemm_wide_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_p, const __grid_constant__ CUtensorMap tmap_d,
                 const __grid_constant__ GemmPeerMaps peers, GemmParams p, int* status) {
  constexpr int CG = 2;
  using InT = typename std::conditional<FMT == 1, __nv_bfloat16, __half>::type;
  constexpr int kStages = kWideStages;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = tiles + kStages * kWideStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(staging + kWideStagingBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full_bar = empty_bar + kStages;   // [1]
  uint64_t* tmem_empty_bar = tmem_full_bar + 1;    // [2]: one per row block
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();
  const bool leader = cta_rank == 0;
  const int group = blockIdx.x / CG, num_groups = gridDim.x / CG;

  const int tiles_m = (p.M + kWideTileM - 1) / kWideTileM;
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
    mbar_init(tmem_full_bar, 1);
    mbar_init(&tmem_empty_bar[0], 8 * CG);  // one arrival per epilogue warp of every CTA
    mbar_init(&tmem_empty_bar[1], 8 * CG);
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    if (p.aux_n > 0) tma_prefetch_desc(&tmap_p);
    if (p.tma_store) tma_prefetch_desc(&tmap_d);
  }
  if (warp == 1) tmem_alloc_cg<CG>(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0 || warp == 10) {
    if (lane == 0) {
      // ---------------- producers ----------------
      const bool is_a = warp == 0;
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      uint32_t ready_mask = 0;
      for (long t = group; t < num_tiles && ok; t += num_groups) {
        GemmTile tile = gemm_tile(t, tiles_m, tiles_n, tiles_nt, p.panel);
        rotate_tile(tile, p, tiles_m);
        const int m0 = tile.tm * kWideTileM + int(cta_rank) * 128;  // row block 1 starts 256 rows further
        if (is_a && p.gather_copy) {
          // Rows that belong to another rank are read from the local copy once every CTA's
          // copier has delivered its slice of that rank's block.
          const int src = m0 / p.a_gather_rows;
          if (src != p.gather_rank && !((ready_mask >> src) & 1u)) {
            const long long start = clock64();
            bool arrived = false;
            while (!(arrived = ld_acquire_gpu(p.gather_done + src) >= int(gridDim.x))) {
              if (clock64() - start > p.wait_cycles) break;
              __nanosleep(128);
            }
            if (!arrived) {
              atomicCAS(status, kStatusOk, kStatusTimeoutFlag);
              ok = false;
              break;
            }
            fence_proxy_async();  // generic-proxy stores of the copiers before this thread's TMA loads
            ready_mask |= 1u << src;
          }
        }
        const int b_rows = tile.aux ? p.aux_n / CG : 128;
        const int n0 = tile.aux ? int(cta_rank) * b_rows : tile.tn * kGemmTileN + int(cta_rank) * b_rows;
        const CUtensorMap* mb = tile.aux ? &tmap_p : &tmap_b;
        const bool b_mn = tile.aux ? false : p.b_mn != 0;
        const uint32_t stage_tx = uint32_t(CG) * uint32_t(kWideABytes + b_rows * kGemmBlockK * 2);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_budget(&empty_bar[stage], phase ^ 1u, p.wait_cycles)) {
            atomicCAS(status, kStatusOk, kStatusTimeoutProducer);
            ok = false;
            break;
          }
          const uint32_t a_dst = smem_u32(tiles + stage * kWideStageBytes);
          if (is_a && leader) mbar_expect_tx(&full_bar[stage], stage_tx);
          const uint32_t bar = map_to_cta(smem_u32(&full_bar[stage]), 0);
          const int k0 = kb * kGemmBlockK;
          if (is_a) {
            load_operand<CG>(a_dst, &tmap_a, bar, p.a_mn != 0, p.a_blocked != 0, 128, m0, k0, tile.batch, three_d);
            load_operand<CG>(a_dst + 16384, &tmap_a, bar, p.a_mn != 0, p.a_blocked != 0, 128, m0 + 256, k0,
                             tile.batch, three_d);
          } else {
            load_operand<CG>(a_dst + kWideABytes, mb, bar, b_mn, p.b_blocked != 0, b_rows, n0, k0, tile.batch,
                             three_d && !tile.aux);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        // Give-up path: wait out in-flight loads (far above a TMA round trip) before the exit.
        const long long start = clock64();
        while (clock64() - start < 400000) {
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (leader) {
      uint32_t stage = 0, phase = 0;
      long local_tile = 0;
      bool ok = true;
      for (long t = group; t < num_tiles && ok; t += num_groups, ++local_tile) {
        const GemmTile tile = gemm_tile(t, tiles_m, tiles_n, tiles_nt, p.panel);
        const uint32_t acc_parity = (uint32_t(local_tile) & 1u) ^ 1u;  // first use: free
        const bool tracing = p.trace != nullptr && lane == 0 && group == 0;
        const long long t_begin = tracing ? clock64() : 0;
        long long full_wait = 0, t_acc1 = 0;
        ok = mbar_wait_budget(&tmem_empty_bar[0], acc_parity, p.wait_cycles);
        const long long t_acc0 = tracing ? clock64() : 0;
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) atomicCAS(status, kStatusOk, kStatusTimeoutMma);
          break;
        }
        tc_fence_after();
        const bool b_mn = tile.aux ? false : p.b_mn != 0;
        const int n_inst = tile.aux ? p.aux_n : kGemmTileN;
        const uint32_t idesc = make_idesc_f16(256, n_inst, FMT, p.a_mn, b_mn ? 1 : 0);
        const uint32_t a_step = p.a_mn ? 2048u : 32u, b_step = b_mn ? 2048u : 32u;
        for (int kb = 0; kb < num_kb; ++kb) {
          const long long w0 = tracing ? clock64() : 0;
          ok = mbar_wait_budget(&full_bar[stage], phase, p.wait_cycles);
          if (tracing) full_wait += clock64() - w0;
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) {
            if (lane == 0) atomicCAS(status, kStatusOk, kStatusTimeoutMma);
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + stage * kWideStageBytes);
          const uint32_t b_addr = a_addr + kWideABytes;
          const uint64_t da0 = p.a_mn ? make_mnmajor_sw128_desc(a_addr, 8192) : make_kmajor_sw128_desc(a_addr);
          const uint64_t da1 = da0 + uint64_t(16384 >> 4);
          const uint64_t db0 = b_mn ? make_mnmajor_sw128_desc(b_addr, 8192) : make_kmajor_sw128_desc(b_addr);
          if (lane == 0) {
#pragma unroll
            for (int k = 0; k < kGemmBlockK / 16; ++k)
              umma_f16_cg<CG>(tmem_base, da0 + uint64_t((a_step * k) >> 4), db0 + uint64_t((b_step * k) >> 4), idesc,
                              (kb | k) != 0 ? 1u : 0u);
          }
          if (kb == 0) {
            // The second row block's accumulator may still be draining from the previous tile.
            ok = mbar_wait_budget(&tmem_empty_bar[1], acc_parity, p.wait_cycles);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
              if (lane == 0) atomicCAS(status, kStatusOk, kStatusTimeoutMma);
              break;
            }
            tc_fence_after();
            if (tracing) t_acc1 = clock64();
          }
          if (lane == 0) {
#pragma unroll
            for (int k = 0; k < kGemmBlockK / 16; ++k)
              umma_f16_cg<CG>(tmem_base + kGemmTileN, da1 + uint64_t((a_step * k) >> 4),
                              db0 + uint64_t((b_step * k) >> 4), idesc, (kb | k) != 0 ? 1u : 0u);
            umma_commit_cg<CG>(&empty_bar[stage]);
          }
          __syncwarp();
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok && lane == 0) umma_commit_cg<CG>(tmem_full_bar);
        if (tracing) {
          long long* tr = p.trace + local_tile * 8;
          tr[0] = t_begin;
          tr[1] = t_acc0;
          tr[2] = clock64();
          tr[3] = full_wait;
          tr[7] = t_acc1;
        }
        __syncwarp();
      }
    }
  } else if (warp < 10) {
    // ---------------- epilogue: 8 warps, (lane quadrant) x (column half) ----------------
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;  // 0: columns 0..127 of each row block, 1: columns 128..255
    long local_tile = 0;
    bool ok = true;
    uint32_t empty_addr[2];
#pragma unroll
    for (int a = 0; a < 2; ++a) empty_addr[a] = map_to_cta(smem_u32(&tmem_empty_bar[a]), 0);
    for (long t = group; t < num_tiles && ok; t += num_groups, ++local_tile) {
      GemmTile tile = gemm_tile(t, tiles_m, tiles_n, tiles_nt, p.panel);
      rotate_tile(tile, p, tiles_m);
      const bool tracing = p.trace != nullptr && group == 0 && leader && warp == 2 && lane == 0;
      const long long e0 = tracing ? clock64() : 0;
      ok = mbar_wait_budget(tmem_full_bar, uint32_t(local_tile) & 1u, p.wait_cycles);
      const long long e1 = tracing ? clock64() : 0;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) atomicCAS(status, kStatusOk, kStatusTimeoutEpilogue);
        break;
      }
      tc_fence_after();
      const int col0 = tile.tn * kGemmTileN;
      const int n_valid = tile.aux ? 0 : (p.N - col0 < kGemmTileN ? p.N - col0 : kGemmTileN);
#pragma unroll 1
      for (int rb = 0; rb < 2; ++rb) {
        const long row = long(tile.tm) * kWideTileM + rb * 256 + long(cta_rank) * 128 + quad * 32 + lane;
        const bool row_ok = row < p.M;
        const uint32_t t_addr = tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(rb) * kGemmTileN;
        if (tile.aux) {
          if (half == 0) {
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
          }
        } else if (!OUT32 && p.tma_store) {
          // This warp's 32 rows x 128 columns go through its private staging slab (two 64-column
          // slabs in the 128-byte swizzle); TMA stores clip at the matrix edges.
          uint8_t* stg = staging + (warp - 2) * 8192;
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // earlier stores
          __syncwarp();
          const uint32_t stg_row = smem_u32(stg) + uint32_t(lane) * 128u;
#pragma unroll 1
          for (int cc = 0; cc < 128; cc += 32) {
            const int c = half * 128 + cc;
            if (c >= n_valid) break;  // uniform over the warp
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
            const uint32_t slab = stg_row + uint32_t(cc >> 6) * 4096u;
            const uint32_t chunk0 = uint32_t(cc & 63) >> 3;  // 16-byte chunk of the 128-byte row: 0 or 4
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              union { uint4 u; InT h[8]; } o;
#pragma unroll
              for (int e = 0; e < 8; ++e) o.h[e] = from_float<InT>(v[j * 8 + e]);
              const uint32_t addr = slab + (((chunk0 + j) ^ (uint32_t(lane) & 7u)) << 4);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(o.u.x), "r"(o.u.y),
                           "r"(o.u.z), "r"(o.u.w)
                           : "memory");
            }
          }
          // The accumulator slice is in shared memory: the row block can go back to the MMA warp
          // before a single byte has reached global memory.
          tc_fence_before();
          fence_proxy_async();
          __syncwarp();
          const int row0 = tile.tm * kWideTileM + rb * 256 + int(cta_rank) * 128 + quad * 32;
          if (lane == 0) {
            mbar_arrive_cluster(empty_addr[rb]);
            if (row0 < p.M) {
              // Reduce-scatter form: these 32 rows go to their owner's buffer (a peer mapping),
              // into this rank's slot, through that rank's tensor map.
              const CUtensorMap* md = &tmap_d;
              int row_dst = row0;
              if (p.d_scatter_rows > 0) {
                const int owner = row0 / p.d_scatter_rows;
                md = &peers.a[owner];
                row_dst = p.d_slot * p.d_scatter_rows + (row0 - owner * p.d_scatter_rows);
              }
              for (int b = 0; b < 2; ++b) {
                const int c = half * 128 + b * 64;
                if (c >= n_valid) break;
                asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                                 reinterpret_cast<uint64_t>(md)),
                             "r"(smem_u32(stg) + uint32_t(b) * 4096u), "r"(col0 + c), "r"(row_dst)
                             : "memory");
              }
            }
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
          if (tracing) p.trace[local_tile * 8 + 5 + rb] = clock64();
          continue;  // this row block is done (barrier arrival included)
        } else {
          long d_row_off = long(tile.batch) * p.d_batch_stride + row * p.ldd + col0;
          void* d_base = p.d;
          if (p.d_scatter_rows > 0 && row_ok) {  // the row's owner receives it in this rank's slot
            const int owner = int(row / p.d_scatter_rows);
            d_base = p.d_peers[owner];
            d_row_off = (long(p.d_slot) * p.d_scatter_rows + (row - long(owner) * p.d_scatter_rows)) * p.ldd + col0;
          }
#pragma unroll 1
          for (int cc = 0; cc < 128; cc += 32) {
            const int c = half * 128 + cc;
            if (c >= n_valid) break;  // uniform over the warp
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
              } else if (nv == 32 && (reinterpret_cast<uintptr_t>(dst) & 31) == 0) {
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                  uint32_t o[8];
#pragma unroll
                  for (int j = 0; j < 8; ++j) {
                    float x = v[i + j];
                    if (p.accumulate) x += dst[i + j];
                    o[j] = __float_as_uint(x);
                  }
                  st_global_v8(dst + i, o);
                }
              } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                  if (i < nv) dst[i] = p.accumulate ? dst[i] + v[i] : v[i];
              }
            } else {
              InT* dst = reinterpret_cast<InT*>(d_base) + d_row_off + c;
              if (nv == 32 && (reinterpret_cast<uintptr_t>(dst) & 31) == 0) {
#pragma unroll
                for (int i = 0; i < 32; i += 16) {
                  union { uint32_t u[8]; InT h[16]; } o;
                  if (p.accumulate) {
                    const uint4 lo = *reinterpret_cast<const uint4*>(dst + i);
                    const uint4 hi = *reinterpret_cast<const uint4*>(dst + i + 8);
                    o.u[0] = lo.x; o.u[1] = lo.y; o.u[2] = lo.z; o.u[3] = lo.w;
                    o.u[4] = hi.x; o.u[5] = hi.y; o.u[6] = hi.z; o.u[7] = hi.w;
#pragma unroll
                    for (int j = 0; j < 16; ++j) o.h[j] = from_float<InT>(to_float<InT>(o.h[j]) + v[i + j]);
                  } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) o.h[j] = from_float<InT>(v[i + j]);
                  }
                  st_global_v8(dst + i, o.u);
                }
              } else if (nv == 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
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
        // This warp's reads of row block `rb` are complete: hand the block back to the MMA warp.
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(empty_addr[rb]);
        if (tracing) p.trace[local_tile * 8 + 5 + rb] = clock64();
      }
      if (tracing) p.trace[local_tile * 8 + 4] = e1;
      (void)e0;
    }
  }

  else if (warp == 11 && p.gather_copy) {
    // ---------------- copier: this CTA's slice of every other rank's row block ----------------
    const long n_vec = long(p.a_gather_rows) * p.K / 8;  // 16-byte packets per rank block
    const long per = (n_vec + gridDim.x - 1) / gridDim.x;
    const long lo = long(blockIdx.x) * per;
    const long hi = lo + per < n_vec ? lo + per : n_vec;
    for (int s = 1; s < p.gather_world; ++s) {
      int r = p.gather_rank + s;
      if (r >= p.gather_world) r -= p.gather_world;
      const uint4* src = reinterpret_cast<const uint4*>(p.gather_src[r]);
      uint4* dst = reinterpret_cast<uint4*>(p.d_gather_dst) + long(r) * n_vec;
      constexpr int kInFlight = 16;
      for (long i = lo + lane; i < hi; i += 32 * kInFlight) {
        uint4 v[kInFlight];
#pragma unroll
        for (int j = 0; j < kInFlight; ++j)
          if (i + 32 * j < hi) v[j] = ld_volatile_v4(src + i + 32 * j);
#pragma unroll
        for (int j = 0; j < kInFlight; ++j)
          if (i + 32 * j < hi) dst[i + 32 * j] = v[j];
      }
      __syncwarp();
      __threadfence();
      if (lane == 0) atomicAdd(p.gather_done + r, 1);
    }
  }

  if (warp >= 2 && warp < 10 && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer may still be reading this CTA's operands
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_cg<CG>(tmem_base, 512);
  }
}

}  // namespace bgn
