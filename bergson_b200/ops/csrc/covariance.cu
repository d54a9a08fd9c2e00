// Kronecker-factor covariance  C += X^T X  for X [T, D] (bf16/fp16, row-major) on tcgen05.
//
// Both MMA operands are the same matrix read "MN-major" (the D axis is contiguous, the
// reduction runs over the token rows), so a TMA box of 64 columns x 64 rows with the
// 128-byte swizzle is directly a canonical MN-major UMMA tile.  Output tiles are 128 rows x 256
// columns; only tiles that touch the upper triangle are computed (the caller mirrors them).  The token range is split over
// gridDim.y CTAs per tile and partial tiles are added to the fp32 output with vector
// reductions, so one launch fills the machine even for D = 768.
//
// Reduce-scatter fusion: the epilogue resolves every output row to the rank that owns it
// (row shards, rank 0 takes the remainder) and adds into that rank's buffer through its
// peer pointer (plain P2P `red.global.add`).  With one rank this degenerates to local adds.
#include "common.cuh"
#include "kernels_cov.h"

#include <mutex>

namespace bgn {

constexpr int kCovBlock = 128;    // output tile rows (MMA M)
constexpr int kCovBlockN = 256;   // output tile columns (MMA N): halves the shared-memory
                                  // bytes read per flop relative to a 128 x 128 tile
constexpr int kCovBlockK = 64;    // token rows per stage
constexpr int kCovBoxBytes = 64 * kCovBlockK * 2;       // one 64-column box
constexpr int kCovABytes = (kCovBlock / 64) * kCovBoxBytes;
constexpr int kCovBBytes = (kCovBlockN / 64) * kCovBoxBytes;
constexpr int kCovStageBytes = kCovABytes + kCovBBytes;
constexpr int kCovStages = 4;
constexpr int kCovThreads = 192;
constexpr int kCovSmemBytes = kCovStages * kCovStageBytes + 1024 + 256;

struct CovParams {
  float* dst[8];       // per-rank destination buffers (row shards), peer-mapped
  int row_start[9];    // row_start[r]..row_start[r+1] = rows owned by rank r
  const float* local;  // optional local accumulator to fold in (flush step), [D, D]
  int world;
  int D;
  long T;
  int tiles_m;         // 128-row tile rows
  int tiles_n;         // 256-column tile columns
  int full;            // 1: every tile is visited (used when the destination must end up
                       // holding complete rows, e.g. the cross-rank reduce-scatter)
  int local_upper;     // 1: `local` holds valid values only in the tiles that touch the upper
                       // triangle (it was filled by non-full launches); elements of the other
                       // tiles are read from their mirror position
};

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c),
               "f"(d)
               : "memory");
}

template <int FMT>
__global__ void __launch_bounds__(kCovThreads, 1)
cov_syrk_kernel(const __grid_constant__ CUtensorMap tmap, CovParams p, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                              ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(tiles + kCovStages * kCovStageBytes);
  uint64_t* empty_bar = full_bar + kCovStages;
  uint64_t* tmem_full_bar = empty_bar + kCovStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_full_bar + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // blockIdx.x enumerates, row by row, the tiles that touch the upper triangle: tile row tm
  // starts at tile column tm / 2 (a 256-wide column block covers two 128-high row blocks).
  int tm = 0, rem = blockIdx.x;
  while (true) {
    const int width = p.full ? p.tiles_n : p.tiles_n - tm / 2;
    if (rem < width) break;
    rem -= width;
    ++tm;
  }
  const int tn = (p.full ? 0 : tm / 2) + rem;

  const long kb_total = (p.T + kCovBlockK - 1) / kCovBlockK;
  const long kb_per = (kb_total + gridDim.y - 1) / gridDim.y;
  const long kb_begin = kb_per * blockIdx.y;
  long kb_end = kb_begin + kb_per;
  if (kb_end > kb_total) kb_end = kb_total;
  const int num_kb = kb_end > kb_begin ? int(kb_end - kb_begin) : 0;
  const bool fold_local = p.local != nullptr && blockIdx.y == 0;
  if (num_kb == 0 && !fold_local) return;  // uniform per CTA: nothing allocated yet

  if (threadIdx.x == 0) {
    for (int s = 0; s < kCovStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(tmem_full_bar, 1);
    fence_barrier_init();
    tma_prefetch_desc(&tmap);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kCovBlockN);
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
      for (int i = 0; i < num_kb; ++i) {
        const int s = i % kCovStages;
        if (!mbar_wait_bounded(&empty_bar[s], ((i / kCovStages) & 1) ^ 1)) {
          atomicCAS(status, kStatusOk, kStatusTimeoutProducer);
          ok = false;
          break;
        }
        uint8_t* a_dst = tiles + s * kCovStageBytes;
        uint8_t* b_dst = a_dst + kCovABytes;
        const int row = int((kb_begin + i) * kCovBlockK);
        mbar_expect_tx(&full_bar[s], kCovStageBytes);
#pragma unroll
        for (int b = 0; b < kCovBlock / 64; ++b)
          tma_load_2d(a_dst + b * kCovBoxBytes, &tmap, &full_bar[s], tm * kCovBlock + b * 64, row);
#pragma unroll
        for (int b = 0; b < kCovBlockN / 64; ++b)
          tma_load_2d(b_dst + b * kCovBoxBytes, &tmap, &full_bar[s], tn * kCovBlockN + b * 64, row);
        issued = i + 1;
      }
      if (!ok) {
        for (int i = issued > kCovStages ? issued - kCovStages : 0; i < issued; ++i)
          mbar_wait_bounded(&full_bar[i % kCovStages], (i / kCovStages) & 1);
      }
    }
  } else if (warp == 1) {
    constexpr uint32_t idesc = make_idesc_f16(kCovBlock, kCovBlockN, FMT, 1, 1);
    bool ok = true;
    for (int i = 0; i < num_kb && ok; ++i) {
      const int s = i % kCovStages;
      ok = mbar_wait_bounded(&full_bar[s], (i / kCovStages) & 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) atomicCAS(status, kStatusOk, kStatusTimeoutMma);
        break;
      }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t a_addr = smem_u32(tiles + s * kCovStageBytes);
        const uint32_t b_addr = a_addr + kCovABytes;
#pragma unroll
        for (int k = 0; k < kCovBlockK / 16; ++k) {
          // 16 token rows = two 8-row swizzle groups = 2048 bytes further into each box.
          const uint64_t da = make_mnmajor_sw128_desc(a_addr + k * 2048, kCovBoxBytes);
          const uint64_t db = make_mnmajor_sw128_desc(b_addr + k * 2048, kCovBoxBytes);
          umma_f16(tmem_base, da, db, idesc, (i | k) != 0 ? 1u : 0u);
        }
        umma_commit(&empty_bar[s]);
      }
      __syncwarp();
    }
    if (lane == 0) umma_commit(tmem_full_bar);
    __syncwarp();
  } else {
    const int quad = warp & 3;
    bool ok = true;
    if (num_kb > 0) {
      ok = mbar_wait_bounded(tmem_full_bar, 0);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok && lane == 0) atomicCAS(status, kStatusOk, kStatusTimeoutEpilogue);
    }
    tc_fence_after();
    const int r = tm * kCovBlock + quad * 32 + lane;  // global output row of this thread
    if (ok) {
      // Owner of row r and its destination row pointer.
      int owner = 0;
      while (owner + 1 < p.world && r >= p.row_start[owner + 1]) ++owner;
      float* drow = nullptr;
      if (r < p.D) drow = p.dst[owner] + long(r - p.row_start[owner]) * p.D;
#pragma unroll 1
      for (int c = 0; c < kCovBlockN; c += 16) {
        float acc[16];
        if (num_kb > 0) {
          tmem_ld_32x16(tmem_base + (uint32_t(quad * 32) << 16) + c, acc);
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) acc[i] = 0.f;
        }
        const int col = tn * kCovBlockN + c;
        if (drow == nullptr || col >= p.D) continue;
        if (fold_local) {
          if (!p.local_upper || tn >= tm / 2) {
            const float* lrow = p.local + long(r) * p.D + col;
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (col + i < p.D) acc[i] += lrow[i];
          } else {
            // mirror: the accumulator is symmetric and only its upper tiles were computed
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (col + i < p.D) acc[i] += p.local[long(col + i) * p.D + r];
          }
        }
        if (col + 16 <= p.D && (p.D & 3) == 0) {
#pragma unroll
          for (int i = 0; i < 16; i += 4)
            red_add_v4(drow + col + i, acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (col + i < p.D) atomicAdd(drow + col + i, acc[i]);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kCovBlockN);
  }
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn cov_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

}  // namespace bgn

using namespace bgn;

extern "C" int bgn_cov_syrk(const void* x, long T, int D, int fmt, float* const* dst, const int* row_start,
                            int world, const float* local, int full, int local_upper, int sm_count, int* status,
                            cudaStream_t stream) {
  if (D % 8 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) || world < 1 || world > 8)
    return int(cudaErrorInvalidValue);
  if (T <= 0 && local == nullptr) return 0;
  ensure_context_bound();
  EncodeTiledFn enc = cov_encode_fn();
  if (!enc) return int(cudaErrorInvalidValue);
  CUtensorMap tmap;
  // A zero-row view would be rejected by the encoder; the fold-only launch still needs a map.
  cuuint64_t dims[2] = {cuuint64_t(D), cuuint64_t(T > 0 ? T : 1)};
  cuuint64_t strides[1] = {cuuint64_t(D) * 2};
  cuuint32_t box[2] = {64, cuuint32_t(kCovBlockK)};
  cuuint32_t estr[2] = {1, 1};
  if (enc(&tmap, fmt == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
          const_cast<void*>(x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return int(cudaErrorInvalidValue);

  CovParams p;
  for (int r = 0; r < 8; ++r) p.dst[r] = r < world ? dst[r] : nullptr;
  for (int r = 0; r <= 8; ++r) p.row_start[r] = r <= world ? row_start[r] : D;
  p.local = local;
  p.world = world;
  p.D = D;
  p.T = T > 0 ? T : 0;
  p.tiles_m = (D + kCovBlock - 1) / kCovBlock;
  p.tiles_n = (D + kCovBlockN - 1) / kCovBlockN;
  p.full = full ? 1 : 0;
  p.local_upper = local_upper ? 1 : 0;
  int tiles = 0;
  for (int tm = 0; tm < p.tiles_m; ++tm) tiles += p.full ? p.tiles_n : p.tiles_n - tm / 2;
  const long kb_total = (p.T + kCovBlockK - 1) / kCovBlockK;
  // Split the token range so that the grid covers the SMs, keeping >= 8 k-blocks per CTA.
  long splits = (sm_count + tiles - 1) / tiles;
  if (splits > kb_total / 8) splits = kb_total / 8;
  if (splits < 1) splits = 1;

  static bool attr_set[2] = {false, false};
  auto kern = fmt == 1 ? cov_syrk_kernel<1> : cov_syrk_kernel<0>;
  if (!attr_set[fmt]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kCovSmemBytes);
    if (e != cudaSuccess) return int(e);
    attr_set[fmt] = true;
  }
  kern<<<dim3(tiles, unsigned(splits)), kCovThreads, kCovSmemBytes, stream>>>(tmap, p, status);
  return int(cudaGetLastError());
}
