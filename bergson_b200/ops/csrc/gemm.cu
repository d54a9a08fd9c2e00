// Host side of the persistent tcgen05 GEMM (gemm.cuh): tensor maps for the four operand
// layouts, grid sizing, and the cluster launch of the CTA-pair variant.
#include "gemm.cuh"
#include "gemm_wide.cuh"

#include <mutex>

#include "kernels_gemm.h"

namespace bgn {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn gemm_encode_fn() {
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

// Row-major 16-bit tensor [batch, rows, inner] with row stride `ld` and batch stride `bs`
// (elements); box = 64 x box_rows x 1 with the 128-byte swizzle.
static bool gemm_tmap(CUtensorMap* map, const void* base, int fmt, uint64_t inner, uint64_t rows, uint64_t batch,
                      uint64_t ld, uint64_t bs, uint32_t box_rows) {
  ensure_context_bound();
  EncodeTiledFn enc = gemm_encode_fn();
  if (!enc || (reinterpret_cast<uintptr_t>(base) & 15) || (ld % 8) || (batch > 1 && bs % 8)) return false;
  const CUtensorMapDataType dt = fmt == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  cuuint64_t dims[3] = {inner, rows, batch > 1 ? batch : 1};
  cuuint64_t strides[2] = {ld * 2, (batch > 1 ? bs : ld * rows) * 2};
  cuuint32_t box[3] = {64, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return enc(map, dt, batch > 1 ? 3 : 2, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// MN-major operand [batch, K, mn] (mn contiguous, a multiple of 64) viewed as
// (64 mn-in-block, K, mn / 64 blocks[, batch]); box = 64 x 64 x blocks x 1, so one load brings
// `blocks` consecutive 64-wide column blocks, each as its own 8 KB swizzled slab.
static bool gemm_tmap_blocked(CUtensorMap* map, const void* base, int fmt, uint64_t mn, uint64_t K, uint64_t batch,
                              uint64_t ld, uint64_t bs, uint32_t blocks) {
  ensure_context_bound();
  EncodeTiledFn enc = gemm_encode_fn();
  if (!enc || (reinterpret_cast<uintptr_t>(base) & 15) || (ld % 8) || (batch > 1 && bs % 8) || (mn % 64)) return false;
  const CUtensorMapDataType dt = fmt == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  cuuint64_t dims[4] = {64, K, mn / 64, batch > 1 ? batch : 1};
  cuuint64_t strides[3] = {ld * 2, 128, (batch > 1 ? bs : ld * K) * 2};
  cuuint32_t box[4] = {64, 64, blocks, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return enc(map, dt, batch > 1 ? 4 : 3, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int CG, int FMT, bool OUT32>
static cudaError_t launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tp, const CUtensorMap& td,
                               const GemmPeerMaps& peers, const GemmParams& p, int grid, int* status,
                               cudaStream_t stream) {
  auto kern = gemm_kernel<CG, FMT, OUT32>;
  static bool attr_set = false;  // one flag per instantiation
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmemV2<CG>::kBytes);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(kGemmThreadsV2, 1, 1);
  cfg.dynamicSmemBytes = GemmSmemV2<CG>::kBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CG;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, ta, tb, tp, td, peers, p, status);
}

template <int FMT, bool OUT32>
static cudaError_t launch_gemm_wide(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tp,
                                    const CUtensorMap& td, const GemmPeerMaps& peers, const GemmParams& p, int grid,
                                    int* status, cudaStream_t stream) {
  auto kern = gemm_wide_kernel<FMT, OUT32>;
  static bool attr_set = false;  // one flag per instantiation
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kWideSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(kWideThreads, 1, 1);
  cfg.dynamicSmemBytes = kWideSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, ta, tb, tp, td, peers, p, status);
}

}  // namespace bgn

using namespace bgn;

extern "C" int bgn_gemm(const BgnGemmArgs* a, int* status, cudaStream_t stream) {
  if (!a || a->M <= 0 || a->N <= 0 || a->K <= 0 || a->batch < 1) return int(cudaErrorInvalidValue);
  const int cg = a->cta_group == 2 ? 2 : 1;
  if (a->aux_n < 0 || a->aux_n > 64 || a->aux_n % 16) return int(cudaErrorInvalidValue);
  if (a->sq_accumulate && !a->out_f32) return int(cudaErrorInvalidValue);
  CUtensorMap ta, tb, tp;
  static GemmPeerMaps no_peers;  // zero-initialised placeholder when A is not gathered
  GemmPeerMaps gathered;
  const bool gather = a->gather_world > 0, scatter = a->scatter_world > 0;
  if (gather || scatter) {
    if (a->batch != 1 || a->a_mn || a->out_f32 || a->accumulate || a->sq_accumulate) return int(cudaErrorInvalidValue);
    if (gather && (a->gather_world > kGemmMaxPeers || a->gather_rows % 128 ||
                   long(a->gather_world) * a->gather_rows != a->M))
      return int(cudaErrorInvalidValue);
    if (gather && a->gather_copy &&
        (a->gather_rows % kWideTileM || a->lda != a->K || !a->gather_done || a->gather_rank < 0 ||
         a->gather_rank >= a->gather_world || cg != 2 || !a->wide || !a->a))
      return int(cudaErrorInvalidValue);
    if (scatter && (a->scatter_world > kGemmMaxPeers || a->scatter_rows <= 0 || a->scatter_slot < 0 ||
                    a->scatter_slot >= a->scatter_world || long(a->scatter_world) * a->scatter_rows < a->M))
      return int(cudaErrorInvalidValue);
  }
  const uint64_t B = uint64_t(a->batch);
  // A: K-major [M, K] (box 64 k x 128 rows) or MN-major [K, M] (64 m x 64 k slabs; one blocked
  // load when M is a multiple of 64, else one load per slab).
  const bool a_blocked = a->a_mn && a->M % 64 == 0;
  const bool b_blocked = a->b_mn && a->N % 64 == 0;
  const bool gather_copy = gather && a->gather_copy;
  if (gather && !gather_copy) {
    for (int r = 0; r < a->gather_world; ++r)
      if (!gemm_tmap(&gathered.a[r], a->a_peers[r], a->fmt, a->K, a->gather_rows, 1, a->lda, 0, 128))
        return int(cudaErrorInvalidPitchValue);
  }
  const void* a_base = gather && !gather_copy ? a->a_peers[0] : a->a;
  const uint64_t a_rows = gather && !gather_copy ? uint64_t(a->gather_rows) : uint64_t(a->M);
  const bool ok_a = !a->a_mn ? gemm_tmap(&ta, a_base, a->fmt, a->K, a_rows, B, a->lda, a->a_batch_stride, 128)
                    : a_blocked ? gemm_tmap_blocked(&ta, a->a, a->fmt, a->M, a->K, B, a->lda, a->a_batch_stride, 2)
                                : gemm_tmap(&ta, a->a, a->fmt, a->M, a->K, B, a->lda, a->a_batch_stride, 64);
  const bool ok_b = !a->b_mn ? gemm_tmap(&tb, a->b, a->fmt, a->K, a->N, B, a->ldb, a->b_batch_stride, kGemmTileN / cg)
                    : b_blocked ? gemm_tmap_blocked(&tb, a->b, a->fmt, a->N, a->K, B, a->ldb, a->b_batch_stride,
                                                    kGemmTileN / cg / 64)
                                : gemm_tmap(&tb, a->b, a->fmt, a->N, a->K, B, a->ldb, a->b_batch_stride, 64);
  // Distinct codes tell the caller which operand's layout was rejected (alignment, strides).
  if (!ok_a) return int(cudaErrorInvalidPitchValue);
  if (!ok_b) return int(cudaErrorInvalidSymbol);
  if (a->aux_n > 0) {
    if (!a->aux_p || !a->aux_out || !gemm_tmap(&tp, a->aux_p, a->fmt, a->K, a->aux_n, 1, a->K, 0, a->aux_n / cg))
      return int(cudaErrorInvalidTexture);
  } else {
    tp = tb;
  }
  GemmParams p;
  p.M = a->M; p.N = a->N; p.K = a->K;
  p.a_mn = a->a_mn ? 1 : 0; p.b_mn = a->b_mn ? 1 : 0;
  p.d = a->d; p.ldd = a->ldd;
  p.bias = a->bias; p.bias_f32 = a->bias_f32;
  p.accumulate = a->accumulate;
  p.aux_n = a->aux_n; p.aux_out = a->aux_out; p.aux_ld = a->aux_n;
  p.batch = a->batch; p.d_batch_stride = a->d_batch_stride; p.sq_accumulate = a->sq_accumulate;
  p.wait_cycles = a->wait_cycles > 0 ? a->wait_cycles : kMaxWaitCycles;
  p.trace = a->trace;
  // 16-bit outputs that are simply overwritten go through shared-memory staging and TMA stores
  // (box 64 columns x 32 rows); anything else is written from registers.
  CUtensorMap td = ta;
  p.tma_store = 0;
  p.a_gather_rows = gather ? a->gather_rows : 0;
  p.gather_copy = gather_copy ? 1 : 0;
  p.gather_rank = gather_copy ? a->gather_rank : 0;
  p.gather_world = gather_copy ? a->gather_world : 0;
  p.tm_shift = gather_copy ? a->gather_rank * (a->gather_rows / kWideTileM) : 0;
  p.gather_done = gather_copy ? a->gather_done : nullptr;
  p.d_gather_dst = gather_copy ? const_cast<void*>(a->a) : nullptr;
  for (int r = 0; r < kGemmMaxPeers; ++r) p.gather_src[r] = gather_copy && r < a->gather_world ? a->a_peers[r] : nullptr;
  p.d_scatter_rows = scatter ? a->scatter_rows : 0;
  p.d_slot = scatter ? a->scatter_slot : 0;
  for (int r = 0; r < kGemmMaxPeers; ++r) p.d_peers[r] = scatter && r < a->scatter_world ? a->d_peers[r] : nullptr;
  if (!a->out_f32 && !a->accumulate && a->batch == 1 && !a->no_tma_store && !scatter) {
    EncodeTiledFn enc = gemm_encode_fn();
    if (enc && (reinterpret_cast<uintptr_t>(a->d) & 15) == 0 && a->ldd % 8 == 0) {
      cuuint64_t dims[2] = {cuuint64_t(a->N), cuuint64_t(a->M)};
      cuuint64_t strides[1] = {cuuint64_t(a->ldd) * 2};
      cuuint32_t box[2] = {64, 32};
      cuuint32_t estr[2] = {1, 1};
      const CUtensorMapDataType dt = a->fmt == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
      if (enc(&td, dt, 2, a->d, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS)
        p.tma_store = 1;
    }
  }
  p.a_blocked = a_blocked ? 1 : 0;
  p.b_blocked = b_blocked ? 1 : 0;
  // Reduce-scatter through the wide kernel's staged epilogue: one output map per owner, each
  // over that rank's [world slots x rows, N] slot region; TMA stores may target peer memory.
  GemmPeerMaps scatter_maps;
  bool scatter_tma = false;
  if (scatter && cg == 2 && a->wide && !a->no_tma_store && a->scatter_rows % 32 == 0 &&
      long(a->scatter_world) * a->scatter_rows == a->M && a->ldd % 8 == 0) {
    EncodeTiledFn enc = gemm_encode_fn();
    scatter_tma = enc != nullptr;
    for (int o = 0; o < a->scatter_world && scatter_tma; ++o) {
      cuuint64_t dims[2] = {cuuint64_t(a->N), cuuint64_t(a->scatter_world) * cuuint64_t(a->scatter_rows)};
      cuuint64_t strides[1] = {cuuint64_t(a->ldd) * 2};
      cuuint32_t box[2] = {64, 32};
      cuuint32_t estr[2] = {1, 1};
      const CUtensorMapDataType dt = a->fmt == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
      scatter_tma = (reinterpret_cast<uintptr_t>(a->d_peers[o]) & 15) == 0 &&
                    enc(&scatter_maps.a[o], dt, 2, a->d_peers[o], dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    }
    if (scatter_tma) p.tma_store = 1;
  }

  // The pair kernel reads gathered rows straight from the peers; the wide kernel has the
  // gather-with-copy form and the scatter epilogue.
  const bool wide = cg == 2 && a->wide && (!gather || gather_copy);
  const int tile_m = wide ? kWideTileM : 128 * cg;
  const long tiles_m = (a->M + tile_m - 1) / tile_m;
  const long tiles_n = (a->N + kGemmTileN - 1) / kGemmTileN + (a->aux_n > 0 ? 1 : 0);
  const long tiles = tiles_m * tiles_n * a->batch;
  // Rasterisation panel: as many tile columns as keep the panel's B slab (256 K-long rows per
  // column) around 32 MB, so that it stays in L2 while the tile rows stream past it.
  long panel = a->panel > 0 ? a->panel : (32l << 20) / (long(kGemmTileN) * a->K * 2);
  if (panel < 2) panel = 2;
  if (panel > 16 && a->panel <= 0) panel = 16;
  if (panel > tiles_n) panel = tiles_n;
  // Keep the aux column in a panel with real columns: alone in a last panel of its own it would
  // stream every slab of A from memory once more.
  if (a->aux_n > 0 && panel < tiles_n && tiles_n % panel == 1) ++panel;
  p.panel = int(panel);
  long groups = a->sm_count / cg;
  if (groups < 1) groups = 1;
  if (groups > tiles) groups = tiles;
  const int grid = int(groups) * cg;
  cudaError_t e;
  const bool bf = a->fmt == 1;
  const GemmPeerMaps& pm = gather && !gather_copy ? gathered : no_peers;
  const GemmPeerMaps& wide_pm = scatter_tma ? scatter_maps : no_peers;
  if (wide) {
    e = a->out_f32 ? (bf ? launch_gemm_wide<1, true>(ta, tb, tp, td, wide_pm, p, grid, status, stream)
                         : launch_gemm_wide<0, true>(ta, tb, tp, td, wide_pm, p, grid, status, stream))
                   : (bf ? launch_gemm_wide<1, false>(ta, tb, tp, td, wide_pm, p, grid, status, stream)
                         : launch_gemm_wide<0, false>(ta, tb, tp, td, wide_pm, p, grid, status, stream));
  } else if (cg == 2) {
    e = a->out_f32 ? (bf ? launch_gemm<2, 1, true>(ta, tb, tp, td, pm, p, grid, status, stream)
                         : launch_gemm<2, 0, true>(ta, tb, tp, td, pm, p, grid, status, stream))
                   : (bf ? launch_gemm<2, 1, false>(ta, tb, tp, td, pm, p, grid, status, stream)
                         : launch_gemm<2, 0, false>(ta, tb, tp, td, pm, p, grid, status, stream));
  } else {
    e = a->out_f32 ? (bf ? launch_gemm<1, 1, true>(ta, tb, tp, td, pm, p, grid, status, stream)
                         : launch_gemm<1, 0, true>(ta, tb, tp, td, pm, p, grid, status, stream))
                   : (bf ? launch_gemm<1, 1, false>(ta, tb, tp, td, pm, p, grid, status, stream)
                         : launch_gemm<1, 0, false>(ta, tb, tp, td, pm, p, grid, status, stream));
  }
  return int(e);
}
