// Per-example projected Linear gradients on tcgen05 tensor cores.
//
// The stored quantity for one Linear and one example n is  P_out (G_n^T A_n) P_in^T  in
// R^{p x p} (p = 16), computed as (G_n P_out^T)^T (A_n P_in^T): two skinny GEMMs with N = 16
// that are bound by streaming A and G once from HBM, and a 16 x S x 16 contraction over the
// example's tokens.  Optimizer (Adafactor) row/column scales are folded into P_out / P_in by
// the caller, so they cost nothing here.
//
//   bgn_proj_right      : A' = A P_in^T                       (forward hook)
//   bgn_proj_left_outer : acc[n] += (G_n P_out^T)^T A'_n      (backward hook; G' never
//                         leaves the SM: TMEM -> registers -> shared memory -> 16x16 sum)
//   bgn_finalize_rows   : clamp / unit-norm / cast the fp32 accumulator rows into the store
//                         dtype, scattering by dataset index.
#include "kernels.h"
#include "tn_gemm.cuh"

#include <mutex>

namespace bgn {

// ---- tensor-map construction ------------------------------------------------------------

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
  });
  return fn;
}

// Row-major 16-bit tensor viewed as (K contiguous, rows, batch); box = 64 x box_rows x 1.
static bool make_tmap_3d(CUtensorMap* map, const void* base, int fmt, uint64_t K, uint64_t rows,
                         uint64_t batch, uint32_t box_rows) {
  ensure_context_bound();
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return false;
  cuuint64_t dims[3] = {K, rows, batch};
  cuuint64_t strides[2] = {K * 2, K * rows * 2};
  cuuint32_t box[3] = {uint32_t(kBlockK), box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMapDataType dt = fmt == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  return enc(map, dt, 3, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static bool make_tmap_2d(CUtensorMap* map, const void* base, int fmt, uint64_t K, uint64_t rows,
                         uint32_t box_rows) {
  ensure_context_bound();
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return false;
  cuuint64_t dims[2] = {K, rows};
  cuuint64_t strides[1] = {K * 2};
  cuuint32_t box[2] = {uint32_t(kBlockK), box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = fmt == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  return enc(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// ---- epilogues --------------------------------------------------------------------------

// Plain fp32 store: thread `row` owns one output row and writes 16 contiguous floats.
struct StoreF32Epilogue {
  float* out;
  long ld;
  int rows;

  __device__ __forceinline__ void operator()(int row, int c, const float (&acc)[16], int tile_m,
                                             int out_col0, int n_valid, int batch, void*) const {
    const long r = long(tile_m) * kBlockM + row;
    if (r >= rows || c >= n_valid) return;
    float* dst = out + (long(batch) * rows + r) * ld + out_col0 + c;
    if (c + 16 <= n_valid && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
      for (int i = 0; i < 16; i += 4)
        *reinterpret_cast<float4*>(dst + i) = make_float4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i)
        if (c + i < n_valid) dst[i] = acc[i];
    }
  }
  __device__ __forceinline__ void finish(int, int, int, int, void*, bool) const {}
};

// G' tile (128 tokens x 16) meets A' (128 tokens x 16): out[i][j] = sum_t G'[t][i] A'[t][j],
// added atomically to the example's fp32 accumulator row.
struct OuterEpilogue {
  const float* a_proj;  // [N*S, 16]
  float* acc;           // [N, ld]
  long ld;
  long col_off;
  int S;

  static constexpr int kGStride = 17;  // padded to keep column reads conflict-free
  static constexpr int kSmemBytes = (kBlockM * kGStride + kBlockM * 16) * 4;

  __device__ __forceinline__ void operator()(int row, int c, const float (&v)[16], int tile_m, int,
                                             int, int batch, void* smem) const {
    float* gs = reinterpret_cast<float*>(smem);
    float* as = gs + kBlockM * kGStride;
#pragma unroll
    for (int i = 0; i < 16; ++i) gs[row * kGStride + i] = v[i];
    const int s = tile_m * kBlockM + row;
    float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0, a2 = a0, a3 = a0;
    if (s < S) {
      const float4* src = reinterpret_cast<const float4*>(a_proj + (long(batch) * S + s) * 16);
      a0 = __ldg(src);
      a1 = __ldg(src + 1);
      a2 = __ldg(src + 2);
      a3 = __ldg(src + 3);
    }
    float4* dst = reinterpret_cast<float4*>(as + row * 16);
    dst[0] = a0;
    dst[1] = a1;
    dst[2] = a2;
    dst[3] = a3;
    (void)c;
  }

  __device__ __forceinline__ void finish(int e, int, int, int batch, void* smem, bool ok) const {
    named_barrier_sync(1, 128);
    if (!ok) return;
    const float* gs = reinterpret_cast<const float*>(smem);
    const float* as = gs + kBlockM * kGStride;
    const int i = e >> 3, j = e & 7;
    float s0 = 0.f, s1 = 0.f;
#pragma unroll 8
    for (int t = 0; t < kBlockM; ++t) {
      const float g = gs[t * kGStride + i];
      s0 = fmaf(g, as[t * 16 + j], s0);
      s1 = fmaf(g, as[t * 16 + j + 8], s1);
    }
    float* dst = acc + long(batch) * ld + col_off + i * 16;
    atomicAdd(dst + j, s0);
    atomicAdd(dst + j + 8, s1);
  }
};

template <int BLOCK_N, int FMT, class Epi>
static cudaError_t launch_tn(const CUtensorMap& ta, const TmapSet& tb, TnGemmShape shape,
                             dim3 grid, Epi epi, int epi_smem, int* status, cudaStream_t stream) {
  using S = TnGemmSmem<BLOCK_N>;
  const int stages = S::stages(epi_smem);
  const int smem = stages * S::kStageBytes + 1024 + 256 + epi_smem;
  auto kern = tn_gemm_kernel<BLOCK_N, FMT, Epi>;
  static bool attr_set = false;  // one flag per template instantiation
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  kern<<<grid, kGemmThreads, smem, stream>>>(ta, tb, shape, stages, epi, status);
  return cudaGetLastError();
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace bgn

using namespace bgn;

extern "C" int bgn_proj_right(const void* a, const void* p, float* out, long T, int K, int fmt,
                              int* status, cudaStream_t stream) {
  if (K % 8 != 0 || !aligned16(a) || !aligned16(p) || T <= 0) return cudaErrorInvalidValue;
  CUtensorMap ta;
  TmapSet tb;
  if (!make_tmap_3d(&ta, a, fmt, K, T, 1, kBlockM)) return cudaErrorInvalidValue;
  if (!make_tmap_2d(&tb.m[0], p, fmt, K, 16, 16)) return cudaErrorInvalidValue;
  TnGemmShape shape{int(T), K, 16, 0};
  StoreF32Epilogue epi{out, 16, int(T)};
  dim3 grid((T + kBlockM - 1) / kBlockM, 1, 1);
  cudaError_t e = fmt == 1 ? launch_tn<16, 1>(ta, tb, shape, grid, epi, 0, status, stream)
                           : launch_tn<16, 0>(ta, tb, shape, grid, epi, 0, status, stream);
  return int(e);
}

extern "C" int bgn_proj_left_outer(const void* g, const void* p, const float* a_proj, float* acc,
                                   int N, int S, int K, long ld, long col_off, int fmt, int* status,
                                   cudaStream_t stream) {
  if (K % 8 != 0 || !aligned16(g) || !aligned16(p) || !aligned16(a_proj) || N <= 0 || S <= 0)
    return cudaErrorInvalidValue;
  CUtensorMap ta;
  TmapSet tb;
  if (!make_tmap_3d(&ta, g, fmt, K, S, N, kBlockM)) return cudaErrorInvalidValue;
  if (!make_tmap_2d(&tb.m[0], p, fmt, K, 16, 16)) return cudaErrorInvalidValue;
  TnGemmShape shape{S, K, 16, 0};
  OuterEpilogue epi{a_proj, acc, ld, col_off, S};
  dim3 grid((S + kBlockM - 1) / kBlockM, 1, N);
  cudaError_t e =
      fmt == 1 ? launch_tn<16, 1>(ta, tb, shape, grid, epi, OuterEpilogue::kSmemBytes, status, stream)
               : launch_tn<16, 0>(ta, tb, shape, grid, epi, OuterEpilogue::kSmemBytes, status, stream);
  return int(e);
}

extern "C" int bgn_tn_gemm(const void* a, const void* b, float* c, long M, int N, int K, long ldc,
                           int fmt, int* status, cudaStream_t stream) {
  if (K % 8 != 0 || !aligned16(a) || !aligned16(b) || M <= 0 || N <= 0) return cudaErrorInvalidValue;
  constexpr int BN = 256;
  CUtensorMap ta;
  TmapSet tb;
  if (!make_tmap_3d(&ta, a, fmt, K, M, 1, kBlockM)) return cudaErrorInvalidValue;
  if (!make_tmap_2d(&tb.m[0], b, fmt, K, N, BN)) return cudaErrorInvalidValue;
  TnGemmShape shape{int(M), K, N, 0};
  StoreF32Epilogue epi{c, ldc, int(M)};
  dim3 grid((M + kBlockM - 1) / kBlockM, (N + BN - 1) / BN, 1);
  cudaError_t e = fmt == 1 ? launch_tn<BN, 1>(ta, tb, shape, grid, epi, 0, status, stream)
                           : launch_tn<BN, 0>(ta, tb, shape, grid, epi, 0, status, stream);
  return int(e);
}

// c[M, world * N] = a[M, K] * [b_0; b_1; ...]^T where b_r [N, K] is rank r's buffer (this GPU's
// or peer-mapped): the all-gather of B is fused into the operand loads -- every CTA pulls
// the B tiles it needs straight from the owning GPU with plain TMA loads while the tensor
// cores work on the previous stage.
extern "C" int bgn_tn_gemm_gathered(const void* a, const void* const* b, int world, float* c, long M, int N,
                                    int K, long ldc, int fmt, int* status, cudaStream_t stream) {
  if (K % 8 != 0 || !aligned16(a) || M <= 0 || N <= 0 || world < 1 || world > 8) return cudaErrorInvalidValue;
  constexpr int BN = 256;
  CUtensorMap ta;
  TmapSet tb;
  if (!make_tmap_3d(&ta, a, fmt, K, M, 1, kBlockM)) return cudaErrorInvalidValue;
  for (int r = 0; r < world; ++r) {
    if (!aligned16(b[r]) || !make_tmap_2d(&tb.m[r], b[r], fmt, K, N, BN)) return cudaErrorInvalidValue;
  }
  const int tiles_per_src = (N + BN - 1) / BN;
  TnGemmShape shape{int(M), K, N, tiles_per_src};
  StoreF32Epilogue epi{c, ldc, int(M)};
  dim3 grid((M + kBlockM - 1) / kBlockM, world * tiles_per_src, 1);
  cudaError_t e = fmt == 1 ? launch_tn<BN, 1>(ta, tb, shape, grid, epi, 0, status, stream)
                           : launch_tn<BN, 0>(ta, tb, shape, grid, epi, 0, status, stream);
  return int(e);
}

// ---- row finalisation ---------------------------------------------------------------------

namespace bgn {

template <typename T>
__global__ void finalize_rows_kernel(const float* __restrict__ acc, T* __restrict__ out,
                                     const long* __restrict__ row_index, long D, long out_ld, float lo,
                                     float hi, int unit_norm) {
  const long r = blockIdx.x;
  const float* src = acc + r * D;
  T* dst = out + (row_index ? row_index[r] : r) * out_ld;
  float scale = 1.f;
  if (unit_norm) {
    float ss = 0.f;
    for (long i = threadIdx.x; i < D; i += blockDim.x) {
      const float v = to_float<T>(from_float<T>(fminf(fmaxf(src[i], lo), hi)));
      ss = fmaf(v, v, ss);
    }
    __shared__ float red[32];
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
      float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
      v = warp_sum(v);
      if (threadIdx.x == 0) red[0] = v;
    }
    __syncthreads();
    // rsqrt(max(sum of squares, eps_fp32^2))
    scale = rsqrtf(fmaxf(red[0], 1.4210854715202004e-14f));
  }
  for (long i = threadIdx.x; i < D; i += blockDim.x) {
    float v = fminf(fmaxf(src[i], lo), hi);
    if (unit_norm) v = to_float<T>(from_float<T>(v)) * scale;
    dst[i] = from_float<T>(v);
  }
}

}  // namespace bgn

extern "C" int bgn_finalize_rows(const float* acc, void* out, const long* row_index, int N, long D,
                                 long out_ld, float lo, float hi, int unit_norm, int out_type,
                                 cudaStream_t stream) {
  if (N <= 0) return 0;
  const int threads = 256;
  switch (out_type) {
    case 0:
      finalize_rows_kernel<__half><<<N, threads, 0, stream>>>(acc, (__half*)out, row_index, D, out_ld, lo, hi, unit_norm);
      break;
    case 1:
      finalize_rows_kernel<__nv_bfloat16><<<N, threads, 0, stream>>>(acc, (__nv_bfloat16*)out, row_index, D, out_ld, lo, hi, unit_norm);
      break;
    default:
      finalize_rows_kernel<float><<<N, threads, 0, stream>>>(acc, (float*)out, row_index, D, out_ld, lo, hi, unit_norm);
  }
  return int(cudaGetLastError());
}

// ---- per-example contraction of the projected operands ---------------------------------------
//
// The Linear layers' GEMMs emit A' = A P_in^T and G' = G P_out^T as fp32 side outputs ([T, ldp]
// with the first p columns meaningful).  The stored block of example n is
//   acc[n, col_off + i * p + j] = sum_s G'[n*S + s, i] * A'[n*S + s, j],
// formed here by one CTA per example in a fixed order (no atomics: two runs give the same bits).

namespace bgn {

constexpr int kContractThreads = 1024;
constexpr int kContractChunk = 64;  // tokens staged per step and group

template <int P>
__global__ void __launch_bounds__(kContractThreads)
proj_contract_kernel(const float* __restrict__ g_proj, const float* __restrict__ a_proj, float* __restrict__ acc,
                     float* __restrict__ partials, int* __restrict__ counters, int S, int ldp, long ld, long col_off) {
  // grid = (examples, splits): CTA (n, k) contracts the k-th slice of example n's tokens into a
  // p x p partial; the last CTA of an example to finish adds the partials up in slice order (so
  // the result does not depend on which CTA that was) and writes the block.
  constexpr int kOut = P * P;
  constexpr int kGroups = kOut >= kContractThreads ? 1 : (kContractThreads / kOut > 4 ? 4 : kContractThreads / kOut);
  constexpr int kPerThread = kOut >= kContractThreads ? kOut / kContractThreads : 1;
  __shared__ float gs[kGroups][kContractChunk][P + 1];
  __shared__ float as[kGroups][kContractChunk][P + 1];
  __shared__ float red[kGroups][kOut >= kContractThreads ? 1 : kOut];
  __shared__ int is_last;
  const int n = blockIdx.x, split = blockIdx.y, splits = gridDim.y;
  const int tid = threadIdx.x;
  const int grp = kOut >= kContractThreads ? 0 : tid / kOut;
  const int o0 = kOut >= kContractThreads ? tid * kPerThread : tid % kOut;
  const int per_split = (S + splits - 1) / splits;
  const int s_begin = split * per_split;
  const int s_end = s_begin + per_split < S ? s_begin + per_split : S;
  const float* g0 = g_proj + long(n) * S * ldp;
  const float* a0 = a_proj + long(n) * S * ldp;
  float sum[kPerThread];
#pragma unroll
  for (int q = 0; q < kPerThread; ++q) sum[q] = 0.f;
  const int span = s_end > s_begin ? s_end - s_begin : 0;
  const int per_group = (span + kGroups - 1) / kGroups;
  for (int base = 0; base < per_group; base += kContractChunk) {
    for (int e = tid; e < kGroups * kContractChunk * P; e += kContractThreads) {
      const int gq = e / (kContractChunk * P);
      const int r = (e / P) % kContractChunk;
      const int c = e % P;
      const int s_local = base + r;
      const int s = s_begin + gq * per_group + s_local;
      const bool ok = s_local < per_group && s < s_end;
      gs[gq][r][c] = ok ? g0[long(s) * ldp + c] : 0.f;
      as[gq][r][c] = ok ? a0[long(s) * ldp + c] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int q = 0; q < kPerThread; ++q) {
      if (grp >= kGroups) break;  // threads beyond kGroups * kOut only help with the loads
      const int o = o0 + q;
      const int i = o / P, j = o % P;
      float acc_q = sum[q];
#pragma unroll 8
      for (int r = 0; r < kContractChunk; ++r) acc_q = fmaf(gs[grp][r][i], as[grp][r][j], acc_q);
      sum[q] = acc_q;
    }
    __syncthreads();
  }
  // this CTA's partial, groups added in fixed order
  float* part = partials + (long(n) * splits + split) * kOut;
  if constexpr (kOut >= kContractThreads) {
#pragma unroll
    for (int q = 0; q < kPerThread; ++q) part[o0 + q] = sum[q];
  } else {
    if (grp < kGroups) red[grp][o0] = sum[0];
    __syncthreads();
    if (tid < kOut) {
      float t = 0.f;
#pragma unroll
      for (int gq = 0; gq < kGroups; ++gq) t += red[gq][tid];
      part[tid] = t;
    }
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int ticket = atomicAdd(&counters[n], 1);
    is_last = ticket == splits - 1;
    if (is_last) counters[n] = 0;  // ready for the next launch
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  float* dst = acc + long(n) * ld + col_off;
  const float* all = partials + long(n) * splits * kOut;
  for (int o = tid; o < kOut; o += kContractThreads) {
    float t = 0.f;
    for (int k = 0; k < splits; ++k) t += __ldcg(all + long(k) * kOut + o);  // slice order
    dst[o] = t;
  }
}

// Per-token rows: out[r, col_off + i * p + j] = G'[t, i] * A'[t, j] for the r-th collected token
// t = token_index[r] (flat position in the [N * S] batch).
__global__ void proj_token_rows_kernel(const float* __restrict__ g_proj, const float* __restrict__ a_proj,
                                       const long* __restrict__ token_index, float* __restrict__ out, int p, int ldp,
                                       long ld, long col_off) {
  const long r = blockIdx.x;
  const long t = token_index[r];
  const float* g = g_proj + t * ldp;
  const float* a = a_proj + t * ldp;
  float* dst = out + r * ld + col_off;
  for (int o = threadIdx.x; o < p * p; o += blockDim.x) dst[o] = g[o / p] * a[o % p];
}

}  // namespace bgn

extern "C" int bgn_proj_contract_splits(int S) {
  int splits = (S + 255) / 256;
  return splits < 1 ? 1 : (splits > 16 ? 16 : splits);
}

extern "C" int bgn_proj_contract(const float* g_proj, const float* a_proj, float* acc, float* partials, int* counters,
                                 int N, int S, int p, int ldp, long ld, long col_off, cudaStream_t stream) {
  if (N <= 0 || S <= 0 || ldp < p || !partials || !counters) return int(cudaErrorInvalidValue);
  const dim3 grid(N, bgn_proj_contract_splits(S));
  switch (p) {
    case 8: proj_contract_kernel<8><<<grid, kContractThreads, 0, stream>>>(g_proj, a_proj, acc, partials, counters, S, ldp, ld, col_off); break;
    case 16: proj_contract_kernel<16><<<grid, kContractThreads, 0, stream>>>(g_proj, a_proj, acc, partials, counters, S, ldp, ld, col_off); break;
    case 32: proj_contract_kernel<32><<<grid, kContractThreads, 0, stream>>>(g_proj, a_proj, acc, partials, counters, S, ldp, ld, col_off); break;
    case 64: proj_contract_kernel<64><<<grid, kContractThreads, 0, stream>>>(g_proj, a_proj, acc, partials, counters, S, ldp, ld, col_off); break;
    default: return int(cudaErrorInvalidValue);
  }
  return int(cudaGetLastError());
}

extern "C" int bgn_proj_token_rows(const float* g_proj, const float* a_proj, const long* token_index, float* out,
                                   long rows, int p, int ldp, long ld, long col_off, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (p <= 0 || ldp < p) return int(cudaErrorInvalidValue);
  proj_token_rows_kernel<<<unsigned(rows), 256, 0, stream>>>(g_proj, a_proj, token_index, out, p, ldp, ld, col_off);
  return int(cudaGetLastError());
}
