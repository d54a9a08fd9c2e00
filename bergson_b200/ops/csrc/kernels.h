// C launch interface of the sm_100a kernels.  Every launcher enqueues on `stream`, never
// synchronises, and returns a cudaError_t (as int).  `fmt` selects the 16-bit input type:
// 0 = fp16, 1 = bf16; element type codes for the elementwise kernels: 0 = fp16, 1 = bf16,
// 2 = fp32.  `status` points at a device int that kernels set to a non-zero KernelStatus
// when one of their bounded waits runs out.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

extern "C" {

// ---- attribution (tcgen05 + TMA) ------------------------------------------------------

// out[T, 16] (fp32) = a[T, K] * p[16, K]^T.          (K multiple of 8, a/p 16-byte aligned)
int bgn_proj_right(const void* a, const void* p, float* out, long T, int K, int fmt, int* status,
                   cudaStream_t stream);

// acc[n, col_off + i*16 + j] += sum_s (g[n, s, :] . p[i, :]) * a_proj[n*S + s, j]
// g: [N, S, K] 16-bit, p: [16, K], a_proj: [N*S, 16] fp32, acc: [N, ld] fp32 (pre-zeroed by
// the caller at the start of a batch; this kernel only adds).
int bgn_proj_left_outer(const void* g, const void* p, const float* a_proj, float* acc, int N, int S,
                        int K, long ld, long col_off, int fmt, int* status, cudaStream_t stream);

// c[M, N] (fp32, row stride ldc) = a[M, K] * b[N, K]^T; optional row_sumsq[M] += sum_k a^2 is
// not computed here (see bgn_row_sumsq).
int bgn_tn_gemm(const void* a, const void* b, float* c, long M, int N, int K, long ldc, int fmt,
                int* status, cudaStream_t stream);

// c[M, world * N] (fp32) = a[M, K] * concat_r(b[r])^T with b[r] [N, K] in rank r's (possibly
// peer-mapped) memory: all-gather of B fused into the GEMM's operand loads.
int bgn_tn_gemm_gathered(const void* a, const void* const* b, int world, float* c, long M, int N, int K,
                         long ldc, int fmt, int* status, cudaStream_t stream);

// acc[n, col_off + i*p + j] = sum_s g_proj[n*S + s, i] * a_proj[n*S + s, j]  (overwrites; fixed
// summation order: bitwise repeatable).  g_proj / a_proj: fp32 [N*S, ldp] with p <= ldp
// meaningful columns; p in {8, 16, 32, 64}.  Scratch: `partials` holds
// N * bgn_proj_contract_splits(S) * p * p floats (any contents), `counters` N ints that are zero
// on entry and are left zero.
int bgn_proj_contract_splits(int S);
int bgn_proj_contract(const float* g_proj, const float* a_proj, float* acc, float* partials, int* counters,
                      int N, int S, int p, int ldp, long ld, long col_off, cudaStream_t stream);

// out[r, col_off + i*p + j] = g_proj[t, i] * a_proj[t, j] with t = token_index[r], r < rows.
int bgn_proj_token_rows(const float* g_proj, const float* a_proj, const long* token_index, float* out,
                        long rows, int p, int ldp, long ld, long col_off, cudaStream_t stream);

// acc fp32 [N, D] -> out rows (type code `out_type`) with clamp to [lo, hi]; if unit_norm,
// every row is divided by max(||row||, eps) computed on the rounded values.  Row r goes to
// out + row_index[r] * out_ld (row_index == nullptr means r).
int bgn_finalize_rows(const float* acc, void* out, const long* row_index, int N, long D, long out_ld,
                      float lo, float hi, int unit_norm, int out_type, cudaStream_t stream);

// ---- model-side elementwise -----------------------------------------------------------

int bgn_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long rows, int d, float eps,
                    int type, cudaStream_t stream);
int bgn_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                    float* dw_partial, int n_partial, long rows, int d, int type,
                    cudaStream_t stream);
int bgn_layernorm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd,
                      long rows, int d, float eps, int type, cudaStream_t stream);
int bgn_layernorm_bwd(const void* dy, const void* x, const void* w, const float* mean,
                      const float* rstd, void* dx, float* dw_partial, float* db_partial,
                      int n_partial, long rows, int d, int type, cudaStream_t stream);
// Backward of bgn_rmsnorm_bwd: cotangents U (of dx, [rows, d]) and Vw (of dw, [d] fp32) -> d_dy, d_x and
// per-block partial sums of d_w ([n_partial, d] fp32, n_partial = number of blocks launched).
int bgn_rmsnorm_bwd_bwd(const void* U, const float* Vw, const void* dy, const void* x, const void* w,
                        const float* rstd, void* d_dy, void* d_x, float* dw_partial, int n_partial, long rows, int d,
                        int type, cudaStream_t stream);
// Backward of bgn_swiglu_bwd: cotangents cg, cu (of dgate, dup) -> d_dy, d_gate, d_up.
int bgn_swiglu_bwd_bwd(const void* cg, const void* cu, const void* dy, const void* gate, const void* up, void* d_dy,
                       void* d_gate, void* d_up, long n, int type, cudaStream_t stream);
// Backward of bgn_layernorm_bwd: cotangents U (of dx, [rows, d], element type), Vw and Sb (of dw and
// db, [d] fp32) -> d_dy, d_x ([rows, d]) and per-block partial sums of d_w ([n_partial, d] fp32,
// n_partial = number of blocks launched; d at most 4 packets per thread).
int bgn_layernorm_bwd_bwd(const void* U, const float* Vw, const float* Sb, const void* dy, const void* x,
                          const void* w, const float* mean, const float* rstd, void* d_dy, void* d_x,
                          float* dw_partial, int n_partial, long rows, int d, int type, cudaStream_t stream);
// x: [B, S, H, D]; cos/sin: [S, rot/2] fp32; rotate-half on the first `rot` features.
int bgn_rotary(const void* x, const float* cos, const float* sin, void* y, long B, int S, int H,
               int D, int rot, int inverse, int type, cudaStream_t stream);
int bgn_swiglu_fwd(const void* gate, const void* up, void* y, long n, int type, cudaStream_t stream);
int bgn_swiglu_bwd(const void* dy, const void* gate, const void* up, void* dgate, void* dup, long n,
                   int type, cudaStream_t stream);
int bgn_gelu_fwd(const void* x, void* y, long n, int tanh_approx, int type, cudaStream_t stream);
int bgn_gelu_bwd(const void* dy, const void* x, void* dx, long n, int tanh_approx, int type,
                 cudaStream_t stream);
// Backward of the softmax backward (dx = y * (dy - sum(dy y)) per row of length n): given the
// cotangent c of dx, d_dy = y * (c - sum(c y)) and d_y = c * (dy - sum(dy y)) - dy * sum(c y).
int bgn_softmax_bwd_bwd(const void* c, const void* dy, const void* y, void* d_dy, void* d_y, long rows, int n,
                        int type, cudaStream_t stream);
// Backward of gelu_bwd (dx = dy * gelu'(x)): given the cotangent c of dx, d_dy = c * gelu'(x) and
// d_x = c * dy * gelu''(x).  n must be a multiple of the 16-byte packet.
int bgn_gelu_bwd_bwd(const void* c, const void* dy, const void* x, void* d_dy, void* d_x, long n, int tanh_approx,
                     int type, cudaStream_t stream);
// logits [T, V]; loss[T], lse[T] fp32; targets int64 (ignore_index -> loss 0).
int bgn_ce_fwd(const void* logits, const long* targets, float* loss, float* lse, long T, int V,
               long ignore_index, int type, cudaStream_t stream);
int bgn_ce_bwd(const void* logits, const long* targets, const float* lse, const float* dloss,
               void* dlogits, long T, int V, long ignore_index, int type, cudaStream_t stream);
// Backward of bgn_ce_bwd: cotangent C [T, V] of dlogits -> d_logits [T, V] and d_dloss [T] (fp32).
int bgn_ce_bwd_bwd(const void* C, const void* logits, const long* targets, const float* lse, const float* dloss,
                   void* d_logits, float* d_dloss, long T, int V, long ignore_index, int type, cudaStream_t stream);
// Fused AdamW on flat fp32 master state; writes the 16-bit/32-bit model copy as well.
int bgn_adamw_step(float* p, float* m, float* v, const void* g, void* p_model, long n, float lr,
                   float b1, float b2, float eps, float eps_root, float wd, float bc1, float bc2,
                   float grad_scale, int g_type, int model_type, cudaStream_t stream);
// AdamW over a list of tensors in one launch.  `table` is a device array of n_tensors entries of
// six 8-byte words {p, m, v, g, n, unused}: p and g of element type `type`, m and v fp32, all
// updated in place; max_n is the largest n.  `coef` (device scalar, may be null) multiplies
// every gradient together with gscale.
int bgn_adamw_multi(const void* table, int n_tensors, long max_n, float lr, float b1, float b2, float eps,
                    float eps_root, float wd, float bc1, float bc2, float gscale, const float* coef,
                    int type, cudaStream_t stream);
// Out-of-place AdamW over a list of tensors (backward == 0) and the vector-Jacobian product of
// that step (backward == 1).  `table`: n_tensors entries of twelve 8-byte words,
//   forward : {p, g, m, v, p_out, m_out, v_out, 0, 0, 0, n, 0}
//   backward: {g, m, v, cp, cm, cv, dp, dg, dm, dv, n, 0}
// with m, v the moments before the step, cp/cm/cv the cotangents of the step's outputs (null =
// zero) and dp/dg/dm/dv the cotangents of its inputs.  p, g and their cotangents have element
// type `type`; moments are fp32.
int bgn_adamw_traced(const void* table, int n_tensors, long max_n, int backward, float lr, float b1, float b2,
                     float eps, float eps_root, float wd, float bc1, float bc2, int type, cudaStream_t stream);
// Sum of squares over a list of tensors (table entries as above, only g and n are read) into
// out[0] (added to it when `accumulate`); with max_norm > 0, out[1] = min(1, max_norm /
// (sqrt(out[0]) + 1e-6)).  `partials` holds bgn_multi_sumsq_blocks() * n_tensors floats (an upper
// bound); max_n is the largest tensor's element count; the partials are added in a fixed order.
int bgn_multi_sumsq_blocks(void);
int bgn_multi_sumsq(const void* table, int n_tensors, long max_n, float* partials, float* out, int accumulate,
                    float max_norm, int type, cudaStream_t stream);
// out[r] += sum_k x[r, k]^2  (x 16-bit or fp32).
int bgn_row_sumsq(const void* x, float* out, long rows, long d, long ldx, int type,
                  cudaStream_t stream);

}  // extern "C"
