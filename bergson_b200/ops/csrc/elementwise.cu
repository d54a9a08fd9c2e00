// Bandwidth-bound model-side kernels: RMSNorm / LayerNorm (fwd, bwd), rotary embedding,
// SwiGLU / GELU (fwd, bwd), per-token cross entropy (fwd, bwd), fused AdamW, row sum of
// squares.  16-bit inputs are read with 16-byte vector loads, statistics are kept in fp32.
#include "common.cuh"
#include "kernels.h"

namespace bgn {

template <typename T>
struct Vec {  // 16-byte packet
  static constexpr int N = 16 / sizeof(T);
  T v[N];
};

template <typename T>
__device__ __forceinline__ Vec<T> load_vec(const T* p) {
  Vec<T> r;
  *reinterpret_cast<uint4*>(r.v) = *reinterpret_cast<const uint4*>(p);
  return r;
}
template <typename T>
__device__ __forceinline__ void store_vec(T* p, const Vec<T>& r) {
  *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(r.v);
}

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = l < (blockDim.x >> 5) ? red[l] : 0.f;
  t = warp_sum(t);
  return t;
}

// Sums N values over the block with one pass through shared memory (`red` holds 33 * N floats);
// every thread gets all N totals.
template <int N>
__device__ __forceinline__ void block_sum_n(float (&v)[N], float* red) {
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
#pragma unroll
  for (int j = 0; j < N; ++j) v[j] = warp_sum(v[j]);
  __syncthreads();  // `red` may still be read from an earlier call
  if (l == 0) {
#pragma unroll
    for (int j = 0; j < N; ++j) red[w * N + j] = v[j];
  }
  __syncthreads();
  if (w == 0) {
#pragma unroll
    for (int j = 0; j < N; ++j) {
      float t = l < nw ? red[l * N + j] : 0.f;
      t = warp_sum(t);
      if (l == 0) red[32 * N + j] = t;
    }
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < N; ++j) v[j] = red[32 * N + j];
}

__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = l < (blockDim.x >> 5) ? red[l] : -INFINITY;
  t = warp_max(t);
  return t;
}

// ---- RMSNorm --------------------------------------------------------------------------
// y = T(T(x * rstd) * w): the normalised value is rounded to the activation dtype before the
// weight multiply, as the eager implementation of the model families does.

template <typename T>
__global__ void rmsnorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y,
                                   float* __restrict__ rstd_out, int d, float eps) {
  __shared__ float red[32];
  const long r = blockIdx.x;
  const T* xr = x + r * d;
  T* yr = y + r * d;
  constexpr int V = Vec<T>::N;
  float ss = 0.f;
  for (int i = threadIdx.x * V; i < d; i += blockDim.x * V) {
    Vec<T> xv = load_vec(xr + i);
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const float f = to_float<T>(xv.v[k]);
      ss = fmaf(f, f, ss);
    }
  }
  ss = block_sum(ss, red);
  const float rstd = rsqrtf(ss / d + eps);
  if (threadIdx.x == 0) rstd_out[r] = rstd;
  for (int i = threadIdx.x * V; i < d; i += blockDim.x * V) {
    Vec<T> xv = load_vec(xr + i), wv = load_vec(w + i), o;
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const float n = to_float<T>(from_float<T>(to_float<T>(xv.v[k]) * rstd));
      o.v[k] = from_float<T>(n * to_float<T>(wv.v[k]));
    }
    store_vec(yr + i, o);
  }
}

// dx = rstd * (dy*w - xhat * mean(dy*w*xhat));  dw partials: block b accumulates rows
// b, b+gridDim, ... into dw_partial[b, :] (summed by the caller).
template <typename T>
__global__ void rmsnorm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                   const T* __restrict__ w, const float* __restrict__ rstd,
                                   T* __restrict__ dx, float* __restrict__ dw_partial, long rows,
                                   int d) {
  __shared__ float red[32];
  constexpr int V = Vec<T>::N;
  constexpr int kMaxPer = 4;  // supports d <= blockDim * V * 4
  float dw_acc[kMaxPer][V];
#pragma unroll
  for (int a = 0; a < kMaxPer; ++a)
#pragma unroll
    for (int k = 0; k < V; ++k) dw_acc[a][k] = 0.f;

  for (long r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* xr = x + r * d;
    const T* gr = dy + r * d;
    T* dr = dx + r * d;
    const float rs = rstd[r];
    float dot = 0.f;
    for (int i = threadIdx.x * V; i < d; i += blockDim.x * V) {
      Vec<T> xv = load_vec(xr + i), gv = load_vec(gr + i), wv = load_vec(w + i);
#pragma unroll
      for (int k = 0; k < V; ++k)
        dot = fmaf(to_float<T>(gv.v[k]) * to_float<T>(wv.v[k]), to_float<T>(xv.v[k]) * rs, dot);
    }
    dot = block_sum(dot, red) / d;
    int a = 0;
    for (int i = threadIdx.x * V; i < d; i += blockDim.x * V, ++a) {
      Vec<T> xv = load_vec(xr + i), gv = load_vec(gr + i), wv = load_vec(w + i), o;
#pragma unroll
      for (int k = 0; k < V; ++k) {
        const float xh = to_float<T>(xv.v[k]) * rs;
        const float g = to_float<T>(gv.v[k]);
        o.v[k] = from_float<T>(rs * (g * to_float<T>(wv.v[k]) - xh * dot));
        if (dw_partial && a < kMaxPer) dw_acc[a][k] = fmaf(g, xh, dw_acc[a][k]);
      }
      store_vec(dr + i, o);
    }
  }
  if (dw_partial) {
    int a = 0;
    for (int i = threadIdx.x * V; i < d && a < kMaxPer; i += blockDim.x * V, ++a)
#pragma unroll
      for (int k = 0; k < V; ++k) dw_partial[long(blockIdx.x) * d + i + k] = dw_acc[a][k];
  }
}

// Backward of rmsnorm_bwd.  With g = dy * w, xh = x * rstd, the first backward is
//   dx = rstd * (g - xh * mean(g xh)),   dw = sum_rows dy xh.
// Given cotangents U (of dx) and Vw (of dw, [d] fp32):
//   d_dy = w * rstd * P(U) + Vw * xh,   d_w = sum_rows dy * rstd * P(U),
//   d_x  = -rstd^2 * (xh * (mean(g U) - mean(g xh) mean(U xh)) + mean(U xh) * P(g) + mean(g xh) * P(U))
//          + rstd * P(Vw * dy),         with P(z) = z - xh * mean(z xh).
template <typename T>
__global__ void rmsnorm_bwd_bwd_kernel(const T* __restrict__ U, const float* __restrict__ Vw,
                                       const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ w,
                                       const float* __restrict__ rstd, T* __restrict__ d_dy, T* __restrict__ d_x,
                                       float* __restrict__ dw_partial, long rows, int d) {
  __shared__ float red[33 * 4];
  constexpr int V = Vec<T>::N;
  constexpr int kMaxPer = 4;
  float dw_acc[kMaxPer][V];
#pragma unroll
  for (int a = 0; a < kMaxPer; ++a)
#pragma unroll
    for (int k = 0; k < V; ++k) dw_acc[a][k] = 0.f;
  for (long r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* xr = x + r * d;
    const T* gr = dy + r * d;
    const T* ur = U + r * d;
    const float rs = rstd[r];
    float sgx = 0.f, sux = 0.f, sgu = 0.f, sqx = 0.f;
    for (int i = threadIdx.x * V; i < d; i += blockDim.x * V) {
      Vec<T> xv = load_vec(xr + i), gv = load_vec(gr + i), uv = load_vec(ur + i), wv = load_vec(w + i);
#pragma unroll
      for (int k = 0; k < V; ++k) {
        const float xh = to_float<T>(xv.v[k]) * rs;
        const float gy = to_float<T>(gv.v[k]);
        const float g = gy * to_float<T>(wv.v[k]);
        const float u = to_float<T>(uv.v[k]);
        sgx = fmaf(g, xh, sgx);
        sux = fmaf(u, xh, sux);
        sgu = fmaf(g, u, sgu);
        sqx = fmaf(Vw[i + k] * gy, xh, sqx);
      }
    }
    const float inv_d = 1.f / d;
    float sums[4] = {sgx, sux, sgu, sqx};
    block_sum_n<4>(sums, red);
    const float b = sums[0] * inv_d, c = sums[1] * inv_d, mgu = sums[2] * inv_d, mqx = sums[3] * inv_d;
    const float e = mgu - b * c;
    int slot = 0;
    for (int i = threadIdx.x * V; i < d; i += blockDim.x * V, ++slot) {
      Vec<T> xv = load_vec(xr + i), gv = load_vec(gr + i), uv = load_vec(ur + i), wv = load_vec(w + i), o1, o2;
#pragma unroll
      for (int k = 0; k < V; ++k) {
        const float xh = to_float<T>(xv.v[k]) * rs;
        const float gy = to_float<T>(gv.v[k]);
        const float wk = to_float<T>(wv.v[k]);
        const float g = gy * wk;
        const float vw = Vw[i + k];
        const float pu = to_float<T>(uv.v[k]) - xh * c;
        const float pg = g - xh * b;
        o1.v[k] = from_float<T>(wk * rs * pu + vw * xh);
        o2.v[k] = from_float<T>(-rs * rs * (xh * e + c * pg + b * pu) + rs * (vw * gy - xh * mqx));
        if (slot < kMaxPer) dw_acc[slot][k] = fmaf(gy, rs * pu, dw_acc[slot][k]);
      }
      store_vec(d_dy + r * d + i, o1);
      store_vec(d_x + r * d + i, o2);
    }
  }
  int slot = 0;
  for (int i = threadIdx.x * V; i < d && slot < kMaxPer; i += blockDim.x * V, ++slot)
#pragma unroll
    for (int k = 0; k < V; ++k) dw_partial[long(blockIdx.x) * d + i + k] = dw_acc[slot][k];
}

// ---- LayerNorm ------------------------------------------------------------------------

template <typename T>
__global__ void layernorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                     const T* __restrict__ b, T* __restrict__ y,
                                     float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                     int d, float eps) {
  __shared__ float red[32];
  const long r = blockIdx.x;
  const T* xr = x + r * d;
  T* yr = y + r * d;
  constexpr int V = Vec<T>::N;
  float s = 0.f;
  for (int i = threadIdx.x * V; i < d; i += blockDim.x * V) {
    Vec<T> xv = load_vec(xr + i);
#pragma unroll
    for (int k = 0; k < V; ++k) s += to_float<T>(xv.v[k]);
  }
  const float mean = block_sum(s, red) / d;
  float ss = 0.f;
  for (int i = threadIdx.x * V; i < d; i += blockDim.x * V) {
    Vec<T> xv = load_vec(xr + i);
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const float c = to_float<T>(xv.v[k]) - mean;
      ss = fmaf(c, c, ss);
    }
  }
  const float rstd = rsqrtf(block_sum(ss, red) / d + eps);
  if (threadIdx.x == 0) {
    mean_out[r] = mean;
    rstd_out[r] = rstd;
  }
  for (int i = threadIdx.x * V; i < d; i += blockDim.x * V) {
    Vec<T> xv = load_vec(xr + i), wv = load_vec(w + i), o;
    Vec<T> bv;
    if (b) bv = load_vec(b + i);
#pragma unroll
    for (int k = 0; k < V; ++k) {
      float v = (to_float<T>(xv.v[k]) - mean) * rstd * to_float<T>(wv.v[k]);
      if (b) v += to_float<T>(bv.v[k]);
      o.v[k] = from_float<T>(v);
    }
    store_vec(yr + i, o);
  }
}

// dx = rstd * (g - mean(g) - xhat * mean(g * xhat)), g = dy * w.
template <typename T>
__global__ void layernorm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                     const T* __restrict__ w, const float* __restrict__ mean,
                                     const float* __restrict__ rstd, T* __restrict__ dx,
                                     float* __restrict__ dw_partial, float* __restrict__ db_partial,
                                     long rows, int d) {
  __shared__ float red[32];
  constexpr int V = Vec<T>::N;
  constexpr int kMaxPer = 4;
  float dw_acc[kMaxPer][V], db_acc[kMaxPer][V];
#pragma unroll
  for (int a = 0; a < kMaxPer; ++a)
#pragma unroll
    for (int k = 0; k < V; ++k) dw_acc[a][k] = db_acc[a][k] = 0.f;

  for (long r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* xr = x + r * d;
    const T* gr = dy + r * d;
    T* dr = dx + r * d;
    const float mu = mean[r], rs = rstd[r];
    float s1 = 0.f, s2 = 0.f;
    for (int i = threadIdx.x * V; i < d; i += blockDim.x * V) {
      Vec<T> xv = load_vec(xr + i), gv = load_vec(gr + i), wv = load_vec(w + i);
#pragma unroll
      for (int k = 0; k < V; ++k) {
        const float g = to_float<T>(gv.v[k]) * to_float<T>(wv.v[k]);
        s1 += g;
        s2 = fmaf(g, (to_float<T>(xv.v[k]) - mu) * rs, s2);
      }
    }
    s1 = block_sum(s1, red) / d;
    s2 = block_sum(s2, red) / d;
    int a = 0;
    for (int i = threadIdx.x * V; i < d; i += blockDim.x * V, ++a) {
      Vec<T> xv = load_vec(xr + i), gv = load_vec(gr + i), wv = load_vec(w + i), o;
#pragma unroll
      for (int k = 0; k < V; ++k) {
        const float xh = (to_float<T>(xv.v[k]) - mu) * rs;
        const float gy = to_float<T>(gv.v[k]);
        const float g = gy * to_float<T>(wv.v[k]);
        o.v[k] = from_float<T>(rs * (g - s1 - xh * s2));
        if (dw_partial && a < kMaxPer) {
          dw_acc[a][k] = fmaf(gy, xh, dw_acc[a][k]);
          db_acc[a][k] += gy;
        }
      }
      store_vec(dr + i, o);
    }
  }
  if (dw_partial) {
    int a = 0;
    for (int i = threadIdx.x * V; i < d && a < kMaxPer; i += blockDim.x * V, ++a)
#pragma unroll
      for (int k = 0; k < V; ++k) {
        dw_partial[long(blockIdx.x) * d + i + k] = dw_acc[a][k];
        db_partial[long(blockIdx.x) * d + i + k] = db_acc[a][k];
      }
  }
}

// Backward of layernorm_bwd.  With g = dy * w, xh = (x - mean) * rstd, the first backward is
//   dx = rstd * (g - mean(g) - xh * mean(g xh)),  dw = sum_rows dy xh,  db = sum_rows dy.
// Given cotangents U (of dx, [rows, d]), Vw (of dw, [d]) and Sb (of db, [d]) this kernel returns
//   d_dy = w * rstd * P(U) + Vw * xh + Sb
//   d_x  = -rstd^2 * (xh * (mean(g U) - mean(g) mean(U) - mean(g xh) mean(U xh)) + mean(U xh) * P'(g) + mean(g xh) * P'(U))
//          + rstd * P(Vw * dy)
//   d_w  = sum_rows dy * rstd * P(U)
// where P(z) = z - mean(z) - xh * mean(z xh) and P'(z) = z - mean(z) - xh * mean(z xh) (the same
// projection; written twice for readability of the formula).  All means run over the row.
template <typename T>
__global__ void layernorm_bwd_bwd_kernel(const T* __restrict__ U, const float* __restrict__ Vw,
                                         const float* __restrict__ Sb, const T* __restrict__ dy,
                                         const T* __restrict__ x, const T* __restrict__ w,
                                         const float* __restrict__ mean, const float* __restrict__ rstd,
                                         T* __restrict__ d_dy, T* __restrict__ d_x, float* __restrict__ dw_partial,
                                         long rows, int d) {
  __shared__ float red[33 * 7];
  constexpr int V = Vec<T>::N;
  constexpr int kMaxPer = 4;
  float dw_acc[kMaxPer][V];
#pragma unroll
  for (int a = 0; a < kMaxPer; ++a)
#pragma unroll
    for (int k = 0; k < V; ++k) dw_acc[a][k] = 0.f;

  for (long r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* xr = x + r * d;
    const T* gr = dy + r * d;
    const T* ur = U + r * d;
    const float mu = mean[r], rs = rstd[r];
    float sg = 0.f, sgx = 0.f, su = 0.f, sux = 0.f, sgu = 0.f, sq = 0.f, sqx = 0.f;
    for (int i = threadIdx.x * V; i < d; i += blockDim.x * V) {
      Vec<T> xv = load_vec(xr + i), gv = load_vec(gr + i), uv = load_vec(ur + i), wv = load_vec(w + i);
#pragma unroll
      for (int k = 0; k < V; ++k) {
        const float xh = (to_float<T>(xv.v[k]) - mu) * rs;
        const float gy = to_float<T>(gv.v[k]);
        const float g = gy * to_float<T>(wv.v[k]);
        const float u = to_float<T>(uv.v[k]);
        const float q = Vw[i + k] * gy;
        sg += g;
        sgx = fmaf(g, xh, sgx);
        su += u;
        sux = fmaf(u, xh, sux);
        sgu = fmaf(g, u, sgu);
        sq += q;
        sqx = fmaf(q, xh, sqx);
      }
    }
    const float inv_d = 1.f / d;
    float sums[7] = {sg, sgx, su, sux, sgu, sq, sqx};
    block_sum_n<7>(sums, red);
    const float a = sums[0] * inv_d, b = sums[1] * inv_d, mU = sums[2] * inv_d, c = sums[3] * inv_d;
    const float mgu = sums[4] * inv_d, mq = sums[5] * inv_d, mqx = sums[6] * inv_d;
    const float e = mgu - a * mU - b * c;
    int slot = 0;
    for (int i = threadIdx.x * V; i < d; i += blockDim.x * V, ++slot) {
      Vec<T> xv = load_vec(xr + i), gv = load_vec(gr + i), uv = load_vec(ur + i), wv = load_vec(w + i), o1, o2;
#pragma unroll
      for (int k = 0; k < V; ++k) {
        const float xh = (to_float<T>(xv.v[k]) - mu) * rs;
        const float gy = to_float<T>(gv.v[k]);
        const float wk = to_float<T>(wv.v[k]);
        const float g = gy * wk;
        const float u = to_float<T>(uv.v[k]);
        const float vw = Vw[i + k];
        const float pu = u - mU - xh * c;
        const float pg = g - a - xh * b;
        const float pq = vw * gy - mq - xh * mqx;
        o1.v[k] = from_float<T>(wk * rs * pu + vw * xh + Sb[i + k]);
        o2.v[k] = from_float<T>(-rs * rs * (xh * e + c * pg + b * pu) + rs * pq);
        if (slot < kMaxPer) dw_acc[slot][k] = fmaf(gy, rs * pu, dw_acc[slot][k]);
      }
      store_vec(d_dy + r * d + i, o1);
      store_vec(d_x + r * d + i, o2);
    }
  }
  int slot = 0;
  for (int i = threadIdx.x * V; i < d && slot < kMaxPer; i += blockDim.x * V, ++slot)
#pragma unroll
    for (int k = 0; k < V; ++k) dw_partial[long(blockIdx.x) * d + i + k] = dw_acc[slot][k];
}

// ---- rotary ---------------------------------------------------------------------------

template <typename T>
__global__ void rotary_kernel(const T* __restrict__ x, const float* __restrict__ cosT,
                              const float* __restrict__ sinT, T* __restrict__ y, long total_pairs,
                              int S, int H, int D, int rot, float sign) {
  // One thread per (b, s, h, i) with i in [0, D/2): handles features i and i + D/2 when inside
  // the rotated prefix (pairs are (i, i + rot/2) for i < rot/2); copies the rest.
  const int half = rot >> 1;
  const long per_head = D - half;  // threads per head: rot/2 pairs + (D - rot) pass-through
  for (long idx = blockIdx.x * long(blockDim.x) + threadIdx.x; idx < total_pairs;
       idx += long(gridDim.x) * blockDim.x) {
    const long head = idx / per_head;
    const int i = int(idx - head * per_head);
    const int s = int((head / H) % S);
    const T* xp = x + head * D;
    T* yp = y + head * D;
    if (i < half) {
      const float c = cosT[long(s) * half + i], sn = sinT[long(s) * half + i] * sign;
      const float a = to_float<T>(xp[i]), b = to_float<T>(xp[i + half]);
      yp[i] = from_float<T>(a * c - b * sn);
      yp[i + half] = from_float<T>(b * c + a * sn);
    } else {
      yp[i + half] = xp[i + half];
    }
  }
}

// Vectorised form: one thread per 16-byte packet of the first half of the rotated prefix (it also
// handles the matching packet of the second half) or per pass-through packet.  Needs the packet
// width to divide rot / 2 and D - rot.
template <typename T>
__global__ void rotary_vec_kernel(const T* __restrict__ x, const float* __restrict__ cosT,
                                  const float* __restrict__ sinT, T* __restrict__ y, long total, int S, int H, int D,
                                  int rot, float sign) {
  constexpr int V = Vec<T>::N;
  const int half = rot >> 1;
  const int rot_packets = half / V, pass_packets = (D - rot) / V;
  const int per_head = rot_packets + pass_packets;
  for (long idx = blockIdx.x * long(blockDim.x) + threadIdx.x; idx < total; idx += long(gridDim.x) * blockDim.x) {
    const long head = idx / per_head;
    const int k = int(idx - head * per_head);
    const T* xp = x + head * D;
    T* yp = y + head * D;
    if (k < rot_packets) {
      const int i = k * V;
      const int s = int((head / H) % S);
      const Vec<T> a = load_vec(xp + i), b = load_vec(xp + i + half);
      const float* cp = cosT + long(s) * half + i;
      const float* sp = sinT + long(s) * half + i;
      Vec<T> oa, ob;
#pragma unroll
      for (int j = 0; j < V; ++j) {
        const float c = __ldg(cp + j), sn = __ldg(sp + j) * sign;
        const float av = to_float<T>(a.v[j]), bv = to_float<T>(b.v[j]);
        oa.v[j] = from_float<T>(av * c - bv * sn);
        ob.v[j] = from_float<T>(bv * c + av * sn);
      }
      store_vec(yp + i, oa);
      store_vec(yp + i + half, ob);
    } else {
      const int i = rot + (k - rot_packets) * V;
      store_vec(yp + i, load_vec(xp + i));
    }
  }
}

// ---- activations ----------------------------------------------------------------------

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

template <typename T>
__global__ void swiglu_fwd_kernel(const T* __restrict__ g, const T* __restrict__ u, T* __restrict__ y,
                                  long n) {
  constexpr int V = Vec<T>::N;
  for (long i = (blockIdx.x * long(blockDim.x) + threadIdx.x) * V; i < n;
       i += long(gridDim.x) * blockDim.x * V) {
    Vec<T> gv = load_vec(g + i), uv = load_vec(u + i), o;
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const float a = to_float<T>(gv.v[k]);
      // silu rounded to the activation dtype before the product, as an eager silu(g) * u is.
      const float s = to_float<T>(from_float<T>(a * sigmoidf_(a)));
      o.v[k] = from_float<T>(s * to_float<T>(uv.v[k]));
    }
    store_vec(y + i, o);
  }
}

template <typename T>
__global__ void swiglu_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ g,
                                  const T* __restrict__ u, T* __restrict__ dg, T* __restrict__ du,
                                  long n) {
  constexpr int V = Vec<T>::N;
  for (long i = (blockIdx.x * long(blockDim.x) + threadIdx.x) * V; i < n;
       i += long(gridDim.x) * blockDim.x * V) {
    Vec<T> yv = load_vec(dy + i), gv = load_vec(g + i), uv = load_vec(u + i), og, ou;
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const float a = to_float<T>(gv.v[k]), d = to_float<T>(yv.v[k]), b = to_float<T>(uv.v[k]);
      const float sg = sigmoidf_(a);
      ou.v[k] = from_float<T>(d * a * sg);
      og.v[k] = from_float<T>(d * b * sg * (1.f + a * (1.f - sg)));
    }
    store_vec(dg + i, og);
    store_vec(du + i, ou);
  }
}

// Backward of swiglu_bwd (dg = dy * u * silu'(g), du = dy * silu(g)).  Given cotangents cg (of dg)
// and cu (of du):  d_dy = cg * u * silu'(g) + cu * silu(g),
//                  d_g  = cg * dy * u * silu''(g) + cu * dy * silu'(g),   d_u = cg * dy * silu'(g).
template <typename T>
__global__ void swiglu_bwd_bwd_kernel(const T* __restrict__ cg, const T* __restrict__ cu, const T* __restrict__ dy,
                                      const T* __restrict__ g, const T* __restrict__ u, T* __restrict__ d_dy,
                                      T* __restrict__ d_g, T* __restrict__ d_u, long n) {
  constexpr int V = Vec<T>::N;
  for (long i = (blockIdx.x * long(blockDim.x) + threadIdx.x) * V; i < n;
       i += long(gridDim.x) * blockDim.x * V) {
    Vec<T> av = load_vec(cg + i), bv = load_vec(cu + i), yv = load_vec(dy + i), gv = load_vec(g + i), uv = load_vec(u + i);
    Vec<T> o1, o2, o3;
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const float a = to_float<T>(gv.v[k]), b = to_float<T>(uv.v[k]), d = to_float<T>(yv.v[k]);
      const float ca = to_float<T>(av.v[k]), cb = to_float<T>(bv.v[k]);
      const float sg = sigmoidf_(a);
      const float s1 = sg * (1.f + a * (1.f - sg));
      const float s2 = sg * (1.f - sg) * (2.f + a * (1.f - 2.f * sg));
      o1.v[k] = from_float<T>(ca * b * s1 + cb * a * sg);
      o2.v[k] = from_float<T>(ca * d * b * s2 + cb * d * s1);
      o3.v[k] = from_float<T>(ca * d * s1);
    }
    store_vec(d_dy + i, o1);
    store_vec(d_g + i, o2);
    store_vec(d_u + i, o3);
  }
}

__device__ __forceinline__ float gelu_f(float x, bool tanh_approx) {
  if (tanh_approx) {
    const float k = 0.7978845608028654f;
    return 0.5f * x * (1.f + tanhf(k * (x + 0.044715f * x * x * x)));
  }
  return 0.5f * x * (1.f + erff(x * 0.7071067811865476f));
}

__device__ __forceinline__ float gelu_grad_f(float x, bool tanh_approx) {
  if (tanh_approx) {
    const float k = 0.7978845608028654f;
    const float t = tanhf(k * (x + 0.044715f * x * x * x));
    return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * k * (1.f + 3.f * 0.044715f * x * x);
  }
  const float cdf = 0.5f * (1.f + erff(x * 0.7071067811865476f));
  return cdf + x * 0.3989422804014327f * __expf(-0.5f * x * x);
}

template <typename T>
__global__ void gelu_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, long n, int tanh_approx) {
  constexpr int V = Vec<T>::N;
  for (long i = (blockIdx.x * long(blockDim.x) + threadIdx.x) * V; i < n;
       i += long(gridDim.x) * blockDim.x * V) {
    Vec<T> xv = load_vec(x + i), o;
#pragma unroll
    for (int k = 0; k < V; ++k) o.v[k] = from_float<T>(gelu_f(to_float<T>(xv.v[k]), tanh_approx));
    store_vec(y + i, o);
  }
}

template <typename T>
__global__ void gelu_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, T* __restrict__ dx,
                                long n, int tanh_approx) {
  constexpr int V = Vec<T>::N;
  for (long i = (blockIdx.x * long(blockDim.x) + threadIdx.x) * V; i < n;
       i += long(gridDim.x) * blockDim.x * V) {
    Vec<T> xv = load_vec(x + i), gv = load_vec(dy + i), o;
#pragma unroll
    for (int k = 0; k < V; ++k)
      o.v[k] = from_float<T>(to_float<T>(gv.v[k]) * gelu_grad_f(to_float<T>(xv.v[k]), tanh_approx));
    store_vec(dx + i, o);
  }
}

// Second derivative of GELU (for the backward of the backward).
__device__ __forceinline__ float gelu_grad2_f(float x, bool tanh_approx) {
  if (tanh_approx) {
    const float k = 0.7978845608028654f, c = 0.044715f;
    const float t = tanhf(k * (x + c * x * x * x));
    const float s = 1.f - t * t;
    const float u1 = k * (1.f + 3.f * c * x * x);  // u'
    const float u2 = k * 6.f * c * x;               // u''
    return s * (u1 + x * (0.5f * u2 - t * u1 * u1));
  }
  return 0.3989422804014327f * __expf(-0.5f * x * x) * (2.f - x * x);
}

// Backward of gelu_bwd: dx = dy * gelu'(x).  Given the cotangent c of dx:
//   d_dy = c * gelu'(x),   d_x = c * dy * gelu''(x).
template <typename T>
__global__ void gelu_bwd_bwd_kernel(const T* __restrict__ c, const T* __restrict__ dy, const T* __restrict__ x,
                                    T* __restrict__ d_dy, T* __restrict__ d_x, long n, int tanh_approx) {
  constexpr int V = Vec<T>::N;
  for (long i = (blockIdx.x * long(blockDim.x) + threadIdx.x) * V; i < n;
       i += long(gridDim.x) * blockDim.x * V) {
    Vec<T> cv = load_vec(c + i), gv = load_vec(dy + i), xv = load_vec(x + i), o1, o2;
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const float xf = to_float<T>(xv.v[k]), cf = to_float<T>(cv.v[k]);
      o1.v[k] = from_float<T>(cf * gelu_grad_f(xf, tanh_approx));
      o2.v[k] = from_float<T>(cf * to_float<T>(gv.v[k]) * gelu_grad2_f(xf, tanh_approx));
    }
    store_vec(d_dy + i, o1);
    store_vec(d_x + i, o2);
  }
}

// ---- softmax: backward of the backward ---------------------------------------------------
// The softmax backward is dx = y * (dy - sum(dy y)) per row.  Given the cotangent c of dx:
//   d_dy = y * (c - sum(c y)),   d_y = c * (dy - sum(dy y)) - dy * sum(c y).
// One warp per row (rows are attention rows: a few hundred to a few thousand elements).
template <typename T>
__global__ void softmax_bwd_bwd_kernel(const T* __restrict__ c, const T* __restrict__ dy, const T* __restrict__ y,
                                       T* __restrict__ d_dy, T* __restrict__ d_y, long rows, int n) {
  constexpr int V = Vec<T>::N;
  const int lane = threadIdx.x & 31;
  const long warp = (blockIdx.x * long(blockDim.x) + threadIdx.x) >> 5;
  const long n_warps = (long(gridDim.x) * blockDim.x) >> 5;
  for (long r = warp; r < rows; r += n_warps) {
    const T* cr = c + r * n;
    const T* gr = dy + r * n;
    const T* yr = y + r * n;
    float s = 0.f, t = 0.f;
    for (int i = lane * V; i < n; i += 32 * V) {
      const Vec<T> cv = load_vec(cr + i), gv = load_vec(gr + i), yv = load_vec(yr + i);
#pragma unroll
      for (int k = 0; k < V; ++k) {
        const float yf = to_float<T>(yv.v[k]);
        s = fmaf(to_float<T>(gv.v[k]), yf, s);
        t = fmaf(to_float<T>(cv.v[k]), yf, t);
      }
    }
    s = warp_sum(s);
    t = warp_sum(t);
    for (int i = lane * V; i < n; i += 32 * V) {
      const Vec<T> cv = load_vec(cr + i), gv = load_vec(gr + i), yv = load_vec(yr + i);
      Vec<T> o1, o2;
#pragma unroll
      for (int k = 0; k < V; ++k) {
        const float cf = to_float<T>(cv.v[k]), gf = to_float<T>(gv.v[k]), yf = to_float<T>(yv.v[k]);
        o1.v[k] = from_float<T>(yf * (cf - t));
        o2.v[k] = from_float<T>(cf * (gf - s) - gf * t);
      }
      store_vec(d_dy + r * n + i, o1);
      store_vec(d_y + r * n + i, o2);
    }
  }
}

// ---- cross entropy --------------------------------------------------------------------

template <typename T>
__global__ void ce_fwd_kernel(const T* __restrict__ logits, const long* __restrict__ targets,
                              float* __restrict__ loss, float* __restrict__ lse_out, int V_,
                              long ignore_index) {
  __shared__ float red[32];
  const long r = blockIdx.x;
  const T* z = logits + r * V_;
  constexpr int V = Vec<T>::N;
  const bool vec_ok = (V_ % V) == 0;
  float m = -INFINITY, s = 0.f;  // online softmax statistics
  auto push = [&](float f) {
    if (f > m) {
      s = s * __expf(m - f) + 1.f;
      m = f;
    } else {
      s += __expf(f - m);
    }
  };
  if (vec_ok) {
    for (int i = threadIdx.x * V; i < V_; i += blockDim.x * V) {
      Vec<T> zv = load_vec(z + i);
#pragma unroll
      for (int k = 0; k < V; ++k) push(to_float<T>(zv.v[k]));
    }
  } else {
    for (int i = threadIdx.x; i < V_; i += blockDim.x) push(to_float<T>(z[i]));
  }
  const float gm = block_max(m, red);
  const float contrib = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  const float gs = block_sum(contrib, red);
  if (threadIdx.x == 0) {
    const float lse = gm + logf(gs);
    lse_out[r] = lse;
    const long t = targets[r];
    loss[r] = (t == ignore_index) ? 0.f : lse - to_float<T>(z[t]);
  }
}

template <typename T>
__global__ void ce_bwd_kernel(const T* __restrict__ logits, const long* __restrict__ targets,
                              const float* __restrict__ lse, const float* __restrict__ dloss,
                              T* __restrict__ dlogits, int V_, long ignore_index) {
  const long r = blockIdx.x;
  const T* z = logits + r * V_;
  T* dz = dlogits + r * V_;
  const long t = targets[r];
  const float g = (t == ignore_index) ? 0.f : dloss[r];
  const float l = lse[r];
  constexpr int V = Vec<T>::N;
  if ((V_ % V) == 0) {
    for (int i = threadIdx.x * V; i < V_; i += blockDim.x * V) {
      Vec<T> zv = load_vec(z + i), o;
#pragma unroll
      for (int k = 0; k < V; ++k) {
        float p = __expf(to_float<T>(zv.v[k]) - l);
        if (i + k == t) p -= 1.f;
        o.v[k] = from_float<T>(p * g);
      }
      store_vec(dz + i, o);
    }
  } else {
    for (int i = threadIdx.x; i < V_; i += blockDim.x) {
      float p = __expf(to_float<T>(z[i]) - l);
      if (i == t) p -= 1.f;
      dz[i] = from_float<T>(p * g);
    }
  }
}

// ---- AdamW ----------------------------------------------------------------------------

template <typename G, typename M>
__global__ void adamw_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                             const G* __restrict__ g, M* __restrict__ pm, long n, float lr, float b1,
                             float b2, float eps, float eps_root, float wd, float bc1, float bc2,
                             float gscale) {
  for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < n;
       i += long(gridDim.x) * blockDim.x) {
    const float gi = to_float<G>(g[i]) * gscale;
    const float mi = b1 * m[i] + (1.f - b1) * gi;
    const float vi = b2 * v[i] + (1.f - b2) * gi * gi;
    m[i] = mi;
    v[i] = vi;
    const float upd = (mi / bc1) / (sqrtf(vi / bc2 + eps_root) + eps) + wd * p[i];
    const float pi = p[i] - lr * upd;
    p[i] = pi;
    if (pm) pm[i] = from_float<M>(pi);
  }
}

// One launch for a whole list of tensors: blockIdx.y selects the table entry, the blocks of
// that row stride over its elements (four at a time when size and addresses allow).
// p and g share the element type T; m and v are fp32.  `coef` (optional, device scalar)
// scales every gradient, e.g. a global-norm clipping coefficient computed on the device.
struct AdamEntry {
  void* p;
  float* m;
  float* v;
  const void* g;
  long n;
  long reserved;
};

template <typename T>
__device__ __forceinline__ void adamw_one(T& p, float& m, float& v, T g, float gs, float lr, float b1, float b2,
                                          float eps, float eps_root, float wd, float bc1, float bc2) {
  const float gi = to_float<T>(g) * gs;
  m = b1 * m + (1.f - b1) * gi;
  v = b2 * v + (1.f - b2) * gi * gi;
  const float pf = to_float<T>(p);
  const float upd = (m / bc1) / (sqrtf(v / bc2 + eps_root) + eps) + wd * pf;
  p = from_float<T>(pf - lr * upd);
}

template <typename T>
__global__ void adamw_multi_kernel(const AdamEntry* __restrict__ table, float lr, float b1, float b2, float eps,
                                   float eps_root, float wd, float bc1, float bc2, float gscale,
                                   const float* __restrict__ coef) {
  const AdamEntry e = table[blockIdx.y];
  const float gs = coef ? gscale * coef[0] : gscale;
  T* p = static_cast<T*>(e.p);
  const T* g = static_cast<const T*>(e.g);
  struct alignas(4 * sizeof(T)) Pack { T v[4]; };
  const bool vec = (e.n & 3) == 0 &&
                   ((reinterpret_cast<uintptr_t>(e.m) | reinterpret_cast<uintptr_t>(e.v)) & 15) == 0 &&
                   ((reinterpret_cast<uintptr_t>(e.p) | reinterpret_cast<uintptr_t>(e.g)) & (4 * sizeof(T) - 1)) == 0;
  const long tid = blockIdx.x * long(blockDim.x) + threadIdx.x, stride = long(gridDim.x) * blockDim.x;
  if (vec) {
    for (long i = tid; i < (e.n >> 2); i += stride) {
      float4 m4 = reinterpret_cast<float4*>(e.m)[i], v4 = reinterpret_cast<float4*>(e.v)[i];
      Pack pp = reinterpret_cast<Pack*>(p)[i];
      const Pack gp = reinterpret_cast<const Pack*>(g)[i];
      adamw_one<T>(pp.v[0], m4.x, v4.x, gp.v[0], gs, lr, b1, b2, eps, eps_root, wd, bc1, bc2);
      adamw_one<T>(pp.v[1], m4.y, v4.y, gp.v[1], gs, lr, b1, b2, eps, eps_root, wd, bc1, bc2);
      adamw_one<T>(pp.v[2], m4.z, v4.z, gp.v[2], gs, lr, b1, b2, eps, eps_root, wd, bc1, bc2);
      adamw_one<T>(pp.v[3], m4.w, v4.w, gp.v[3], gs, lr, b1, b2, eps, eps_root, wd, bc1, bc2);
      reinterpret_cast<float4*>(e.m)[i] = m4;
      reinterpret_cast<float4*>(e.v)[i] = v4;
      reinterpret_cast<Pack*>(p)[i] = pp;
    }
  } else {
    for (long i = tid; i < e.n; i += stride) {
      float mi = e.m[i], vi = e.v[i];
      T pi = p[i];
      adamw_one<T>(pi, mi, vi, g[i], gs, lr, b1, b2, eps, eps_root, wd, bc1, bc2);
      e.m[i] = mi;
      e.v[i] = vi;
      p[i] = pi;
    }
  }
}

// Out-of-place AdamW over a list of tensors for steps that stay in an autograd graph, and the
// vector-Jacobian product of that step.  Entries are 12 eight-byte words.
//   forward : {p, g, m, v, p_out, m_out, v_out, -, -, -, n, -}
//   backward: {g, m, v, cp, cm, cv, dp, dg, dm, dv, n, -}  (cp/cm/cv: cotangents of the outputs,
//             null = zero; m and v are the moments *before* the step)
// p, g, p_out, cp, dp, dg have element type T; moments and their cotangents are fp32.
struct AdamTraceEntry {
  void* w[10];
  long n;
  long reserved;
};

template <typename T>
struct alignas(4 * sizeof(T)) Pack4 {
  T v[4];
};

// True when the element count and every non-null pointer allow 4-element packets.
__device__ __forceinline__ bool packs_ok(const AdamTraceEntry& e, int n_ptr, size_t t_bytes, unsigned t_mask) {
  if (e.n & 3) return false;
  for (int i = 0; i < n_ptr; ++i) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(e.w[i]);
    const size_t need = ((t_mask >> i) & 1u) ? 4 * t_bytes : 16;  // T-typed or fp32 slot
    if (a & (need - 1)) return false;
  }
  return true;
}

template <typename T>
__device__ __forceinline__ void adamw_fwd_one(T p, T g, float m, float v, T& po, float& mo, float& vo, float lr, float b1,
                                              float b2, float eps, float eps_root, float wd, float bc1, float bc2) {
  const float gi = to_float<T>(g);
  mo = b1 * m + (1.f - b1) * gi;
  vo = b2 * v + (1.f - b2) * gi * gi;
  const float pf = to_float<T>(p);
  const float upd = (mo / bc1) / (sqrtf(vo / bc2 + eps_root) + eps) + wd * pf;
  po = from_float<T>(pf - lr * upd);
}

template <typename T>
__global__ void adamw_traced_fwd_kernel(const AdamTraceEntry* __restrict__ table, float lr, float b1, float b2,
                                        float eps, float eps_root, float wd, float bc1, float bc2) {
  const AdamTraceEntry e = table[blockIdx.y];
  const T* p = static_cast<const T*>(e.w[0]);
  const T* g = static_cast<const T*>(e.w[1]);
  const float* m = static_cast<const float*>(e.w[2]);
  const float* v = static_cast<const float*>(e.w[3]);
  T* po = static_cast<T*>(e.w[4]);
  float* mo = static_cast<float*>(e.w[5]);
  float* vo = static_cast<float*>(e.w[6]);
  const long tid = blockIdx.x * long(blockDim.x) + threadIdx.x, stride = long(gridDim.x) * blockDim.x;
  if (packs_ok(e, 7, sizeof(T), 0b0010011u)) {
    for (long i = tid; i < (e.n >> 2); i += stride) {
      const Pack4<T> pp = reinterpret_cast<const Pack4<T>*>(p)[i], gp = reinterpret_cast<const Pack4<T>*>(g)[i];
      const float4 m4 = reinterpret_cast<const float4*>(m)[i], v4 = reinterpret_cast<const float4*>(v)[i];
      Pack4<T> o;
      float4 mo4, vo4;
      adamw_fwd_one<T>(pp.v[0], gp.v[0], m4.x, v4.x, o.v[0], mo4.x, vo4.x, lr, b1, b2, eps, eps_root, wd, bc1, bc2);
      adamw_fwd_one<T>(pp.v[1], gp.v[1], m4.y, v4.y, o.v[1], mo4.y, vo4.y, lr, b1, b2, eps, eps_root, wd, bc1, bc2);
      adamw_fwd_one<T>(pp.v[2], gp.v[2], m4.z, v4.z, o.v[2], mo4.z, vo4.z, lr, b1, b2, eps, eps_root, wd, bc1, bc2);
      adamw_fwd_one<T>(pp.v[3], gp.v[3], m4.w, v4.w, o.v[3], mo4.w, vo4.w, lr, b1, b2, eps, eps_root, wd, bc1, bc2);
      reinterpret_cast<Pack4<T>*>(po)[i] = o;
      reinterpret_cast<float4*>(mo)[i] = mo4;
      reinterpret_cast<float4*>(vo)[i] = vo4;
    }
    return;
  }
  for (long i = tid; i < e.n; i += stride)
    adamw_fwd_one<T>(p[i], g[i], m[i], v[i], po[i], mo[i], vo[i], lr, b1, b2, eps, eps_root, wd, bc1, bc2);
}

template <typename T>
__device__ __forceinline__ void adamw_vjp_one(T g, float m, float v, float c_p, float c_m, float c_v, T& dp, T& dg,
                                              float& dm, float& dv, float lr, float b1, float b2, float eps,
                                              float eps_root, float wd, float bc1, float bc2) {
  const float gi = to_float<T>(g);
  const float mi = b1 * m + (1.f - b1) * gi;  // the step's new moments, recomputed
  const float vi = b2 * v + (1.f - b2) * gi * gi;
  const float s = sqrtf(vi / bc2 + eps_root);
  const float den = s + eps;
  const float du = -lr * c_p;  // cotangent of the update direction
  const float d_mhat = du / den;
  const float d_s = -du * (mi / bc1) / (den * den);
  const float d_vhat = s > 0.f ? d_s / (2.f * s) : 0.f;
  const float d_m = c_m + d_mhat / bc1;
  const float d_v = c_v + d_vhat / bc2;
  dp = from_float<T>(c_p * (1.f - lr * wd));
  dg = from_float<T>((1.f - b1) * d_m + 2.f * (1.f - b2) * gi * d_v);
  dm = b1 * d_m;
  dv = b2 * d_v;
}

template <typename T>
__global__ void adamw_vjp_kernel(const AdamTraceEntry* __restrict__ table, float lr, float b1, float b2, float eps,
                                 float eps_root, float wd, float bc1, float bc2) {
  const AdamTraceEntry e = table[blockIdx.y];
  const T* g = static_cast<const T*>(e.w[0]);
  const float* m = static_cast<const float*>(e.w[1]);
  const float* v = static_cast<const float*>(e.w[2]);
  const T* cp = static_cast<const T*>(e.w[3]);
  const float* cm = static_cast<const float*>(e.w[4]);
  const float* cv = static_cast<const float*>(e.w[5]);
  T* dp = static_cast<T*>(e.w[6]);
  T* dg = static_cast<T*>(e.w[7]);
  float* dm = static_cast<float*>(e.w[8]);
  float* dv = static_cast<float*>(e.w[9]);
  const long tid = blockIdx.x * long(blockDim.x) + threadIdx.x, stride = long(gridDim.x) * blockDim.x;
  if (packs_ok(e, 10, sizeof(T), 0b0011001001u)) {  // null cotangent pointers are aligned by definition
    for (long i = tid; i < (e.n >> 2); i += stride) {
      const Pack4<T> gp = reinterpret_cast<const Pack4<T>*>(g)[i];
      const float4 m4 = reinterpret_cast<const float4*>(m)[i], v4 = reinterpret_cast<const float4*>(v)[i];
      Pack4<T> cpp;
      float c_p[4] = {0.f, 0.f, 0.f, 0.f};
      if (cp) {
        cpp = reinterpret_cast<const Pack4<T>*>(cp)[i];
#pragma unroll
        for (int k = 0; k < 4; ++k) c_p[k] = to_float<T>(cpp.v[k]);
      }
      const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
      const float4 cm4 = cm ? reinterpret_cast<const float4*>(cm)[i] : zero;
      const float4 cv4 = cv ? reinterpret_cast<const float4*>(cv)[i] : zero;
      Pack4<T> dpp, dgp;
      float4 dm4, dv4;
      adamw_vjp_one<T>(gp.v[0], m4.x, v4.x, c_p[0], cm4.x, cv4.x, dpp.v[0], dgp.v[0], dm4.x, dv4.x, lr, b1, b2, eps, eps_root, wd, bc1, bc2);
      adamw_vjp_one<T>(gp.v[1], m4.y, v4.y, c_p[1], cm4.y, cv4.y, dpp.v[1], dgp.v[1], dm4.y, dv4.y, lr, b1, b2, eps, eps_root, wd, bc1, bc2);
      adamw_vjp_one<T>(gp.v[2], m4.z, v4.z, c_p[2], cm4.z, cv4.z, dpp.v[2], dgp.v[2], dm4.z, dv4.z, lr, b1, b2, eps, eps_root, wd, bc1, bc2);
      adamw_vjp_one<T>(gp.v[3], m4.w, v4.w, c_p[3], cm4.w, cv4.w, dpp.v[3], dgp.v[3], dm4.w, dv4.w, lr, b1, b2, eps, eps_root, wd, bc1, bc2);
      reinterpret_cast<Pack4<T>*>(dp)[i] = dpp;
      reinterpret_cast<Pack4<T>*>(dg)[i] = dgp;
      reinterpret_cast<float4*>(dm)[i] = dm4;
      reinterpret_cast<float4*>(dv)[i] = dv4;
    }
    return;
  }
  for (long i = tid; i < e.n; i += stride)
    adamw_vjp_one<T>(g[i], m[i], v[i], cp ? to_float<T>(cp[i]) : 0.f, cm ? cm[i] : 0.f, cv ? cv[i] : 0.f, dp[i], dg[i],
                     dm[i], dv[i], lr, b1, b2, eps, eps_root, wd, bc1, bc2);
}

// Sum of squares over a list of tensors (entries reuse AdamEntry: g = data, n = elements).
// Every block writes one partial; `multi_sumsq_finish` adds them in a fixed order, so the
// result does not depend on scheduling.
template <typename T>
__global__ void multi_sumsq_kernel(const AdamEntry* __restrict__ table, float* __restrict__ partials) {
  __shared__ float red[32];
  const AdamEntry e = table[blockIdx.y];
  const T* g = static_cast<const T*>(e.g);
  constexpr int V = 16 / sizeof(T);
  float ss = 0.f;
  const long tid = blockIdx.x * long(blockDim.x) + threadIdx.x, stride = long(gridDim.x) * blockDim.x;
  if ((reinterpret_cast<uintptr_t>(g) & 15) == 0) {
    const long n_vec = e.n / V;
    for (long i = tid; i < n_vec; i += stride) {
      const Vec<T> v = load_vec(g + i * V);
#pragma unroll
      for (int k = 0; k < V; ++k) {
        const float f = to_float<T>(v.v[k]);
        ss = fmaf(f, f, ss);
      }
    }
    for (long i = n_vec * V + tid; i < e.n; i += stride) {
      const float f = to_float<T>(g[i]);
      ss = fmaf(f, f, ss);
    }
  } else {
    for (long i = tid; i < e.n; i += stride) {
      const float f = to_float<T>(g[i]);
      ss = fmaf(f, f, ss);
    }
  }
  ss = block_sum(ss, red);
  if (threadIdx.x == 0) partials[blockIdx.y * long(gridDim.x) + blockIdx.x] = ss;
}

// out[0] = sum(partials) (+ out[0] when `accumulate`); out[1] = min(1, max_norm / (sqrt(out[0]) + 1e-6))
// when max_norm > 0.
__global__ void multi_sumsq_finish_kernel(const float* __restrict__ partials, long n, float* __restrict__ out,
                                          int accumulate, float max_norm) {
  __shared__ float red[32];
  float ss = 0.f;
  for (long i = threadIdx.x; i < n; i += blockDim.x) ss += partials[i];
  ss = block_sum(ss, red);
  if (threadIdx.x == 0) {
    const float total = accumulate ? out[0] + ss : ss;
    out[0] = total;
    if (max_norm > 0.f) out[1] = fminf(1.f, max_norm / (sqrtf(total) + 1e-6f));
  }
}

template <typename T>
__global__ void row_sumsq_kernel(const T* __restrict__ x, float* __restrict__ out, long d, long ldx) {
  __shared__ float red[32];
  const long r = blockIdx.x;
  const T* xr = x + r * ldx;
  float ss = 0.f;
  for (long i = threadIdx.x; i < d; i += blockDim.x) {
    const float f = to_float<T>(xr[i]);
    ss = fmaf(f, f, ss);
  }
  ss = block_sum(ss, red);
  if (threadIdx.x == 0) out[r] += ss;
}

static inline int grid_for(long n, int per_block) {
  long b = (n + per_block - 1) / per_block;
  const long cap = 148L * 16;
  return int(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace bgn

using namespace bgn;

#define BGN_DISPATCH(type, ...)                         \
  switch (type) {                                       \
    case 0: { using T = __half; __VA_ARGS__; break; }   \
    case 1: { using T = __nv_bfloat16; __VA_ARGS__; break; } \
    case 2: { using T = float; __VA_ARGS__; break; }    \
    default: return int(cudaErrorInvalidValue);         \
  }

static inline int vec_threads(int d, int vec) {
  int t = (d / vec + 31) / 32 * 32;
  return t < 32 ? 32 : (t > 512 ? 512 : t);
}

extern "C" int bgn_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long rows, int d,
                               float eps, int type, cudaStream_t st) {
  BGN_DISPATCH(type, {
    if (d % Vec<T>::N) return int(cudaErrorInvalidValue);
    rmsnorm_fwd_kernel<T><<<rows, vec_threads(d, Vec<T>::N), 0, st>>>((const T*)x, (const T*)w, (T*)y, rstd, d, eps);
  });
  return int(cudaGetLastError());
}

extern "C" int bgn_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd,
                               void* dx, float* dw_partial, int n_partial, long rows, int d, int type,
                               cudaStream_t st) {
  BGN_DISPATCH(type, {
    const int threads = vec_threads(d, Vec<T>::N);
    if (d % Vec<T>::N || (dw_partial && d > threads * Vec<T>::N * 4)) return int(cudaErrorInvalidValue);
    const int grid = dw_partial ? n_partial : int(rows < 148L * 8 ? rows : 148L * 8);
    rmsnorm_bwd_kernel<T><<<grid, threads, 0, st>>>((const T*)dy, (const T*)x, (const T*)w, rstd, (T*)dx, dw_partial, rows, d);
  });
  return int(cudaGetLastError());
}

extern "C" int bgn_rmsnorm_bwd_bwd(const void* U, const float* Vw, const void* dy, const void* x, const void* w,
                                   const float* rstd, void* d_dy, void* d_x, float* dw_partial, int n_partial,
                                   long rows, int d, int type, cudaStream_t st) {
  BGN_DISPATCH(type, {
    const int threads = vec_threads(d, Vec<T>::N);
    if (d % Vec<T>::N || d > threads * Vec<T>::N * 4 || n_partial < 1) return int(cudaErrorInvalidValue);
    rmsnorm_bwd_bwd_kernel<T><<<n_partial, threads, 0, st>>>((const T*)U, Vw, (const T*)dy, (const T*)x, (const T*)w, rstd,
                                                            (T*)d_dy, (T*)d_x, dw_partial, rows, d);
  });
  return int(cudaGetLastError());
}

extern "C" int bgn_swiglu_bwd_bwd(const void* cg, const void* cu, const void* dy, const void* g, const void* u, void* d_dy,
                                  void* d_g, void* d_u, long n, int type, cudaStream_t st) {
  BGN_DISPATCH(type, {
    if (n % Vec<T>::N) return int(cudaErrorInvalidValue);
    swiglu_bwd_bwd_kernel<T><<<grid_for(n, 256 * Vec<T>::N), 256, 0, st>>>((const T*)cg, (const T*)cu, (const T*)dy,
                                                                           (const T*)g, (const T*)u, (T*)d_dy, (T*)d_g,
                                                                           (T*)d_u, n);
  });
  return int(cudaGetLastError());
}

extern "C" int bgn_layernorm_fwd(const void* x, const void* w, const void* b, void* y, float* mean,
                                 float* rstd, long rows, int d, float eps, int type, cudaStream_t st) {
  BGN_DISPATCH(type, {
    if (d % Vec<T>::N) return int(cudaErrorInvalidValue);
    layernorm_fwd_kernel<T><<<rows, vec_threads(d, Vec<T>::N), 0, st>>>((const T*)x, (const T*)w, (const T*)b, (T*)y, mean, rstd, d, eps);
  });
  return int(cudaGetLastError());
}

extern "C" int bgn_layernorm_bwd(const void* dy, const void* x, const void* w, const float* mean,
                                 const float* rstd, void* dx, float* dw_partial, float* db_partial,
                                 int n_partial, long rows, int d, int type, cudaStream_t st) {
  BGN_DISPATCH(type, {
    const int threads = vec_threads(d, Vec<T>::N);
    if (d % Vec<T>::N || (dw_partial && d > threads * Vec<T>::N * 4)) return int(cudaErrorInvalidValue);
    const int grid = dw_partial ? n_partial : int(rows < 148L * 8 ? rows : 148L * 8);
    layernorm_bwd_kernel<T><<<grid, threads, 0, st>>>((const T*)dy, (const T*)x, (const T*)w, mean, rstd, (T*)dx, dw_partial, db_partial, rows, d);
  });
  return int(cudaGetLastError());
}

extern "C" int bgn_layernorm_bwd_bwd(const void* U, const float* Vw, const float* Sb, const void* dy, const void* x,
                                     const void* w, const float* mean, const float* rstd, void* d_dy, void* d_x,
                                     float* dw_partial, int n_partial, long rows, int d, int type, cudaStream_t st) {
  BGN_DISPATCH(type, {
    const int threads = vec_threads(d, Vec<T>::N);
    if (d % Vec<T>::N || d > threads * Vec<T>::N * 4 || n_partial < 1) return int(cudaErrorInvalidValue);
    layernorm_bwd_bwd_kernel<T><<<n_partial, threads, 0, st>>>((const T*)U, Vw, Sb, (const T*)dy, (const T*)x,
                                                              (const T*)w, mean, rstd, (T*)d_dy, (T*)d_x, dw_partial,
                                                              rows, d);
  });
  return int(cudaGetLastError());
}

extern "C" int bgn_rotary(const void* x, const float* cosT, const float* sinT, void* y, long B, int S,
                          int H, int D, int rot, int inverse, int type, cudaStream_t st) {
  const long heads = B * S * H;
  const long total = heads * (D - rot / 2);
  BGN_DISPATCH(type, {
    constexpr int V = Vec<T>::N;
    const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
    if (aligned && (rot / 2) % V == 0 && (D - rot) % V == 0 && D % V == 0) {
      const long packets = heads * ((rot / 2) / V + (D - rot) / V);
      rotary_vec_kernel<T><<<grid_for(packets, 256), 256, 0, st>>>((const T*)x, cosT, sinT, (T*)y, packets, S, H, D, rot,
                                                                   inverse ? -1.f : 1.f);
    } else {
      rotary_kernel<T><<<grid_for(total, 256), 256, 0, st>>>((const T*)x, cosT, sinT, (T*)y, total, S, H, D, rot, inverse ? -1.f : 1.f);
    }
  });
  return int(cudaGetLastError());
}

extern "C" int bgn_swiglu_fwd(const void* g, const void* u, void* y, long n, int type, cudaStream_t st) {
  BGN_DISPATCH(type, {
    if (n % Vec<T>::N) return int(cudaErrorInvalidValue);
    swiglu_fwd_kernel<T><<<grid_for(n, 256 * Vec<T>::N), 256, 0, st>>>((const T*)g, (const T*)u, (T*)y, n);
  });
  return int(cudaGetLastError());
}

extern "C" int bgn_swiglu_bwd(const void* dy, const void* g, const void* u, void* dg, void* du, long n,
                              int type, cudaStream_t st) {
  BGN_DISPATCH(type, {
    if (n % Vec<T>::N) return int(cudaErrorInvalidValue);
    swiglu_bwd_kernel<T><<<grid_for(n, 256 * Vec<T>::N), 256, 0, st>>>((const T*)dy, (const T*)g, (const T*)u, (T*)dg, (T*)du, n);
  });
  return int(cudaGetLastError());
}

extern "C" int bgn_gelu_fwd(const void* x, void* y, long n, int tanh_approx, int type, cudaStream_t st) {
  BGN_DISPATCH(type, {
    if (n % Vec<T>::N) return int(cudaErrorInvalidValue);
    gelu_fwd_kernel<T><<<grid_for(n, 256 * Vec<T>::N), 256, 0, st>>>((const T*)x, (T*)y, n, tanh_approx);
  });
  return int(cudaGetLastError());
}

extern "C" int bgn_softmax_bwd_bwd(const void* c, const void* dy, const void* y, void* d_dy, void* d_y, long rows, int n,
                                   int type, cudaStream_t st) {
  BGN_DISPATCH(type, {
    if (n % Vec<T>::N || rows <= 0) return int(cudaErrorInvalidValue);
    long blocks = (rows + 7) / 8;  // eight warps (rows) per block
    if (blocks > 148L * 32) blocks = 148L * 32;
    softmax_bwd_bwd_kernel<T><<<int(blocks), 256, 0, st>>>((const T*)c, (const T*)dy, (const T*)y, (T*)d_dy, (T*)d_y,
                                                           rows, n);
  });
  return int(cudaGetLastError());
}

extern "C" int bgn_gelu_bwd_bwd(const void* c, const void* dy, const void* x, void* d_dy, void* d_x, long n,
                                int tanh_approx, int type, cudaStream_t st) {
  BGN_DISPATCH(type, {
    if (n % Vec<T>::N) return int(cudaErrorInvalidValue);
    gelu_bwd_bwd_kernel<T><<<grid_for(n, 256 * Vec<T>::N), 256, 0, st>>>((const T*)c, (const T*)dy, (const T*)x,
                                                                         (T*)d_dy, (T*)d_x, n, tanh_approx);
  });
  return int(cudaGetLastError());
}

extern "C" int bgn_gelu_bwd(const void* dy, const void* x, void* dx, long n, int tanh_approx, int type,
                            cudaStream_t st) {
  BGN_DISPATCH(type, {
    if (n % Vec<T>::N) return int(cudaErrorInvalidValue);
    gelu_bwd_kernel<T><<<grid_for(n, 256 * Vec<T>::N), 256, 0, st>>>((const T*)dy, (const T*)x, (T*)dx, n, tanh_approx);
  });
  return int(cudaGetLastError());
}

extern "C" int bgn_ce_fwd(const void* logits, const long* targets, float* loss, float* lse, long T_,
                          int V, long ignore_index, int type, cudaStream_t st) {
  BGN_DISPATCH(type, {
    ce_fwd_kernel<T><<<T_, 512, 0, st>>>((const T*)logits, targets, loss, lse, V, ignore_index);
  });
  return int(cudaGetLastError());
}

// Backward of ce_bwd (dlogits = (softmax(z) - onehot) * dloss per row).  Given the cotangent C of
// dlogits:  with p = softmax(z) and s = sum_v C_v p_v,
//   d_dloss = s - C_target,    d_z_v = dloss * p_v * (C_v - s);   both zero for ignored rows.
namespace bgn {
template <typename T>
__global__ void ce_bwd_bwd_kernel(const T* __restrict__ C, const T* __restrict__ logits,
                                  const long* __restrict__ targets, const float* __restrict__ lse,
                                  const float* __restrict__ dloss, T* __restrict__ d_logits,
                                  float* __restrict__ d_dloss, int V_, long ignore_index) {
  __shared__ float red[32];
  const long r = blockIdx.x;
  const T* z = logits + r * V_;
  const T* c = C + r * V_;
  T* dz = d_logits + r * V_;
  const long t = targets[r];
  const bool ignored = t == ignore_index;
  const float l = lse[r];
  constexpr int V = Vec<T>::N;
  const bool vec_ok = (V_ % V) == 0;
  float s = 0.f;
  if (!ignored) {
    if (vec_ok) {
      for (int i = threadIdx.x * V; i < V_; i += blockDim.x * V) {
        const Vec<T> zv = load_vec(z + i), cv = load_vec(c + i);
#pragma unroll
        for (int k = 0; k < V; ++k) s = fmaf(to_float<T>(cv.v[k]), __expf(to_float<T>(zv.v[k]) - l), s);
      }
    } else {
      for (int i = threadIdx.x; i < V_; i += blockDim.x) s = fmaf(to_float<T>(c[i]), __expf(to_float<T>(z[i]) - l), s);
    }
  }
  s = block_sum(s, red);
  const float g = ignored ? 0.f : dloss[r];
  if (threadIdx.x == 0) d_dloss[r] = ignored ? 0.f : s - to_float<T>(c[t]);
  if (vec_ok) {
    for (int i = threadIdx.x * V; i < V_; i += blockDim.x * V) {
      const Vec<T> zv = load_vec(z + i), cv = load_vec(c + i);
      Vec<T> o;
#pragma unroll
      for (int k = 0; k < V; ++k)
        o.v[k] = from_float<T>(g * __expf(to_float<T>(zv.v[k]) - l) * (to_float<T>(cv.v[k]) - s));
      store_vec(dz + i, o);
    }
  } else {
    for (int i = threadIdx.x; i < V_; i += blockDim.x)
      dz[i] = from_float<T>(g * __expf(to_float<T>(z[i]) - l) * (to_float<T>(c[i]) - s));
  }
}
}  // namespace bgn

extern "C" int bgn_ce_bwd_bwd(const void* C, const void* logits, const long* targets, const float* lse,
                              const float* dloss, void* d_logits, float* d_dloss, long T_, int V, long ignore_index,
                              int type, cudaStream_t st) {
  BGN_DISPATCH(type, {
    ce_bwd_bwd_kernel<T><<<T_, 512, 0, st>>>((const T*)C, (const T*)logits, targets, lse, dloss, (T*)d_logits, d_dloss,
                                             V, ignore_index);
  });
  return int(cudaGetLastError());
}

extern "C" int bgn_ce_bwd(const void* logits, const long* targets, const float* lse, const float* dloss,
                          void* dlogits, long T_, int V, long ignore_index, int type, cudaStream_t st) {
  BGN_DISPATCH(type, {
    ce_bwd_kernel<T><<<T_, 512, 0, st>>>((const T*)logits, targets, lse, dloss, (T*)dlogits, V, ignore_index);
  });
  return int(cudaGetLastError());
}

extern "C" int bgn_adamw_step(float* p, float* m, float* v, const void* g, void* pm, long n, float lr,
                              float b1, float b2, float eps, float eps_root, float wd, float bc1,
                              float bc2, float gscale, int g_type, int model_type, cudaStream_t st) {
  const int grid = grid_for(n, 256);
#define ADAM_LAUNCH(G, M) \
  adamw_kernel<G, M><<<grid, 256, 0, st>>>(p, m, v, (const G*)g, (M*)pm, n, lr, b1, b2, eps, eps_root, wd, bc1, bc2, gscale)
  if (g_type == 1 && model_type == 1) ADAM_LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (g_type == 2 && model_type == 1) ADAM_LAUNCH(float, __nv_bfloat16);
  else if (g_type == 2 && model_type == 2) ADAM_LAUNCH(float, float);
  else if (g_type == 0 && model_type == 0) ADAM_LAUNCH(__half, __half);
  else if (g_type == 2 && model_type == 0) ADAM_LAUNCH(float, __half);
  else return int(cudaErrorInvalidValue);
#undef ADAM_LAUNCH
  return int(cudaGetLastError());
}

extern "C" int bgn_adamw_multi(const void* table, int n_tensors, long max_n, float lr, float b1, float b2,
                               float eps, float eps_root, float wd, float bc1, float bc2, float gscale,
                               const float* coef, int type, cudaStream_t st) {
  if (n_tensors <= 0) return 0;
  if (n_tensors > 65535) return int(cudaErrorInvalidValue);
  // About eight 4-element packets per thread for the largest tensor, at most 128 blocks per
  // tensor; blocks of shorter tensors run out of work early and retire.
  long per_row = (max_n / 4 + 256 * 8 - 1) / (256 * 8);
  per_row = per_row < 1 ? 1 : (per_row > 128 ? 128 : per_row);
  const dim3 grid((unsigned)per_row, (unsigned)n_tensors);
  BGN_DISPATCH(type, {
    adamw_multi_kernel<T><<<grid, 256, 0, st>>>((const AdamEntry*)table, lr, b1, b2, eps, eps_root, wd, bc1, bc2,
                                                gscale, coef);
  });
  return int(cudaGetLastError());
}

static inline dim3 multi_grid(int n_tensors, long max_n) {
  long per_row = (max_n / 4 + 256 * 8 - 1) / (256 * 8);
  per_row = per_row < 1 ? 1 : (per_row > 128 ? 128 : per_row);
  return dim3((unsigned)per_row, (unsigned)n_tensors);
}

extern "C" int bgn_adamw_traced(const void* table, int n_tensors, long max_n, int backward, float lr, float b1,
                                float b2, float eps, float eps_root, float wd, float bc1, float bc2, int type,
                                cudaStream_t st) {
  if (n_tensors <= 0) return 0;
  if (n_tensors > 65535) return int(cudaErrorInvalidValue);
  const dim3 grid = multi_grid(n_tensors, max_n);
  BGN_DISPATCH(type, {
    if (backward)
      adamw_vjp_kernel<T><<<grid, 256, 0, st>>>((const AdamTraceEntry*)table, lr, b1, b2, eps, eps_root, wd, bc1, bc2);
    else
      adamw_traced_fwd_kernel<T><<<grid, 256, 0, st>>>((const AdamTraceEntry*)table, lr, b1, b2, eps, eps_root, wd,
                                                       bc1, bc2);
  });
  return int(cudaGetLastError());
}

extern "C" int bgn_multi_sumsq_blocks(void) { return 128; }

extern "C" int bgn_multi_sumsq(const void* table, int n_tensors, long max_n, float* partials, float* out,
                               int accumulate, float max_norm, int type, cudaStream_t st) {
  if (n_tensors <= 0 || n_tensors > 65535) return int(cudaErrorInvalidValue);
  // Blocks per tensor follow the largest one (about eight 16-byte packets per thread, at most
  // 128); blocks of shorter tensors write a zero partial and retire.
  int blocks = int((max_n / 8 + 256 * 8 - 1) / (256 * 8));
  blocks = blocks < 1 ? 1 : (blocks > 128 ? 128 : blocks);
  const dim3 grid((unsigned)blocks, (unsigned)n_tensors);
  BGN_DISPATCH(type, { multi_sumsq_kernel<T><<<grid, 256, 0, st>>>((const AdamEntry*)table, partials); });
  multi_sumsq_finish_kernel<<<1, 1024, 0, st>>>(partials, long(blocks) * n_tensors, out, accumulate, max_norm);
  return int(cudaGetLastError());
}

extern "C" int bgn_row_sumsq(const void* x, float* out, long rows, long d, long ldx, int type,
                             cudaStream_t st) {
  BGN_DISPATCH(type, { row_sumsq_kernel<T><<<rows, 256, 0, st>>>((const T*)x, out, d, ldx); });
  return int(cudaGetLastError());
}
