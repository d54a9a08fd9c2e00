// Python bindings: tensor checks, output allocation, current-stream lookup; the kernels
// themselves are behind the C interface in kernels.h.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <array>
#include <cstring>

#include <map>
#include <mutex>

#include "kernels.h"
#include "kernels_cov.h"
#include "kernels_peer.h"
#include "kernels_gemm.h"

namespace {

int type_code(const at::Tensor& t) {
  switch (t.scalar_type()) {
    case at::kHalf: return 0;
    case at::kBFloat16: return 1;
    case at::kFloat: return 2;
    default: TORCH_CHECK(false, "bergson_b200: unsupported dtype ", t.scalar_type());
  }
}

int fmt16(const at::Tensor& t) {
  TORCH_CHECK(t.scalar_type() == at::kHalf || t.scalar_type() == at::kBFloat16,
              "bergson_b200: tensor-core kernels take fp16 or bf16 inputs, got ", t.scalar_type());
  return t.scalar_type() == at::kBFloat16 ? 1 : 0;
}

void check(int err, const char* what) {
  TORCH_CHECK(err == 0, "bergson_b200: ", what, " failed: ",
              cudaGetErrorString(static_cast<cudaError_t>(err)));
}

cudaStream_t stream() { return at::cuda::getCurrentCUDAStream().stream(); }

#define CHECK_CUDA_CONTIG(x) TORCH_CHECK((x).is_cuda() && (x).is_contiguous(), #x " must be a contiguous CUDA tensor")

// One status word per device, written by kernels whose bounded waits run out.
at::Tensor status_tensor(int device) {
  static std::mutex mu;
  static std::map<int, at::Tensor> words;
  std::lock_guard<std::mutex> lock(mu);
  auto it = words.find(device);
  if (it == words.end()) {
    it = words.emplace(device, at::zeros({1}, at::TensorOptions().dtype(at::kInt).device(at::kCUDA, device))).first;
  }
  return it->second;
}

// Arrival counters of the contraction kernel: zero between launches (the kernel resets them), so
// one buffer per device serves every call issued on one stream.
at::Tensor contract_counters(int device, int64_t n) {
  static std::mutex mu;
  static std::map<int, at::Tensor> bufs;
  std::lock_guard<std::mutex> lock(mu);
  auto it = bufs.find(device);
  if (it == bufs.end() || it->second.numel() < n) {
    auto t = at::zeros({std::max<int64_t>(n, 256)}, at::TensorOptions().dtype(at::kInt).device(at::kCUDA, device));
    if (it == bufs.end()) it = bufs.emplace(device, t).first;
    else it->second = t;
  }
  return it->second;
}

int* status_ptr(const at::Tensor& like) { return status_tensor(like.get_device()).data_ptr<int>(); }
// Blocks (= rows of partial weight-gradient sums) of the norm backward kernels: narrow rows use
// small blocks, so more of them are needed to fill the SMs.
static int64_t partial_blocks(int64_t d) { return d <= 1024 ? 148 * 8 : (d <= 2048 ? 148 * 4 : 148 * 2); }

int* status_ptr_current() { return status_tensor(at::cuda::current_device()).data_ptr<int>(); }

}  // namespace

std::vector<at::Tensor> rmsnorm_fwd(at::Tensor x, at::Tensor w, double eps) {
  CHECK_CUDA_CONTIG(x); CHECK_CUDA_CONTIG(w);
  c10::cuda::CUDAGuard guard(x.device());
  auto y = at::empty_like(x);
  auto rstd = at::empty({x.size(0)}, x.options().dtype(at::kFloat));
  auto wc = w.scalar_type() == x.scalar_type() ? w : w.to(x.scalar_type());
  check(bgn_rmsnorm_fwd(x.data_ptr(), wc.data_ptr(), y.data_ptr(), rstd.data_ptr<float>(), x.size(0),
                        (int)x.size(1), (float)eps, type_code(x), stream()), "rmsnorm_fwd");
  return {y, rstd};
}

std::vector<at::Tensor> rmsnorm_bwd(at::Tensor dy, at::Tensor x, at::Tensor w, at::Tensor rstd, bool need_dw) {
  CHECK_CUDA_CONTIG(dy); CHECK_CUDA_CONTIG(x);
  c10::cuda::CUDAGuard guard(x.device());
  auto dx = at::empty_like(x);
  auto wc = w.scalar_type() == x.scalar_type() ? w : w.to(x.scalar_type());
  at::Tensor partial, dw;
  int n_partial = 0;
  if (need_dw) {
    n_partial = (int)std::min<int64_t>(x.size(0), partial_blocks(x.size(1)));
    partial = at::empty({n_partial, x.size(1)}, x.options().dtype(at::kFloat));
  }
  check(bgn_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), wc.data_ptr(), rstd.data_ptr<float>(), dx.data_ptr(),
                        need_dw ? partial.data_ptr<float>() : nullptr, n_partial, x.size(0), (int)x.size(1),
                        type_code(x), stream()), "rmsnorm_bwd");
  if (need_dw) dw = partial.sum(0).to(w.scalar_type());
  return {dx, dw};
}

std::vector<at::Tensor> layernorm_fwd(at::Tensor x, at::Tensor w, c10::optional<at::Tensor> b, double eps) {
  CHECK_CUDA_CONTIG(x);
  c10::cuda::CUDAGuard guard(x.device());
  auto y = at::empty_like(x);
  auto mean = at::empty({x.size(0)}, x.options().dtype(at::kFloat));
  auto rstd = at::empty_like(mean);
  auto wc = w.to(x.scalar_type()).contiguous();
  at::Tensor bc;
  if (b.has_value()) bc = b->to(x.scalar_type()).contiguous();
  check(bgn_layernorm_fwd(x.data_ptr(), wc.data_ptr(), b.has_value() ? bc.data_ptr() : nullptr, y.data_ptr(),
                          mean.data_ptr<float>(), rstd.data_ptr<float>(), x.size(0), (int)x.size(1), (float)eps,
                          type_code(x), stream()), "layernorm_fwd");
  return {y, mean, rstd};
}

std::vector<at::Tensor> layernorm_bwd(at::Tensor dy, at::Tensor x, at::Tensor w, at::Tensor mean, at::Tensor rstd,
                                      bool need_dw) {
  CHECK_CUDA_CONTIG(dy); CHECK_CUDA_CONTIG(x);
  c10::cuda::CUDAGuard guard(x.device());
  auto dx = at::empty_like(x);
  auto wc = w.to(x.scalar_type()).contiguous();
  at::Tensor pw, pb, dw, db;
  int n_partial = 0;
  if (need_dw) {
    n_partial = (int)std::min<int64_t>(x.size(0), partial_blocks(x.size(1)));
    pw = at::empty({n_partial, x.size(1)}, x.options().dtype(at::kFloat));
    pb = at::empty_like(pw);
  }
  check(bgn_layernorm_bwd(dy.data_ptr(), x.data_ptr(), wc.data_ptr(), mean.data_ptr<float>(), rstd.data_ptr<float>(),
                          dx.data_ptr(), need_dw ? pw.data_ptr<float>() : nullptr,
                          need_dw ? pb.data_ptr<float>() : nullptr, n_partial, x.size(0), (int)x.size(1),
                          type_code(x), stream()), "layernorm_bwd");
  if (need_dw) {
    dw = pw.sum(0).to(w.scalar_type());
    db = pb.sum(0).to(w.scalar_type());
  }
  return {dx, dw, db};
}

// Backward of rmsnorm_bwd: (cotangent of dx, of dw) -> (d_dy, d_x, d_w).
std::vector<at::Tensor> rmsnorm_bwd_bwd(at::Tensor cu, at::Tensor cw, at::Tensor dy, at::Tensor x, at::Tensor w,
                                        at::Tensor rstd) {
  CHECK_CUDA_CONTIG(cu); CHECK_CUDA_CONTIG(dy); CHECK_CUDA_CONTIG(x);
  TORCH_CHECK(cu.scalar_type() == x.scalar_type() && dy.scalar_type() == x.scalar_type() && cu.numel() == x.numel() &&
              dy.numel() == x.numel() && x.dim() == 2);
  c10::cuda::CUDAGuard guard(x.device());
  auto wc = w.to(x.scalar_type()).contiguous();
  auto vw = cw.to(at::kFloat).contiguous();
  TORCH_CHECK(vw.numel() == x.size(1));
  auto d_dy = at::empty_like(x), d_x = at::empty_like(x);
  const int n_partial = (int)std::min<int64_t>(x.size(0), partial_blocks(x.size(1)));
  auto pw = at::empty({n_partial, x.size(1)}, x.options().dtype(at::kFloat));
  check(bgn_rmsnorm_bwd_bwd(cu.data_ptr(), vw.data_ptr<float>(), dy.data_ptr(), x.data_ptr(), wc.data_ptr(),
                            rstd.data_ptr<float>(), d_dy.data_ptr(), d_x.data_ptr(), pw.data_ptr<float>(), n_partial,
                            x.size(0), (int)x.size(1), type_code(x), stream()), "rmsnorm_bwd_bwd");
  return {d_dy, d_x, pw.sum(0).to(w.scalar_type())};
}

std::vector<at::Tensor> swiglu_bwd_bwd(at::Tensor cg, at::Tensor cu, at::Tensor dy, at::Tensor g, at::Tensor u) {
  CHECK_CUDA_CONTIG(cg); CHECK_CUDA_CONTIG(cu); CHECK_CUDA_CONTIG(dy); CHECK_CUDA_CONTIG(g); CHECK_CUDA_CONTIG(u);
  TORCH_CHECK(cg.numel() == g.numel() && cu.numel() == g.numel() && dy.numel() == g.numel() && u.numel() == g.numel() &&
              cg.scalar_type() == g.scalar_type() && cu.scalar_type() == g.scalar_type() &&
              dy.scalar_type() == g.scalar_type() && u.scalar_type() == g.scalar_type());
  c10::cuda::CUDAGuard guard(g.device());
  auto d_dy = at::empty_like(g), d_g = at::empty_like(g), d_u = at::empty_like(g);
  check(bgn_swiglu_bwd_bwd(cg.data_ptr(), cu.data_ptr(), dy.data_ptr(), g.data_ptr(), u.data_ptr(), d_dy.data_ptr(),
                           d_g.data_ptr(), d_u.data_ptr(), g.numel(), type_code(g), stream()), "swiglu_bwd_bwd");
  return {d_dy, d_g, d_u};
}

// Backward of layernorm_bwd: (cotangent of dx, of dw, of db) -> (d_dy, d_x, d_w).
std::vector<at::Tensor> layernorm_bwd_bwd(at::Tensor cu, at::Tensor cw, at::Tensor cb, at::Tensor dy, at::Tensor x,
                                          at::Tensor w, at::Tensor mean, at::Tensor rstd) {
  CHECK_CUDA_CONTIG(cu); CHECK_CUDA_CONTIG(dy); CHECK_CUDA_CONTIG(x);
  TORCH_CHECK(cu.scalar_type() == x.scalar_type() && dy.scalar_type() == x.scalar_type() && cu.numel() == x.numel() &&
              dy.numel() == x.numel() && x.dim() == 2);
  c10::cuda::CUDAGuard guard(x.device());
  auto wc = w.to(x.scalar_type()).contiguous();
  auto vw = cw.to(at::kFloat).contiguous(), sb = cb.to(at::kFloat).contiguous();
  TORCH_CHECK(vw.numel() == x.size(1) && sb.numel() == x.size(1));
  auto d_dy = at::empty_like(x), d_x = at::empty_like(x);
  const int n_partial = (int)std::min<int64_t>(x.size(0), partial_blocks(x.size(1)));
  auto pw = at::empty({n_partial, x.size(1)}, x.options().dtype(at::kFloat));
  check(bgn_layernorm_bwd_bwd(cu.data_ptr(), vw.data_ptr<float>(), sb.data_ptr<float>(), dy.data_ptr(), x.data_ptr(),
                              wc.data_ptr(), mean.data_ptr<float>(), rstd.data_ptr<float>(), d_dy.data_ptr(),
                              d_x.data_ptr(), pw.data_ptr<float>(), n_partial, x.size(0), (int)x.size(1), type_code(x),
                              stream()), "layernorm_bwd_bwd");
  return {d_dy, d_x, pw.sum(0).to(w.scalar_type())};
}

at::Tensor rotary(at::Tensor x, at::Tensor cos, at::Tensor sin, int64_t rot, bool inverse) {
  CHECK_CUDA_CONTIG(x);
  TORCH_CHECK(x.dim() == 4, "rotary expects [B, S, H, D]");
  c10::cuda::CUDAGuard guard(x.device());
  auto y = at::empty_like(x);
  auto c = cos.to(at::kFloat).contiguous(), s = sin.to(at::kFloat).contiguous();
  TORCH_CHECK(c.size(0) >= x.size(1) && c.size(1) == rot / 2, "rotary table shape mismatch");
  check(bgn_rotary(x.data_ptr(), c.data_ptr<float>(), s.data_ptr<float>(), y.data_ptr(), x.size(0), (int)x.size(1),
                   (int)x.size(2), (int)x.size(3), (int)rot, inverse ? 1 : 0, type_code(x), stream()), "rotary");
  return y;
}

at::Tensor swiglu_fwd(at::Tensor g, at::Tensor u) {
  CHECK_CUDA_CONTIG(g); CHECK_CUDA_CONTIG(u);
  c10::cuda::CUDAGuard guard(g.device());
  auto y = at::empty_like(g);
  check(bgn_swiglu_fwd(g.data_ptr(), u.data_ptr(), y.data_ptr(), g.numel(), type_code(g), stream()), "swiglu_fwd");
  return y;
}

std::vector<at::Tensor> swiglu_bwd(at::Tensor dy, at::Tensor g, at::Tensor u) {
  CHECK_CUDA_CONTIG(dy); CHECK_CUDA_CONTIG(g); CHECK_CUDA_CONTIG(u);
  c10::cuda::CUDAGuard guard(g.device());
  auto dg = at::empty_like(g), du = at::empty_like(u);
  check(bgn_swiglu_bwd(dy.data_ptr(), g.data_ptr(), u.data_ptr(), dg.data_ptr(), du.data_ptr(), g.numel(),
                       type_code(g), stream()), "swiglu_bwd");
  return {dg, du};
}

at::Tensor gelu_fwd(at::Tensor x, bool tanh_approx) {
  CHECK_CUDA_CONTIG(x);
  c10::cuda::CUDAGuard guard(x.device());
  auto y = at::empty_like(x);
  check(bgn_gelu_fwd(x.data_ptr(), y.data_ptr(), x.numel(), tanh_approx, type_code(x), stream()), "gelu_fwd");
  return y;
}

std::vector<at::Tensor> softmax_bwd_bwd(at::Tensor c, at::Tensor dy, at::Tensor y) {
  CHECK_CUDA_CONTIG(c); CHECK_CUDA_CONTIG(dy); CHECK_CUDA_CONTIG(y);
  TORCH_CHECK(c.scalar_type() == y.scalar_type() && dy.scalar_type() == y.scalar_type() && c.numel() == y.numel() &&
              dy.numel() == y.numel() && y.dim() >= 1);
  c10::cuda::CUDAGuard guard(y.device());
  auto d_dy = at::empty_like(y), d_y = at::empty_like(y);
  const int64_t n = y.size(-1);
  check(bgn_softmax_bwd_bwd(c.data_ptr(), dy.data_ptr(), y.data_ptr(), d_dy.data_ptr(), d_y.data_ptr(), y.numel() / n,
                            (int)n, type_code(y), stream()), "softmax_bwd_bwd");
  return {d_dy, d_y};
}

std::vector<at::Tensor> gelu_bwd_bwd(at::Tensor c, at::Tensor dy, at::Tensor x, bool tanh_approx) {
  CHECK_CUDA_CONTIG(c); CHECK_CUDA_CONTIG(dy); CHECK_CUDA_CONTIG(x);
  TORCH_CHECK(c.scalar_type() == x.scalar_type() && dy.scalar_type() == x.scalar_type() && c.numel() == x.numel() &&
              dy.numel() == x.numel());
  c10::cuda::CUDAGuard guard(x.device());
  auto d_dy = at::empty_like(x), d_x = at::empty_like(x);
  check(bgn_gelu_bwd_bwd(c.data_ptr(), dy.data_ptr(), x.data_ptr(), d_dy.data_ptr(), d_x.data_ptr(), x.numel(),
                         tanh_approx, type_code(x), stream()), "gelu_bwd_bwd");
  return {d_dy, d_x};
}

at::Tensor gelu_bwd(at::Tensor dy, at::Tensor x, bool tanh_approx) {
  CHECK_CUDA_CONTIG(dy); CHECK_CUDA_CONTIG(x);
  c10::cuda::CUDAGuard guard(x.device());
  auto dx = at::empty_like(x);
  check(bgn_gelu_bwd(dy.data_ptr(), x.data_ptr(), dx.data_ptr(), x.numel(), tanh_approx, type_code(x), stream()),
        "gelu_bwd");
  return dx;
}

std::vector<at::Tensor> ce_fwd(at::Tensor logits, at::Tensor targets, int64_t ignore_index) {
  CHECK_CUDA_CONTIG(logits); CHECK_CUDA_CONTIG(targets);
  TORCH_CHECK(logits.dim() == 2 && targets.scalar_type() == at::kLong);
  c10::cuda::CUDAGuard guard(logits.device());
  auto loss = at::empty({logits.size(0)}, logits.options().dtype(at::kFloat));
  auto lse = at::empty_like(loss);
  if (logits.size(0) > 0)
    check(bgn_ce_fwd(logits.data_ptr(), targets.data_ptr<int64_t>(), loss.data_ptr<float>(), lse.data_ptr<float>(),
                     logits.size(0), (int)logits.size(1), ignore_index, type_code(logits), stream()), "ce_fwd");
  return {loss, lse};
}

std::vector<at::Tensor> ce_bwd_bwd(at::Tensor c, at::Tensor logits, at::Tensor targets, at::Tensor lse, at::Tensor dloss,
                                   int64_t ignore_index) {
  CHECK_CUDA_CONTIG(c); CHECK_CUDA_CONTIG(logits); CHECK_CUDA_CONTIG(targets); CHECK_CUDA_CONTIG(lse); CHECK_CUDA_CONTIG(dloss);
  TORCH_CHECK(logits.dim() == 2 && c.sizes() == logits.sizes() && c.scalar_type() == logits.scalar_type() &&
              targets.scalar_type() == at::kLong && lse.scalar_type() == at::kFloat && dloss.scalar_type() == at::kFloat);
  c10::cuda::CUDAGuard guard(logits.device());
  auto d_logits = at::empty_like(logits);
  auto d_dloss = at::empty({logits.size(0)}, logits.options().dtype(at::kFloat));
  check(bgn_ce_bwd_bwd(c.data_ptr(), logits.data_ptr(), targets.data_ptr<int64_t>(), lse.data_ptr<float>(),
                       dloss.data_ptr<float>(), d_logits.data_ptr(), d_dloss.data_ptr<float>(), logits.size(0),
                       (int)logits.size(1), ignore_index, type_code(logits), stream()), "ce_bwd_bwd");
  return {d_logits, d_dloss};
}

at::Tensor ce_bwd(at::Tensor logits, at::Tensor targets, at::Tensor lse, at::Tensor dloss, int64_t ignore_index) {
  CHECK_CUDA_CONTIG(logits); CHECK_CUDA_CONTIG(dloss);
  c10::cuda::CUDAGuard guard(logits.device());
  auto dlogits = at::empty_like(logits);
  if (logits.size(0) > 0)
    check(bgn_ce_bwd(logits.data_ptr(), targets.data_ptr<int64_t>(), lse.data_ptr<float>(), dloss.data_ptr<float>(),
                     dlogits.data_ptr(), logits.size(0), (int)logits.size(1), ignore_index, type_code(logits),
                     stream()), "ce_bwd");
  return dlogits;
}

at::Tensor proj_right(at::Tensor a, at::Tensor p) {
  CHECK_CUDA_CONTIG(a); CHECK_CUDA_CONTIG(p);
  TORCH_CHECK(a.dim() == 2 && p.dim() == 2 && p.size(0) == 16 && p.size(1) == a.size(1) &&
              p.scalar_type() == a.scalar_type(), "proj_right: a [T, K], p [16, K] of the same 16-bit dtype");
  c10::cuda::CUDAGuard guard(a.device());
  auto out = at::empty({a.size(0), 16}, a.options().dtype(at::kFloat));
  check(bgn_proj_right(a.data_ptr(), p.data_ptr(), out.data_ptr<float>(), a.size(0), (int)a.size(1), fmt16(a),
                       status_ptr(a), stream()), "proj_right");
  return out;
}

void proj_left_outer(at::Tensor g, at::Tensor p, at::Tensor a_proj, at::Tensor acc, int64_t col_off) {
  CHECK_CUDA_CONTIG(g); CHECK_CUDA_CONTIG(p); CHECK_CUDA_CONTIG(a_proj);
  TORCH_CHECK(g.dim() == 3 && p.size(0) == 16 && p.size(1) == g.size(2) && p.scalar_type() == g.scalar_type());
  TORCH_CHECK(a_proj.scalar_type() == at::kFloat && a_proj.numel() == g.size(0) * g.size(1) * 16);
  TORCH_CHECK(acc.scalar_type() == at::kFloat && acc.dim() == 2 && acc.size(0) == g.size(0) && acc.stride(1) == 1 &&
              col_off + 256 <= acc.size(1));
  c10::cuda::CUDAGuard guard(g.device());
  check(bgn_proj_left_outer(g.data_ptr(), p.data_ptr(), a_proj.data_ptr<float>(), acc.data_ptr<float>(),
                            (int)g.size(0), (int)g.size(1), (int)g.size(2), acc.stride(0), col_off, fmt16(g),
                            status_ptr(g), stream()), "proj_left_outer");
}

at::Tensor tn_gemm(at::Tensor a, at::Tensor b) {
  CHECK_CUDA_CONTIG(a); CHECK_CUDA_CONTIG(b);
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.size(1) == b.size(1) && a.scalar_type() == b.scalar_type());
  c10::cuda::CUDAGuard guard(a.device());
  auto c = at::empty({a.size(0), b.size(0)}, a.options().dtype(at::kFloat));
  check(bgn_tn_gemm(a.data_ptr(), b.data_ptr(), c.data_ptr<float>(), a.size(0), (int)b.size(0), (int)a.size(1),
                    c.stride(0), fmt16(a), status_ptr(a), stream()), "tn_gemm");
  return c;
}

at::Tensor tn_gemm_gathered(at::Tensor a, std::vector<int64_t> b_ptrs, int64_t n_per_rank) {
  // b_ptrs: device addresses of every rank's [n_per_rank, K] block of B, same dtype as a.
  CHECK_CUDA_CONTIG(a);
  const int world = (int)b_ptrs.size();
  TORCH_CHECK(a.dim() == 2 && world >= 1 && world <= 8);
  c10::cuda::CUDAGuard guard(a.device());
  auto c = at::empty({a.size(0), world * n_per_rank}, a.options().dtype(at::kFloat));
  const void* b[8];
  for (int r = 0; r < world; ++r) b[r] = reinterpret_cast<const void*>(b_ptrs[r]);
  check(bgn_tn_gemm_gathered(a.data_ptr(), b, world, c.data_ptr<float>(), a.size(0), (int)n_per_rank, (int)a.size(1),
                             c.stride(0), fmt16(a), status_ptr(a), stream()), "tn_gemm_gathered");
  return c;
}

void finalize_rows(at::Tensor acc, at::Tensor out, c10::optional<at::Tensor> row_index, double lo, double hi,
                   bool unit_norm) {
  TORCH_CHECK(acc.is_cuda() && acc.is_contiguous() && acc.scalar_type() == at::kFloat && acc.dim() == 2);
  TORCH_CHECK(out.dim() == 2 && out.stride(1) == 1 && out.size(1) >= acc.size(1));
  // `out` may be device memory or page-locked host memory mapped into the device address space.
  c10::cuda::CUDAGuard guard(acc.device());
  const long* idx = nullptr;
  if (row_index.has_value()) {
    TORCH_CHECK(row_index->is_cuda() && row_index->scalar_type() == at::kLong && row_index->numel() == acc.size(0));
    idx = row_index->data_ptr<int64_t>();
  }
  check(bgn_finalize_rows(acc.data_ptr<float>(), out.data_ptr(), idx, (int)acc.size(0), acc.size(1), out.stride(0),
                          (float)lo, (float)hi, unit_norm, type_code(out), stream()), "finalize_rows");
}

void adamw_step(at::Tensor p, at::Tensor m, at::Tensor v, at::Tensor g, c10::optional<at::Tensor> p_model, double lr,
                double b1, double b2, double eps, double eps_root, double wd, int64_t step, double grad_scale) {
  CHECK_CUDA_CONTIG(p); CHECK_CUDA_CONTIG(m); CHECK_CUDA_CONTIG(v); CHECK_CUDA_CONTIG(g);
  TORCH_CHECK(p.scalar_type() == at::kFloat && m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat);
  c10::cuda::CUDAGuard guard(p.device());
  const float bc1 = 1.f - (float)std::pow(b1, (double)step), bc2 = 1.f - (float)std::pow(b2, (double)step);
  void* pm = nullptr;
  int mt = 2;
  if (p_model.has_value()) {
    pm = p_model->data_ptr();
    mt = type_code(*p_model);
  }
  check(bgn_adamw_step(p.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), g.data_ptr(), pm, p.numel(),
                       (float)lr, (float)b1, (float)b2, (float)eps, (float)eps_root, (float)wd, bc1, bc2,
                       (float)grad_scale, type_code(g), mt, stream()), "adamw_step");
}

// Device copy of a pointer table for the multi-tensor kernels: six 8-byte words per entry.
// The host side is pinned so that the copy is asynchronous; the caching host allocator keeps
// the pinned block alive until the copy has run.
static at::Tensor upload_table(const std::vector<std::array<int64_t, 6>>& rows, const at::Device& device) {
  auto host = at::empty({(int64_t)rows.size(), 6}, at::TensorOptions().dtype(at::kLong).pinned_memory(true));
  std::memcpy(host.data_ptr<int64_t>(), rows.data(), rows.size() * sizeof(rows[0]));
  return host.to(device, /*non_blocking=*/true);
}

void adamw_multi(std::vector<at::Tensor> ps, std::vector<at::Tensor> ms, std::vector<at::Tensor> vs,
                 std::vector<at::Tensor> gs, double lr, double b1, double b2, double eps, double eps_root, double wd,
                 int64_t step, double grad_scale, c10::optional<at::Tensor> coef) {
  const size_t n = ps.size();
  TORCH_CHECK(n > 0 && ms.size() == n && vs.size() == n && gs.size() == n, "adamw_multi: list lengths differ");
  std::vector<std::array<int64_t, 6>> rows(n);
  int64_t max_n = 0;
  for (size_t i = 0; i < n; ++i) {
    CHECK_CUDA_CONTIG(ps[i]); CHECK_CUDA_CONTIG(ms[i]); CHECK_CUDA_CONTIG(vs[i]); CHECK_CUDA_CONTIG(gs[i]);
    TORCH_CHECK(ps[i].scalar_type() == ps[0].scalar_type() && gs[i].scalar_type() == ps[0].scalar_type(),
                "adamw_multi: parameters and gradients must share one element type");
    TORCH_CHECK(ms[i].scalar_type() == at::kFloat && vs[i].scalar_type() == at::kFloat, "adamw_multi: fp32 moments");
    TORCH_CHECK(ms[i].numel() == ps[i].numel() && vs[i].numel() == ps[i].numel() && gs[i].numel() == ps[i].numel());
    TORCH_CHECK(ps[i].device() == ps[0].device());
    rows[i] = {(int64_t)ps[i].data_ptr(), (int64_t)ms[i].data_ptr(), (int64_t)vs[i].data_ptr(),
               (int64_t)gs[i].data_ptr(), ps[i].numel(), 0};
    max_n = std::max<int64_t>(max_n, ps[i].numel());
  }
  c10::cuda::CUDAGuard guard(ps[0].device());
  const float* cf = nullptr;
  if (coef.has_value()) {
    TORCH_CHECK(coef->is_cuda() && coef->scalar_type() == at::kFloat && coef->numel() >= 1);
    cf = coef->data_ptr<float>();
  }
  auto table = upload_table(rows, ps[0].device());
  const float bc1 = 1.f - (float)std::pow(b1, (double)step), bc2 = 1.f - (float)std::pow(b2, (double)step);
  check(bgn_adamw_multi(table.data_ptr(), (int)n, max_n, (float)lr, (float)b1, (float)b2, (float)eps, (float)eps_root,
                        (float)wd, bc1, bc2, (float)grad_scale, cf, type_code(ps[0]), stream()), "adamw_multi");
}

static at::Tensor upload_table12(const std::vector<std::array<int64_t, 12>>& rows, const at::Device& device) {
  auto host = at::empty({(int64_t)rows.size(), 12}, at::TensorOptions().dtype(at::kLong).pinned_memory(true));
  std::memcpy(host.data_ptr<int64_t>(), rows.data(), rows.size() * sizeof(rows[0]));
  return host.to(device, /*non_blocking=*/true);
}

static void check_moments(const at::Tensor& p, const at::Tensor& t) {
  CHECK_CUDA_CONTIG(t);
  TORCH_CHECK(t.scalar_type() == at::kFloat && t.numel() == p.numel() && t.device() == p.device(),
              "adamw_traced: moments are fp32 tensors of the parameter's size");
}

// Out-of-place AdamW step for graphs: returns (new params, new mu, new nu), one launch.
std::vector<std::vector<at::Tensor>> adamw_traced_fwd(std::vector<at::Tensor> ps, std::vector<at::Tensor> gs,
                                                      std::vector<at::Tensor> ms, std::vector<at::Tensor> vs, double lr,
                                                      double b1, double b2, double eps, double eps_root, double wd,
                                                      int64_t step) {
  const size_t n = ps.size();
  TORCH_CHECK(n > 0 && gs.size() == n && ms.size() == n && vs.size() == n, "adamw_traced: list lengths differ");
  c10::cuda::CUDAGuard guard(ps[0].device());
  std::vector<at::Tensor> po(n), mo(n), vo(n);
  std::vector<std::array<int64_t, 12>> rows(n);
  int64_t max_n = 0;
  for (size_t i = 0; i < n; ++i) {
    CHECK_CUDA_CONTIG(ps[i]); CHECK_CUDA_CONTIG(gs[i]);
    TORCH_CHECK(ps[i].scalar_type() == ps[0].scalar_type() && gs[i].scalar_type() == ps[0].scalar_type() &&
                gs[i].numel() == ps[i].numel() && ps[i].device() == ps[0].device());
    check_moments(ps[i], ms[i]); check_moments(ps[i], vs[i]);
    po[i] = at::empty_like(ps[i]); mo[i] = at::empty_like(ms[i]); vo[i] = at::empty_like(vs[i]);
    rows[i] = {(int64_t)ps[i].data_ptr(), (int64_t)gs[i].data_ptr(), (int64_t)ms[i].data_ptr(), (int64_t)vs[i].data_ptr(),
               (int64_t)po[i].data_ptr(), (int64_t)mo[i].data_ptr(), (int64_t)vo[i].data_ptr(), 0, 0, 0, ps[i].numel(), 0};
    max_n = std::max<int64_t>(max_n, ps[i].numel());
  }
  auto table = upload_table12(rows, ps[0].device());
  const float bc1 = 1.f - (float)std::pow(b1, (double)step), bc2 = 1.f - (float)std::pow(b2, (double)step);
  check(bgn_adamw_traced(table.data_ptr(), (int)n, max_n, 0, (float)lr, (float)b1, (float)b2, (float)eps, (float)eps_root,
                         (float)wd, bc1, bc2, type_code(ps[0]), stream()), "adamw_traced_fwd");
  return {po, mo, vo};
}

// Vector-Jacobian product of that step: cotangents (cp, cm, cv; undefined tensors count as zero)
// of the outputs -> cotangents (dp, dg, dm, dv) of the inputs.
std::vector<std::vector<at::Tensor>> adamw_traced_bwd(std::vector<at::Tensor> gs, std::vector<at::Tensor> ms,
                                                      std::vector<at::Tensor> vs,
                                                      std::vector<c10::optional<at::Tensor>> cps,
                                                      std::vector<c10::optional<at::Tensor>> cms,
                                                      std::vector<c10::optional<at::Tensor>> cvs, double lr, double b1,
                                                      double b2, double eps, double eps_root, double wd, int64_t step) {
  const size_t n = gs.size();
  TORCH_CHECK(n > 0 && ms.size() == n && vs.size() == n && cps.size() == n && cms.size() == n && cvs.size() == n);
  c10::cuda::CUDAGuard guard(gs[0].device());
  std::vector<at::Tensor> dp(n), dg(n), dm(n), dv(n), keep;
  std::vector<std::array<int64_t, 12>> rows(n);
  int64_t max_n = 0;
  auto ptr_of = [&](const c10::optional<at::Tensor>& t, const at::Tensor& like, at::ScalarType st) -> int64_t {
    if (!t.has_value() || !t->defined()) return 0;
    at::Tensor c = t->contiguous();
    TORCH_CHECK(c.is_cuda() && c.scalar_type() == st && c.numel() == like.numel(), "adamw_traced: bad cotangent");
    keep.push_back(c);
    return (int64_t)c.data_ptr();
  };
  for (size_t i = 0; i < n; ++i) {
    CHECK_CUDA_CONTIG(gs[i]);
    TORCH_CHECK(gs[i].scalar_type() == gs[0].scalar_type() && gs[i].device() == gs[0].device());
    check_moments(gs[i], ms[i]); check_moments(gs[i], vs[i]);
    dp[i] = at::empty_like(gs[i]); dg[i] = at::empty_like(gs[i]); dm[i] = at::empty_like(ms[i]); dv[i] = at::empty_like(vs[i]);
    rows[i] = {(int64_t)gs[i].data_ptr(), (int64_t)ms[i].data_ptr(), (int64_t)vs[i].data_ptr(),
               ptr_of(cps[i], gs[i], gs[0].scalar_type()), ptr_of(cms[i], gs[i], at::kFloat), ptr_of(cvs[i], gs[i], at::kFloat),
               (int64_t)dp[i].data_ptr(), (int64_t)dg[i].data_ptr(), (int64_t)dm[i].data_ptr(), (int64_t)dv[i].data_ptr(),
               gs[i].numel(), 0};
    max_n = std::max<int64_t>(max_n, gs[i].numel());
  }
  auto table = upload_table12(rows, gs[0].device());
  const float bc1 = 1.f - (float)std::pow(b1, (double)step), bc2 = 1.f - (float)std::pow(b2, (double)step);
  check(bgn_adamw_traced(table.data_ptr(), (int)n, max_n, 1, (float)lr, (float)b1, (float)b2, (float)eps, (float)eps_root,
                         (float)wd, bc1, bc2, type_code(gs[0]), stream()), "adamw_traced_bwd");
  return {dp, dg, dm, dv};
}

// out[0] (+)= sum of squares of every tensor in `xs`; with max_norm > 0 also
// out[1] = min(1, max_norm / (sqrt(out[0]) + 1e-6)).  `out` is fp32 with at least two elements.
void multi_sumsq(std::vector<at::Tensor> xs, at::Tensor out, bool accumulate, double max_norm) {
  const size_t n = xs.size();
  TORCH_CHECK(n > 0 && out.is_cuda() && out.scalar_type() == at::kFloat && out.numel() >= 2 && out.is_contiguous());
  std::vector<std::array<int64_t, 6>> rows(n);
  int64_t max_n = 0;
  for (size_t i = 0; i < n; ++i) {
    CHECK_CUDA_CONTIG(xs[i]);
    TORCH_CHECK(xs[i].scalar_type() == xs[0].scalar_type() && xs[i].device() == out.device());
    rows[i] = {0, 0, 0, (int64_t)xs[i].data_ptr(), xs[i].numel(), 0};
    max_n = std::max<int64_t>(max_n, xs[i].numel());
  }
  c10::cuda::CUDAGuard guard(out.device());
  auto table = upload_table(rows, out.device());
  auto partials = at::empty({(int64_t)n * bgn_multi_sumsq_blocks()}, out.options());
  check(bgn_multi_sumsq(table.data_ptr(), (int)n, max_n, partials.data_ptr<float>(), out.data_ptr<float>(), accumulate,
                        (float)max_norm, type_code(xs[0]), stream()), "multi_sumsq");
}

void row_sumsq(at::Tensor x, at::Tensor out) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.stride(1) == 1 && out.scalar_type() == at::kFloat &&
              out.numel() == x.size(0));
  c10::cuda::CUDAGuard guard(x.device());
  check(bgn_row_sumsq(x.data_ptr(), out.data_ptr<float>(), x.size(0), x.size(1), x.stride(0), type_code(x), stream()),
        "row_sumsq");
}

void cov_syrk(at::Tensor x, std::vector<int64_t> dst_ptrs, std::vector<int64_t> row_start,
              c10::optional<at::Tensor> local, bool full, int64_t num_rows, bool local_upper) {
  // x: [T, D] 16-bit; dst_ptrs: device addresses (this GPU's or peer-mapped) of every rank's
  // fp32 row shard; row_start: world + 1 row boundaries.
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.is_contiguous());
  const int world = (int)dst_ptrs.size();
  TORCH_CHECK(world >= 1 && world <= 8 && (int)row_start.size() == world + 1);
  c10::cuda::CUDAGuard guard(x.device());
  float* dst[8];
  int rs[9];
  for (int r = 0; r < world; ++r) dst[r] = reinterpret_cast<float*>(dst_ptrs[r]);
  for (int r = 0; r <= world; ++r) rs[r] = (int)row_start[r];
  const float* loc = nullptr;
  if (local.has_value()) {
    TORCH_CHECK(local->is_cuda() && local->is_contiguous() && local->scalar_type() == at::kFloat &&
                local->size(0) == x.size(1) && local->size(1) == x.size(1));
    loc = local->data_ptr<float>();
  }
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  // num_rows < 0: use every row of x; num_rows == 0: only push `local`.
  const long T = num_rows < 0 ? x.size(0) : std::min<int64_t>(num_rows, x.size(0));
  check(bgn_cov_syrk(x.data_ptr(), T, (int)x.size(1), fmt16(x), dst, rs, world, loc, full ? 1 : 0, local_upper ? 1 : 0, sms,
                     status_ptr(x), stream()), "cov_syrk");
}


// Persistent tcgen05 GEMM.  a: [M, K] (or [K, M] when a_mn), b: [N, K] (or [K, N] when b_mn); a
// leading batch dimension on both selects the batched form.  Last dimensions contiguous.
std::vector<at::Tensor> gemm(at::Tensor a, at::Tensor b, bool a_mn, bool b_mn, c10::optional<at::Tensor> out,
                             bool out_f32, c10::optional<at::Tensor> bias, bool accumulate,
                             c10::optional<at::Tensor> aux_p, int64_t cta_group, bool sq_accumulate,
                             int64_t wait_cycles, c10::optional<at::Tensor> status, int64_t panel, c10::optional<at::Tensor> trace, bool no_tma_store, bool wide,
                             std::vector<int64_t> a_peer_ptrs, std::vector<int64_t> d_peer_ptrs, int64_t d_rows_per_rank,
                             int64_t d_slot, c10::optional<at::Tensor> gather_done, int64_t gather_rank) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.scalar_type() == b.scalar_type(), "gemm: CUDA operands of one dtype");
  TORCH_CHECK((a.dim() == 2 || a.dim() == 3) && a.dim() == b.dim() && a.stride(-1) == 1 && b.stride(-1) == 1,
              "gemm: 2-D or 3-D operands with contiguous last dimension");
  c10::cuda::CUDAGuard guard(a.device());
  const int fmt = fmt16(a);
  const bool batched = a.dim() == 3;
  const int64_t nb = batched ? a.size(0) : 1;
  if (batched) { TORCH_CHECK(b.size(0) == nb, "gemm: batch sizes differ"); }
  // With a_peer_ptrs, `a` is this rank's [rows, K] block (shape, dtype and row stride of every
  // rank's block) and the product runs over the concatenation of all ranks' blocks.
  const int64_t gather_world = (int64_t)a_peer_ptrs.size(), scatter_world = (int64_t)d_peer_ptrs.size();
  TORCH_CHECK(gather_world <= 8 && scatter_world <= 8, "gemm: at most 8 peers");
  if (gather_world || scatter_world) {
    TORCH_CHECK(!batched && !a_mn && !out_f32 && !accumulate && !sq_accumulate, "gemm: peer forms take a K-major 2-D A and write 16-bit outputs");
  }
  // With gather_done, `a` is the local [M, K] buffer that the kernel completes from the peers'
  // blocks while it computes (gather-with-copy); otherwise `a` is this rank's block.
  const bool gather_copy = gather_world > 0 && gather_done.has_value();
  const int64_t M = (a_mn ? a.size(-1) : a.size(-2)) * (gather_world && !gather_copy ? gather_world : 1),
                K = a_mn ? a.size(-2) : a.size(-1);
  const int64_t N = b_mn ? b.size(-1) : b.size(-2), Kb = b_mn ? b.size(-2) : b.size(-1);
  TORCH_CHECK(K == Kb, "gemm: reduction lengths differ (", K, " vs ", Kb, ")");
  const auto out_type = out_f32 ? at::kFloat : a.scalar_type();
  at::Tensor d;
  if (out.has_value()) {
    d = *out;
    TORCH_CHECK(d.is_cuda() && d.scalar_type() == out_type && d.stride(-1) == 1, "gemm: bad output tensor");
    if (sq_accumulate) {
      TORCH_CHECK(d.dim() == 2 && d.size(0) == M && d.size(1) == N, "gemm: sq_accumulate output must be [M, N]");
    } else {
      TORCH_CHECK(d.dim() == a.dim() && d.size(-2) == M && d.size(-1) == N && (!batched || d.size(0) == nb),
                  "gemm: output shape mismatch");
    }
  } else if (scatter_world) {
    d = at::empty({0, N}, a.options().dtype(out_type));  // results go to the peers' buffers
  } else {
    TORCH_CHECK(!accumulate && !sq_accumulate, "gemm: accumulation needs an output tensor");
    d = batched ? at::empty({nb, M, N}, a.options().dtype(out_type)) : at::empty({M, N}, a.options().dtype(out_type));
  }
  BgnGemmArgs g = {};
  g.a = a.data_ptr(); g.b = b.data_ptr(); g.d = d.data_ptr();
  g.M = (int)M; g.N = (int)N; g.K = (int)K;
  g.lda = a.stride(-2); g.ldb = b.stride(-2); g.ldd = scatter_world ? N : d.stride(-2);
  if (gather_world) {
    g.gather_world = (int)gather_world; g.gather_rows = (int)(gather_copy ? a.size(0) / gather_world : a.size(0));
    if (gather_copy) {
      TORCH_CHECK(gather_done->is_cuda() && gather_done->scalar_type() == at::kInt && gather_done->numel() >= gather_world &&
                  a.is_contiguous() && a.size(0) % gather_world == 0, "gemm: gather_done is an int32 tensor of >= world entries; A contiguous");
      gather_done->zero_();
      g.gather_copy = 1; g.gather_rank = (int)gather_rank; g.gather_done = gather_done->data_ptr<int>();
    }
    for (int64_t r = 0; r < gather_world; ++r) g.a_peers[r] = reinterpret_cast<const void*>(a_peer_ptrs[r]);
  }
  if (scatter_world) {
    TORCH_CHECK(d_rows_per_rank > 0 && d_rows_per_rank * scatter_world >= M && d_slot >= 0 && d_slot < scatter_world,
                "gemm: scatter needs rows_per_rank * world >= M and a slot below world");
    g.scatter_world = (int)scatter_world; g.scatter_rows = (int)d_rows_per_rank; g.scatter_slot = (int)d_slot;
    for (int64_t r = 0; r < scatter_world; ++r) g.d_peers[r] = reinterpret_cast<void*>(d_peer_ptrs[r]);
  }
  g.a_mn = a_mn; g.b_mn = b_mn; g.fmt = fmt; g.out_f32 = out_f32;
  at::Tensor bias_c;
  if (bias.has_value()) {
    bias_c = bias->contiguous();
    TORCH_CHECK(bias_c.numel() == N && (bias_c.scalar_type() == a.scalar_type() || bias_c.scalar_type() == at::kFloat));
    g.bias = bias_c.data_ptr();
    g.bias_f32 = bias_c.scalar_type() == at::kFloat;
  }
  g.accumulate = accumulate;
  at::Tensor aux_out, aux_c;
  if (aux_p.has_value()) {
    aux_c = aux_p->contiguous();
    TORCH_CHECK(aux_c.dim() == 2 && aux_c.size(1) == K && aux_c.scalar_type() == a.scalar_type() &&
                aux_c.size(0) % 16 == 0 && aux_c.size(0) <= 64, "gemm: aux operand must be [16..64, K] of the input dtype");
    aux_out = at::empty({nb * M, aux_c.size(0)}, a.options().dtype(at::kFloat));
    g.aux_p = aux_c.data_ptr(); g.aux_n = (int)aux_c.size(0); g.aux_out = aux_out.data_ptr<float>();
  }
  g.batch = (int)nb;
  g.a_batch_stride = batched ? a.stride(0) : 0;
  g.b_batch_stride = batched ? b.stride(0) : 0;
  g.d_batch_stride = (batched && !sq_accumulate) ? d.stride(0) : 0;
  g.sq_accumulate = sq_accumulate;
  g.cta_group = (int)cta_group;
  g.sm_count = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  g.wait_cycles = wait_cycles;
  g.panel = (int)panel;
  g.no_tma_store = no_tma_store;
  g.wide = wide;
  if (trace.has_value()) {
    TORCH_CHECK(trace->is_cuda() && trace->scalar_type() == at::kLong && trace->is_contiguous());
    g.trace = reinterpret_cast<long long*>(trace->data_ptr<int64_t>());
  }
  int* st = status.has_value() ? status->data_ptr<int>() : status_ptr(a);
  check(bgn_gemm(&g, st, stream()), "gemm");
  return {d, aux_out};
}

// ---- peer-memory helpers -------------------------------------------------------------------

void peer_barrier(std::vector<int64_t> flag_ptrs, int64_t rank, int64_t epoch, int64_t budget_cycles,
                  c10::optional<at::Tensor> status) {
  const int64_t world = (int64_t)flag_ptrs.size();
  TORCH_CHECK(world >= 1 && world <= kPeerMax && rank >= 0 && rank < world, "peer_barrier: 1..8 ranks");
  PeerFlagTable table = {};
  for (int64_t r = 0; r < world; ++r) table.flags[r] = reinterpret_cast<unsigned*>(flag_ptrs[r]);
  int* st = status.has_value() ? status->data_ptr<int>() : status_ptr_current();
  check(bgn_peer_barrier(&table, (int)rank, (int)world, (unsigned)epoch, budget_cycles, st, stream()), "peer_barrier");
}

// out = residual + sum over slots; `slots` is a [world, rows, cols] view of this rank's slot region.
at::Tensor slot_reduce(at::Tensor slots, c10::optional<at::Tensor> residual, c10::optional<at::Tensor> out) {
  CHECK_CUDA_CONTIG(slots);
  TORCH_CHECK(slots.dim() == 3, "slot_reduce: [world, rows, cols]");
  c10::cuda::CUDAGuard guard(slots.device());
  at::Tensor o = out.has_value() ? *out : at::empty({slots.size(1), slots.size(2)}, slots.options());
  CHECK_CUDA_CONTIG(o);
  TORCH_CHECK(o.numel() == slots.size(1) * slots.size(2) && o.scalar_type() == slots.scalar_type());
  const void* res = nullptr;
  if (residual.has_value()) {
    CHECK_CUDA_CONTIG((*residual));
    TORCH_CHECK(residual->numel() == o.numel() && residual->scalar_type() == slots.scalar_type());
    res = residual->data_ptr();
  }
  check(bgn_slot_reduce(slots.data_ptr(), (int)slots.size(0), o.numel(), res, o.data_ptr(), fmt16(slots), stream()),
        "slot_reduce");
  return o;
}

// Row block o of src [world * rows, cols] goes to peer o's slot region at slot `slot`.
void peer_push(at::Tensor src, std::vector<int64_t> dst_ptrs, int64_t slot) {
  TORCH_CHECK(src.is_cuda() && src.dim() == 2 && src.stride(1) == 1 && src.element_size() == 2, "peer_push: 16-bit 2-D source");
  const int64_t world = (int64_t)dst_ptrs.size();
  TORCH_CHECK(world >= 1 && world <= kPeerMax && src.size(0) % world == 0 && slot >= 0 && slot < world);
  c10::cuda::CUDAGuard guard(src.device());
  PeerPtrTable table = {};
  for (int64_t r = 0; r < world; ++r) table.ptrs[r] = reinterpret_cast<void*>(dst_ptrs[r]);
  check(bgn_peer_push(src.data_ptr(), src.stride(0), &table, (int)slot, src.size(0) / world, src.size(1), (int)world,
                      stream()), "peer_push");
}

void proj_contract(at::Tensor g_proj, at::Tensor a_proj, at::Tensor acc, int64_t n, int64_t s, int64_t p, int64_t col_off) {
  CHECK_CUDA_CONTIG(g_proj); CHECK_CUDA_CONTIG(a_proj);
  TORCH_CHECK(g_proj.scalar_type() == at::kFloat && a_proj.scalar_type() == at::kFloat && g_proj.dim() == 2 &&
              g_proj.sizes() == a_proj.sizes() && g_proj.size(0) == n * s && g_proj.size(1) >= p);
  TORCH_CHECK(acc.is_cuda() && acc.scalar_type() == at::kFloat && acc.dim() == 2 && acc.stride(1) == 1 &&
              acc.size(0) >= n && col_off + p * p <= acc.size(1));
  c10::cuda::CUDAGuard guard(acc.device());
  const int splits = bgn_proj_contract_splits((int)s);
  auto partials = at::empty({n * splits * p * p}, acc.options());
  auto counters = contract_counters(acc.get_device(), n);
  check(bgn_proj_contract(g_proj.data_ptr<float>(), a_proj.data_ptr<float>(), acc.data_ptr<float>(),
                          partials.data_ptr<float>(), counters.data_ptr<int>(), (int)n, (int)s, (int)p,
                          (int)g_proj.size(1), acc.stride(0), col_off, stream()), "proj_contract");
}

void proj_token_rows(at::Tensor g_proj, at::Tensor a_proj, at::Tensor token_index, at::Tensor out, int64_t p,
                     int64_t col_off) {
  CHECK_CUDA_CONTIG(g_proj); CHECK_CUDA_CONTIG(a_proj); CHECK_CUDA_CONTIG(token_index);
  TORCH_CHECK(g_proj.scalar_type() == at::kFloat && g_proj.sizes() == a_proj.sizes() && g_proj.size(1) >= p &&
              token_index.scalar_type() == at::kLong);
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kFloat && out.dim() == 2 && out.stride(1) == 1 &&
              out.size(0) >= token_index.numel() && col_off + p * p <= out.size(1));
  c10::cuda::CUDAGuard guard(out.device());
  check(bgn_proj_token_rows(g_proj.data_ptr<float>(), a_proj.data_ptr<float>(), token_index.data_ptr<int64_t>(),
                            out.data_ptr<float>(), token_index.numel(), (int)p, (int)g_proj.size(1), out.stride(0),
                            col_off, stream()), "proj_token_rows");
}

at::Tensor wait_probe(int64_t budget_cycles, at::Tensor status) {
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == at::kInt && status.numel() == 1);
  c10::cuda::CUDAGuard guard(status.device());
  auto waited = at::zeros({1}, status.options().dtype(at::kLong));
  check(bgn_wait_probe(budget_cycles, status.data_ptr<int>(), reinterpret_cast<long long*>(waited.data_ptr<int64_t>()),
                       stream()), "wait_probe");
  return waited;
}

at::Tensor kernel_status(int64_t device) { return status_tensor((int)device); }

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("layernorm_fwd", &layernorm_fwd);
  m.def("layernorm_bwd", &layernorm_bwd);
  m.def("layernorm_bwd_bwd", &layernorm_bwd_bwd);
  m.def("rmsnorm_bwd_bwd", &rmsnorm_bwd_bwd);
  m.def("swiglu_bwd_bwd", &swiglu_bwd_bwd);
  m.def("rotary", &rotary);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("gelu_fwd", &gelu_fwd);
  m.def("gelu_bwd", &gelu_bwd);
  m.def("gelu_bwd_bwd", &gelu_bwd_bwd);
  m.def("softmax_bwd_bwd", &softmax_bwd_bwd);
  m.def("ce_fwd", &ce_fwd);
  m.def("ce_bwd", &ce_bwd);
  m.def("ce_bwd_bwd", &ce_bwd_bwd);
  m.def("proj_right", &proj_right);
  m.def("proj_left_outer", &proj_left_outer);
  m.def("tn_gemm", &tn_gemm);
  m.def("tn_gemm_gathered", &tn_gemm_gathered);
  m.def("finalize_rows", &finalize_rows);
  m.def("adamw_step", &adamw_step);
  m.def("adamw_multi", &adamw_multi, py::arg("params"), py::arg("mu"), py::arg("nu"), py::arg("grads"), py::arg("lr"),
        py::arg("b1"), py::arg("b2"), py::arg("eps"), py::arg("eps_root"), py::arg("weight_decay"), py::arg("step"),
        py::arg("grad_scale") = 1.0, py::arg("coef") = py::none());
  m.def("adamw_traced_fwd", &adamw_traced_fwd);
  m.def("adamw_traced_bwd", &adamw_traced_bwd);
  m.def("multi_sumsq", &multi_sumsq, py::arg("tensors"), py::arg("out"), py::arg("accumulate") = false,
        py::arg("max_norm") = 0.0);
  m.def("row_sumsq", &row_sumsq);
  m.def("peer_barrier", &peer_barrier, py::arg("flag_ptrs"), py::arg("rank"), py::arg("epoch"),
        py::arg("budget_cycles") = 0, py::arg("status") = py::none());
  m.def("slot_reduce", &slot_reduce, py::arg("slots"), py::arg("residual") = py::none(), py::arg("out") = py::none());
  m.def("peer_push", &peer_push, py::arg("src"), py::arg("dst_ptrs"), py::arg("slot"));
  m.def("cov_syrk", &cov_syrk, py::arg("x"), py::arg("dst_ptrs"), py::arg("row_start"), py::arg("local"),
        py::arg("full") = false, py::arg("num_rows") = -1, py::arg("local_upper") = false);
  m.def("gemm", &gemm, py::arg("a"), py::arg("b"), py::arg("a_mn") = false, py::arg("b_mn") = false,
        py::arg("out") = py::none(), py::arg("out_f32") = false, py::arg("bias") = py::none(),
        py::arg("accumulate") = false, py::arg("aux_p") = py::none(), py::arg("cta_group") = 2,
        py::arg("sq_accumulate") = false, py::arg("wait_cycles") = 0, py::arg("status") = py::none(), py::arg("panel") = 0, py::arg("trace") = py::none(), py::arg("no_tma_store") = false, py::arg("wide") = false, py::arg("a_peer_ptrs") = std::vector<int64_t>{}, py::arg("d_peer_ptrs") = std::vector<int64_t>{},
        py::arg("d_rows_per_rank") = 0, py::arg("d_slot") = 0, py::arg("gather_done") = py::none(), py::arg("gather_rank") = 0);
  m.def("proj_contract", &proj_contract);
  m.def("proj_token_rows", &proj_token_rows);
  m.def("wait_probe", &wait_probe);
  m.def("kernel_status", &kernel_status);
}
