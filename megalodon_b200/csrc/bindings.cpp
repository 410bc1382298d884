// Python bindings: tensor checks, output allocation and stream selection around
// the raw-pointer launchers in kernels.h.  The extension module is
// `megalodon_b200._C`.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAException.h>
#include <torch/extension.h>

#include <type_traits>

#include <optional>
#include <tuple>
#include <vector>

#include "kernels.h"

namespace {

using torch::Tensor;
using OptTensor = std::optional<Tensor>;

int dtype_code(const Tensor& t) {
  switch (t.scalar_type()) {
    case at::kFloat: return 0;
    case at::kBFloat16: return 1;
    case at::kHalf: return 2;
    default: TORCH_CHECK(false, "unsupported dtype ", t.scalar_type());
  }
  return -1;
}

void check_cuda_contig(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}

int weight_code(const Tensor& x, const Tensor& w) {
  TORCH_CHECK(w.scalar_type() == at::kFloat || w.scalar_type() == x.scalar_type(),
              "weight dtype must be fp32 or the activation dtype");
  return dtype_code(w);
}

cudaStream_t stream() { return at::cuda::getCurrentCUDAStream().stream(); }

const void* opt_ptr(const OptTensor& t) { return t.has_value() ? t->data_ptr() : nullptr; }

// ------------------------------------------------------------------ norms
std::tuple<Tensor, Tensor> rms_norm_fwd(const Tensor& x, const OptTensor& w, double w_off, double eps) {
  check_cuda_contig(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  const int D = x.size(-1);
  const long long M = x.numel() / D;
  TORCH_CHECK(D <= 8192, "rms_norm: last dim > 8192 is not supported");
  Tensor y = torch::empty_like(x);
  Tensor rstd = torch::empty({M}, x.options().dtype(at::kFloat));
  int wc = 0;
  if (w.has_value()) { check_cuda_contig(*w, "weight"); wc = weight_code(x, *w); }
  mb::rms_norm_fwd(x.data_ptr(), opt_ptr(w), (float)w_off, y.data_ptr(), rstd.data_ptr<float>(), M, D,
                   (float)eps, dtype_code(x), wc, stream());
  return {y, rstd};
}

std::tuple<Tensor, OptTensor> rms_norm_bwd(const Tensor& dy, const Tensor& x, const OptTensor& w, double w_off,
                                           const Tensor& rstd) {
  check_cuda_contig(dy, "dy");
  check_cuda_contig(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  const int D = x.size(-1);
  const long long M = x.numel() / D;
  Tensor dx = torch::empty_like(x);
  OptTensor dw;
  int wc = 0;
  if (w.has_value()) {
    dw = torch::zeros({D}, x.options().dtype(at::kFloat));
    wc = weight_code(x, *w);
  }
  Tensor ws;     // partial column sums of the wide-row kernel (caching allocator: no device call)
  if (w.has_value() && D > 1024) ws = torch::empty({(long long)mb::kColsumRows * D}, x.options().dtype(at::kFloat));
  mb::rms_norm_bwd(dy.data_ptr(), x.data_ptr(), opt_ptr(w), (float)w_off, rstd.data_ptr<float>(), dx.data_ptr(),
                   dw.has_value() ? dw->data_ptr<float>() : nullptr, M, D, dtype_code(x), wc, stream(),
                   ws.defined() ? ws.data_ptr<float>() : nullptr);
  return {dx, dw};
}

// fp32 column sums of a 16-bit matrix [M, N] (the bias gradient of a linear layer)
Tensor colsum(const Tensor& g) {
  check_cuda_contig(g, "g");
  TORCH_CHECK(g.dim() == 2, "colsum: a matrix");
  c10::cuda::CUDAGuard guard(g.device());
  const int N = g.size(1);
  const long long M = g.size(0);
  Tensor out = torch::zeros({N}, g.options().dtype(at::kFloat));
  Tensor ws = torch::empty({(long long)mb::kColsumRows * N}, g.options().dtype(at::kFloat));
  const bool done = g.element_size() == 2 &&
                    mb::colsum_16bit(g.data_ptr(), M, N, ws.data_ptr<float>(), out.data_ptr<float>(), dtype_code(g), stream());
  if (!done) return g.sum(0, /*keepdim=*/false, at::kFloat);
  return out;
}

std::tuple<Tensor, Tensor, Tensor> layer_norm_fwd(const Tensor& x, const OptTensor& w, const OptTensor& b,
                                                  double w_off, double eps) {
  check_cuda_contig(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  const int D = x.size(-1);
  const long long M = x.numel() / D;
  TORCH_CHECK(D <= 8192, "layer_norm: last dim > 8192 is not supported");
  Tensor y = torch::empty_like(x);
  Tensor mean = torch::empty({M}, x.options().dtype(at::kFloat));
  Tensor rstd = torch::empty({M}, x.options().dtype(at::kFloat));
  int wc = 0;
  if (w.has_value()) { wc = weight_code(x, *w); }
  if (b.has_value()) { TORCH_CHECK(w.has_value() && b->scalar_type() == w->scalar_type(), "bias/weight dtype"); }
  mb::layer_norm_fwd(x.data_ptr(), opt_ptr(w), opt_ptr(b), (float)w_off, y.data_ptr(), mean.data_ptr<float>(),
                     rstd.data_ptr<float>(), M, D, (float)eps, dtype_code(x), wc, stream());
  return {y, mean, rstd};
}

std::tuple<Tensor, OptTensor, OptTensor> layer_norm_bwd(const Tensor& dy, const Tensor& x, const OptTensor& w,
                                                        double w_off, const Tensor& mean, const Tensor& rstd) {
  check_cuda_contig(dy, "dy");
  check_cuda_contig(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  const int D = x.size(-1);
  const long long M = x.numel() / D;
  Tensor dx = torch::empty_like(x);
  OptTensor dw, db;
  int wc = 0;
  if (w.has_value()) {
    dw = torch::zeros({D}, x.options().dtype(at::kFloat));
    db = torch::zeros({D}, x.options().dtype(at::kFloat));
    wc = weight_code(x, *w);
  }
  Tensor ws;
  if (w.has_value() && D > 1024) ws = torch::empty({2LL * mb::kColsumRows * D}, x.options().dtype(at::kFloat));
  mb::layer_norm_bwd(dy.data_ptr(), x.data_ptr(), opt_ptr(w), (float)w_off, mean.data_ptr<float>(),
                     rstd.data_ptr<float>(), dx.data_ptr(), dw.has_value() ? dw->data_ptr<float>() : nullptr,
                     db.has_value() ? db->data_ptr<float>() : nullptr, M, D, dtype_code(x), wc, stream(),
                     ws.defined() ? ws.data_ptr<float>() : nullptr);
  return {dx, dw, db};
}

// ------------------------------------------------------------------ TimestepNorm
// returns y, count, mean, var, cummean, cumrstd
std::vector<Tensor> timestep_norm_fwd(const Tensor& x, const Tensor& prev_count, const Tensor& prev_mean,
                                      const Tensor& prev_var, const Tensor& gamma, double gamma_off,
                                      const Tensor& beta, const OptTensor& mask, int64_t G, double eps) {
  check_cuda_contig(x, "x");
  check_cuda_contig(prev_mean, "prev_mean");
  check_cuda_contig(prev_var, "prev_var");
  check_cuda_contig(gamma, "gamma");
  check_cuda_contig(beta, "beta");
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 3, "x must be [B, L, H]");
  const int B = x.size(0), L = x.size(1), H = x.size(2);
  TORCH_CHECK(H % G == 0 && H <= 8192, "bad feature/group sizes");
  TORCH_CHECK(prev_count.scalar_type() == at::kLong && prev_count.is_contiguous());
  TORCH_CHECK(prev_mean.scalar_type() == x.scalar_type() && prev_var.scalar_type() == x.scalar_type());
  TORCH_CHECK(gamma.scalar_type() == beta.scalar_type());
  if (mask.has_value()) TORCH_CHECK(mask->scalar_type() == at::kBool && mask->is_contiguous());
  auto f32 = x.options().dtype(at::kFloat);
  Tensor y = torch::empty_like(x);
  Tensor count = torch::empty_like(prev_count);
  Tensor mean = torch::empty_like(prev_mean);
  Tensor var = torch::empty_like(prev_var);
  Tensor cummean = torch::empty({B, L, G}, f32);
  Tensor cumrstd = torch::empty({B, L, G}, f32);
  Tensor gu = torch::empty({B, L, G}, f32);
  Tensor gv = torch::empty({B, L, G}, f32);
  Tensor seg = torch::empty({3LL * B * mb::tsn_num_segments(L) * G}, x.options().dtype(at::kDouble));
  mb::timestep_norm_fwd(x.data_ptr(), (const long long*)prev_count.data_ptr<int64_t>(), prev_mean.data_ptr(),
                        prev_var.data_ptr(), gamma.data_ptr(), (float)gamma_off, beta.data_ptr(),
                        mask.has_value() ? mask->data_ptr<bool>() : nullptr, y.data_ptr(),
                        (long long*)count.data_ptr<int64_t>(), mean.data_ptr(), var.data_ptr(),
                        cummean.data_ptr<float>(), cumrstd.data_ptr<float>(), gu.data_ptr<float>(),
                        gv.data_ptr<float>(), seg.data_ptr<double>(), B, L, H, (int)G, (float)eps, dtype_code(x),
                        weight_code(x, gamma), stream());
  return {y, count, mean, var, cummean, cumrstd};
}

// returns dx, dprev_mean, dprev_var, dgamma(fp32), dbeta(fp32)
std::vector<Tensor> timestep_norm_bwd(const Tensor& dy, const Tensor& dmean, const Tensor& dvar, const Tensor& x,
                                      const Tensor& prev_mean, const Tensor& count, const Tensor& cummean,
                                      const Tensor& cumrstd, const Tensor& gamma, double gamma_off,
                                      const OptTensor& mask, int64_t G) {
  check_cuda_contig(dy, "dy");
  check_cuda_contig(x, "x");
  check_cuda_contig(dmean, "dmean");
  check_cuda_contig(dvar, "dvar");
  c10::cuda::CUDAGuard guard(x.device());
  const int B = x.size(0), L = x.size(1), H = x.size(2);
  auto f32 = x.options().dtype(at::kFloat);
  Tensor dx = torch::empty_like(x);
  Tensor dpm = torch::empty_like(prev_mean);
  Tensor dpv = torch::empty_like(prev_mean);
  Tensor dgamma = torch::zeros({H}, f32);
  Tensor dbeta = torch::zeros({H}, f32);
  Tensor scratch = torch::empty({5, B, L, G}, f32);
  float* sp = scratch.data_ptr<float>();
  const long long n = (long long)B * L * G;
  Tensor seg = torch::empty({4LL * B * mb::tsn_num_segments(L) * G}, x.options().dtype(at::kDouble));
  Tensor cumvalid = torch::empty({mask.has_value() ? (long long)B * L : 0}, x.options().dtype(at::kInt));
  Tensor ws = torch::empty({2LL * mb::kColsumRows * H}, f32);    // partial sums of dgamma | dbeta per CTA
  mb::timestep_norm_bwd(dy.data_ptr(), dmean.data_ptr(), dvar.data_ptr(), x.data_ptr(), prev_mean.data_ptr(),
                        (const long long*)count.data_ptr<int64_t>(), cummean.data_ptr<float>(),
                        cumrstd.data_ptr<float>(), gamma.data_ptr(), (float)gamma_off,
                        mask.has_value() ? mask->data_ptr<bool>() : nullptr, dx.data_ptr(), dpm.data_ptr(),
                        dpv.data_ptr(), dgamma.data_ptr<float>(), dbeta.data_ptr<float>(), sp, sp + n, sp + 2 * n,
                        sp + 3 * n, sp + 4 * n, seg.data_ptr<double>(), cumvalid.data_ptr<int>(), B, L, H, (int)G,
                        dtype_code(x), weight_code(x, gamma), stream(), ws.data_ptr<float>());
  return {dx, dpm, dpv, dgamma, dbeta};
}

// ------------------------------------------------------------------ CEMA
// p [D,N] f32, q/gamma [D,N,2] f32, omega [D] f32, hx [B,D,N,2] f32 or none
std::tuple<Tensor, OptTensor> cema_fwd(const Tensor& x, const Tensor& p, const Tensor& q, const Tensor& gamma,
                                       const Tensor& omega, const OptTensor& hx, bool want_last) {
  check_cuda_contig(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  const int B = x.size(0), L = x.size(1), D = x.size(2), N = p.size(1);
  TORCH_CHECK(mb::cema_supported_ndim(N), "cema: ndim must be one of 1,2,4,8,16,32");
  for (const Tensor* t : {&p, &q, &gamma, &omega}) {
    TORCH_CHECK(t->is_cuda() && t->is_contiguous() && t->scalar_type() == at::kFloat, "cema coefficients must be contiguous fp32");
  }
  auto f32 = x.options().dtype(at::kFloat);
  Tensor y = torch::empty_like(x);
  OptTensor h_last;
  if (want_last) h_last = torch::empty({B, D, N, 2}, f32);
  const int S = mb::cema_num_segments(L);
  Tensor carry = torch::empty({S > 1 ? (long long)B * S * N * D * 2 : 0}, f32);
  mb::cema_fwd(x.data_ptr(), p.data_ptr<float>(), q.data_ptr<float>(), gamma.data_ptr<float>(),
               omega.data_ptr<float>(), hx.has_value() ? hx->data_ptr<float>() : nullptr, y.data_ptr(),
               h_last.has_value() ? h_last->data_ptr<float>() : nullptr, carry.data_ptr<float>(), B, L, D, N,
               dtype_code(x), stream());
  return {y, h_last};
}

// returns dx, dp, dq, dgamma, domega, dhx
std::vector<Tensor> cema_bwd(const Tensor& dy, const Tensor& x, const Tensor& p, const Tensor& q,
                             const Tensor& gamma, const Tensor& omega, const OptTensor& hx,
                             const OptTensor& dh_last) {
  check_cuda_contig(dy, "dy");
  check_cuda_contig(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  const int B = x.size(0), L = x.size(1), D = x.size(2), N = p.size(1);
  auto f32 = x.options().dtype(at::kFloat);
  Tensor dx = torch::empty_like(x);
  Tensor dp = torch::zeros({D, N}, f32);
  Tensor dq = torch::zeros({D, N, 2}, f32);
  Tensor dgamma = torch::zeros({D, N, 2}, f32);
  Tensor domega = torch::zeros({D}, f32);
  Tensor dhx = torch::empty({B, D, N, 2}, f32);
  const int S = mb::cema_num_segments(L);
  const long long cn = S > 1 ? (long long)B * S * N * D * 2 : 0;
  Tensor carry = torch::empty({2 * cn}, f32);
  if (dh_last.has_value()) TORCH_CHECK(dh_last->is_contiguous() && dh_last->scalar_type() == at::kFloat);
  mb::cema_bwd(dy.data_ptr(), x.data_ptr(), p.data_ptr<float>(), q.data_ptr<float>(), gamma.data_ptr<float>(),
               omega.data_ptr<float>(), hx.has_value() ? hx->data_ptr<float>() : nullptr,
               dh_last.has_value() ? dh_last->data_ptr<float>() : nullptr, dx.data_ptr(), dp.data_ptr<float>(),
               dq.data_ptr<float>(), dgamma.data_ptr<float>(), domega.data_ptr<float>(), dhx.data_ptr<float>(),
               carry.data_ptr<float>(), carry.data_ptr<float>() + cn, B, L, D, N, dtype_code(x), stream());
  return {dx, dp, dq, dgamma, domega, dhx};
}

// ------------------------------------------------------------------ element-wise
Tensor swiglu_fwd(const Tensor& a, const Tensor& b) {
  check_cuda_contig(a, "a");
  check_cuda_contig(b, "b");
  c10::cuda::CUDAGuard guard(a.device());
  Tensor out = torch::empty_like(a);
  mb::swiglu_fwd(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), dtype_code(a), stream());
  return out;
}

Tensor silu_bwd(const Tensor& g, const Tensor& a) {
  check_cuda_contig(g, "g");
  check_cuda_contig(a, "a");
  TORCH_CHECK(g.numel() == a.numel() && g.scalar_type() == a.scalar_type(), "silu_bwd: g and a must match");
  c10::cuda::CUDAGuard guard(a.device());
  Tensor da = torch::empty_like(a);
  mb::silu_bwd(g.data_ptr(), a.data_ptr(), da.data_ptr(), a.numel(), dtype_code(a), stream());
  return da;
}

std::tuple<Tensor, Tensor> swiglu_bwd(const Tensor& g, const Tensor& a, const Tensor& b) {
  check_cuda_contig(g, "g");
  c10::cuda::CUDAGuard guard(a.device());
  Tensor da = torch::empty_like(a), db = torch::empty_like(b);
  mb::swiglu_bwd(g.data_ptr(), a.data_ptr(), b.data_ptr(), da.data_ptr(), db.data_ptr(), a.numel(), dtype_code(a),
                 stream());
  return {da, db};
}

// x [rows, H, Dh]; freqs [L, Dh/2, 2] fp32 (cos, sin); position = row % L
Tensor rotary(const Tensor& x, const Tensor& freqs, bool conj) {
  check_cuda_contig(x, "x");
  check_cuda_contig(freqs, "freqs");
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(freqs.scalar_type() == at::kFloat && x.dim() >= 3);
  const int Dh = x.size(-1), H = x.size(-2), L = freqs.size(0);
  TORCH_CHECK(Dh % 2 == 0 && freqs.size(1) == Dh / 2);
  const long long rows = x.numel() / ((long long)H * Dh);
  Tensor out = torch::empty_like(x);
  mb::rotary_apply(x.data_ptr(), freqs.data_ptr<float>(), out.data_ptr(), rows, L, H, Dh, conj, dtype_code(x),
                   stream());
  return out;
}

// z [..., S] (16-bit, S = H * Dh), gamma / beta [2, S] (fp32 or z's dtype), freqs [P, Dh/2, 2] fp32 -> (q, k) like z
std::tuple<Tensor, Tensor> qk_rotary_fwd(const Tensor& z, const Tensor& gamma, const Tensor& beta, const Tensor& freqs,
                                         int64_t Dh) {
  check_cuda_contig(z, "z");
  check_cuda_contig(gamma, "gamma");
  check_cuda_contig(beta, "beta");
  check_cuda_contig(freqs, "freqs");
  c10::cuda::CUDAGuard guard(z.device());
  const int S = z.size(-1), P = freqs.size(0);
  TORCH_CHECK(z.scalar_type() == at::kBFloat16 || z.scalar_type() == at::kHalf, "16-bit activations only");
  TORCH_CHECK(S % 8 == 0 && S <= 8192 && S % Dh == 0 && Dh % 2 == 0 && freqs.scalar_type() == at::kFloat &&
              freqs.size(1) == Dh / 2 && gamma.numel() == 2 * S && beta.numel() == 2 * S);
  TORCH_CHECK(gamma.scalar_type() == beta.scalar_type() &&
              (gamma.scalar_type() == at::kFloat || gamma.scalar_type() == z.scalar_type()));
  Tensor q = torch::empty_like(z), k = torch::empty_like(z);
  mb::qk_rotary_fwd(z.data_ptr(), gamma.data_ptr(), beta.data_ptr(), freqs.data_ptr<float>(), q.data_ptr(), k.data_ptr(),
                    z.numel() / S, S, (int)Dh, P, dtype_code(z), dtype_code(gamma), stream());
  return {q, k};
}

// -> (dz like z, dgamma [2, S] fp32, dbeta [2, S] fp32)
std::tuple<Tensor, Tensor, Tensor> qk_rotary_bwd(const Tensor& dq, const Tensor& dk, const Tensor& z, const Tensor& gamma,
                                                 const Tensor& freqs, int64_t Dh) {
  check_cuda_contig(dq, "dq");
  check_cuda_contig(dk, "dk");
  check_cuda_contig(z, "z");
  check_cuda_contig(gamma, "gamma");
  c10::cuda::CUDAGuard guard(z.device());
  const int S = z.size(-1), P = freqs.size(0);
  const long long rows = z.numel() / S;
  TORCH_CHECK(dq.sizes() == z.sizes() && dk.sizes() == z.sizes() && dq.scalar_type() == z.scalar_type() &&
              dk.scalar_type() == z.scalar_type() && S % 8 == 0 && S <= 8192);
  Tensor dz = torch::empty_like(z);
  const int ctas = mb::qk_rotary_bwd_ctas(rows);
  Tensor partial = torch::empty({ctas, 4, S}, z.options().dtype(at::kFloat));
  mb::qk_rotary_bwd(dq.data_ptr(), dk.data_ptr(), z.data_ptr(), gamma.data_ptr(), freqs.data_ptr<float>(), dz.data_ptr(),
                    partial.data_ptr<float>(), rows, S, (int)Dh, P, dtype_code(z), dtype_code(gamma), stream());
  Tensor sums = partial.sum(0);                       // [4, S]
  return {dz, sums.narrow(0, 0, 2), sums.narrow(0, 2, 2)};
}

std::tuple<Tensor, Tensor> cross_entropy_fwd(const Tensor& logits, const Tensor& target, int64_t ignore_index) {
  check_cuda_contig(logits, "logits");
  check_cuda_contig(target, "target");
  c10::cuda::CUDAGuard guard(logits.device());
  TORCH_CHECK(logits.dim() == 2 && target.scalar_type() == at::kLong);
  const long long rows = logits.size(0);
  auto f32 = logits.options().dtype(at::kFloat);
  Tensor loss = torch::empty({rows}, f32), lse = torch::empty({rows}, f32);
  mb::cross_entropy_fwd(logits.data_ptr(), (const long long*)target.data_ptr<int64_t>(), loss.data_ptr<float>(),
                        lse.data_ptr<float>(), rows, (int)logits.size(1), ignore_index, dtype_code(logits), stream());
  return {loss, lse};
}

Tensor cross_entropy_bwd(const Tensor& logits, const Tensor& target, const Tensor& lse, const Tensor& dloss,
                         int64_t ignore_index) {
  c10::cuda::CUDAGuard guard(logits.device());
  Tensor dlogits = torch::empty_like(logits);
  Tensor dl = dloss.to(at::kFloat).contiguous();
  mb::cross_entropy_bwd(logits.data_ptr(), (const long long*)target.data_ptr<int64_t>(), lse.data_ptr<float>(),
                        dl.data_ptr<float>(), dlogits.data_ptr(), logits.size(0), (int)logits.size(1), ignore_index,
                        dtype_code(logits), stream());
  return dlogits;
}

void adamw_step(Tensor& p, const Tensor& g, Tensor& m, Tensor& v, const OptTensor& low, double lr, double beta1,
                double beta2, double eps, double wd, int64_t step, double grad_scale, const OptTensor& scale_ptr) {
  check_cuda_contig(p, "param");
  check_cuda_contig(g, "grad");
  c10::cuda::CUDAGuard guard(p.device());
  TORCH_CHECK(p.scalar_type() == at::kFloat && m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat);
  TORCH_CHECK(g.numel() == p.numel() && m.numel() == p.numel() && v.numel() == p.numel());
  if (low.has_value()) TORCH_CHECK(low->numel() == p.numel() && low->is_contiguous());
  for (const void* ptr : {(const void*)p.data_ptr(), (const void*)g.data_ptr(), (const void*)m.data_ptr(),
                          (const void*)v.data_ptr()})
    TORCH_CHECK(reinterpret_cast<uintptr_t>(ptr) % 16 == 0, "adamw_step: tensors must be 16-byte aligned");
  if (low.has_value()) TORCH_CHECK(reinterpret_cast<uintptr_t>(low->data_ptr()) % 8 == 0);
  mb::adamw_step(p.data_ptr<float>(), g.data_ptr(), m.data_ptr<float>(), v.data_ptr<float>(),
                 low.has_value() ? low->data_ptr() : nullptr, p.numel(), (float)lr, (float)beta1, (float)beta2,
                 (float)eps, (float)wd, (int)step, (float)grad_scale,
                 scale_ptr.has_value() ? scale_ptr->data_ptr<float>() : nullptr, dtype_code(g),
                 low.has_value() ? dtype_code(*low) : 1, stream());
}

void sum_squares(const Tensor& g, Tensor& out) {
  check_cuda_contig(g, "g");
  c10::cuda::CUDAGuard guard(g.device());
  TORCH_CHECK(out.scalar_type() == at::kDouble && out.numel() == 1);
  mb::sum_squares(g.data_ptr(), g.numel(), out.data_ptr<double>(), dtype_code(g), stream());
}

void scale_by_ptr(Tensor& g, const Tensor& scale) {
  check_cuda_contig(g, "g");
  c10::cuda::CUDAGuard guard(g.device());
  mb::scale_by_ptr(g.data_ptr(), g.numel(), scale.data_ptr<float>(), dtype_code(g), stream());
}

std::tuple<Tensor, Tensor> clip_coef(const Tensor& sumsq, double max_norm) {
  c10::cuda::CUDAGuard guard(sumsq.device());
  auto f32 = sumsq.options().dtype(at::kFloat);
  Tensor norm = torch::empty({}, f32), coef = torch::empty({}, f32);
  mb::clip_coef(sumsq.data_ptr<double>(), (float)max_norm, norm.data_ptr<float>(), coef.data_ptr<float>(), stream());
  return {norm, coef};
}

// ------------------------------------------------------------------ GEMM
// C = act(alpha * A B^T + bias) on the tcgen05 kernel.  A, B (and `out`) are 2-D matrices or 3-D
// batches of matrices whose last dim is contiguous; row and batch strides are taken from the tensors,
// so strided views (one head of a [B, L, H, d] tensor, a slice of a flat buffer) need no copy.
// a_mn / b_mn: the operand is stored [K, rows] instead of [rows, K].  mode: causal tile structure
// (0 dense; see gemm_sm100.cu).  Returns (C, preact or None, launch status); `err` is a persistent
// int32 device flag that the kernel sets if one of its bounded waits gives up.
std::tuple<Tensor, OptTensor, int64_t> gemm(const Tensor& A, const Tensor& B, const OptTensor& out,
                                            const OptTensor& bias, int64_t act, bool a_mn, bool b_mn,
                                            bool want_preact, int64_t out_dtype_code, int64_t mode, double alpha,
                                            Tensor& err, const std::vector<int64_t>& a_part_ptrs, int64_t a_first,
                                            const std::vector<int64_t>& c_part_ptrs, bool accumulate,
                                            const std::vector<int64_t>& b_gather_ptrs, int64_t b_gather_rank,
                                            int64_t epi_kind, const OptTensor& row_in, const OptTensor& row_in2,
                                            const OptTensor& row_out, const OptTensor& aux, int64_t causal_off) {
  TORCH_CHECK(A.is_cuda() && B.is_cuda(), "operands must be CUDA tensors");
  c10::cuda::CUDAGuard guard(A.device());
  TORCH_CHECK((A.dim() == 2 || A.dim() == 3) && A.dim() == B.dim(), "operands must both be 2-D or both 3-D");
  TORCH_CHECK(A.scalar_type() == B.scalar_type());
  TORCH_CHECK(A.scalar_type() == at::kBFloat16 || A.scalar_type() == at::kHalf, "tcgen05 GEMM takes bf16/fp16");
  TORCH_CHECK(A.stride(-1) == 1 && B.stride(-1) == 1, "last dim of the operands must be contiguous");
  const int batch = A.dim() == 3 ? (int)A.size(0) : 1;
  TORCH_CHECK(A.dim() == 2 || B.size(0) == batch, "batch sizes differ");
  // with a gathered A, `A` is this rank's piece [M, K / parts] and only supplies shape, stride and dtype
  const int a_parts = a_part_ptrs.empty() ? 1 : (int)a_part_ptrs.size();
  const int M = a_mn ? A.size(-1) : A.size(-2);
  const int K = (a_mn ? A.size(-2) : A.size(-1)) * a_parts;
  const int N = b_mn ? B.size(-1) : B.size(-2);
  TORCH_CHECK((b_mn ? B.size(-2) : B.size(-1)) == K, "inner dimensions differ");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(A.data_ptr()) % 16 == 0 && reinterpret_cast<uintptr_t>(B.data_ptr()) % 16 == 0,
              "operands must be 16-byte aligned");
  at::ScalarType odt = out_dtype_code == 0 ? at::kFloat : (out_dtype_code == 1 ? at::kBFloat16 : at::kHalf);
  Tensor C;
  if (out.has_value()) {
    C = *out;
    TORCH_CHECK(C.is_cuda() && C.scalar_type() == odt && C.dim() == A.dim() && C.stride(-1) == 1);
    TORCH_CHECK(C.size(-2) == M && C.size(-1) == N && (A.dim() == 2 || C.size(0) == batch), "bad output shape");
    TORCH_CHECK(reinterpret_cast<uintptr_t>(C.data_ptr()) % 16 == 0, "output must be 16-byte aligned");
  } else {
    C = A.dim() == 3 ? torch::empty({batch, M, N}, A.options().dtype(odt)) : torch::empty({M, N}, A.options().dtype(odt));
  }
  OptTensor pre;
  if (want_preact) {
    TORCH_CHECK(batch == 1 && !out.has_value(), "pre-activation output is only available for plain 2-D calls");
    pre = torch::empty({M, N}, A.options().dtype(odt));
  }
  int bias_code = 0;
  if (bias.has_value()) {
    check_cuda_contig(*bias, "bias");
    bias_code = dtype_code(*bias);
    TORCH_CHECK(bias->numel() == N);
  }
  const long long a_bs = A.dim() == 3 ? A.stride(0) : 0, b_bs = B.dim() == 3 ? B.stride(0) : 0;
  const long long c_bs = C.dim() == 3 ? C.stride(0) : 0;
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  mb::GemmPeerSpec peers;
  TORCH_CHECK(a_part_ptrs.size() <= 8 && c_part_ptrs.size() <= 8, "at most 8 peers");
  if (a_parts > 1) {
    peers.a_parts = a_parts;
    peers.a_first = (int)a_first;
    for (int i = 0; i < a_parts; ++i) peers.a_ptrs[i] = reinterpret_cast<const void*>(a_part_ptrs[i]);
  }
  if (c_part_ptrs.size() > 1) {
    peers.c_nparts = (int)c_part_ptrs.size();
    for (size_t i = 0; i < c_part_ptrs.size(); ++i) peers.c_ptrs[i] = reinterpret_cast<void*>(c_part_ptrs[i]);
  }
  // gathered weight operand: b_gather_ptrs[r] = rank r's row block, B = the local full matrix it lands in
  mb::GemmGatherSpec gather;
  if (!b_gather_ptrs.empty()) {
    TORCH_CHECK(b_gather_ptrs.size() <= 8 && B.dim() == 2 && B.is_contiguous(), "gathered B must be a contiguous matrix");
    TORCH_CHECK(mb::gemm_gather_supported(M, N, K, (int)b_gather_ptrs.size()), "shape not supported by the gathering GEMM");
    gather.world = (int)b_gather_ptrs.size();
    gather.rank = (int)b_gather_rank;
    for (size_t i = 0; i < b_gather_ptrs.size(); ++i) gather.src[i] = reinterpret_cast<const void*>(b_gather_ptrs[i]);
    gather.dst = B.data_ptr();
    static thread_local Tensor flags;          // one scratch per device is enough: uses are ordered on the stream
    if (!flags.defined() || flags.device() != A.device())
      flags = torch::zeros({512}, A.options().dtype(at::kInt));
    TORCH_CHECK(mb::gemm_gather_flag_words(N) <= flags.numel());
    gather.flags = reinterpret_cast<unsigned int*>(flags.data_ptr<int>());
  }
  // softmax fused into the epilogue (attention products): fp32 row vectors [batch, M]
  mb::GemmSoftmaxSpec sm;
  bool with_addend = false;
  if (epi_kind == 0 && aux.has_value()) {
    TORCH_CHECK(aux->is_cuda() && aux->scalar_type() == C.scalar_type() && aux->sizes() == C.sizes() &&
                aux->strides() == C.strides(), "the addend must have the dtype and layout of the output");
    sm.aux = aux->data_ptr();
    with_addend = true;
  }
  if (epi_kind != 0) {
    auto rowvec = [&](const OptTensor& t, const char* what) -> float* {
      TORCH_CHECK(t.has_value() && t->is_cuda() && t->scalar_type() == at::kFloat && t->is_contiguous() &&
                  t->numel() == (int64_t)batch * M, what, ": expected a contiguous fp32 [batch, M] CUDA tensor");
      return t->data_ptr<float>();
    };
    sm.kind = (int)epi_kind;
    sm.causal_off = (int)causal_off;
    if (epi_kind == 1) sm.row_out = rowvec(row_out, "row_out");
    if (epi_kind == 2) { sm.row_in = rowvec(row_in, "row_in"); sm.row_out = rowvec(row_out, "row_out"); }
    if (epi_kind == 3) sm.row_in = rowvec(row_in, "row_in");
    if (epi_kind == 4) {
      sm.row_in = rowvec(row_in, "row_in");
      sm.row_in2 = rowvec(row_in2, "row_in2");
      TORCH_CHECK(aux.has_value() && aux->scalar_type() == C.scalar_type() && aux->sizes() == C.sizes() &&
                  aux->strides() == C.strides(), "aux must have the dtype and layout of the output");
      sm.aux = aux->data_ptr();
    }
  }
  const int rc = mb::gemm_bf16_tcgen05(A.data_ptr(), B.data_ptr(), C.data_ptr(),
                                       pre.has_value() ? pre->data_ptr() : nullptr, opt_ptr(bias), bias_code,
                                       (int)act, M, N, K, A.stride(-2), B.stride(-2), C.stride(-2), a_mn, b_mn,
                                       (int)mode, (float)alpha, batch, a_bs, b_bs, c_bs, dtype_code(A),
                                       (int)out_dtype_code, err.data_ptr<int>(), sms, stream(),
                                       (a_parts > 1 || c_part_ptrs.size() > 1) ? &peers : nullptr,
                                       accumulate && out.has_value(), gather.world > 0 ? &gather : nullptr,
                                       (sm.kind != 0 || with_addend) ? &sm : nullptr);
  // the launcher's status goes back to Python, which raises on a non-zero code
  return {C, pre, (int64_t)rc};
}

// x [M <= 16, K], w [N, K] (rows contiguous) -> y [M, N]; returns an empty optional if the kernel does not apply
OptTensor gemv_small_m(const Tensor& x, const Tensor& w, const OptTensor& bias, int64_t act, int64_t out_dtype_code,
                       double alpha) {
  TORCH_CHECK(x.is_cuda() && w.is_cuda() && x.dim() == 2 && w.dim() == 2 && x.size(1) == w.size(1));
  TORCH_CHECK(x.stride(1) == 1 && w.stride(1) == 1 && x.scalar_type() == w.scalar_type());
  c10::cuda::CUDAGuard guard(x.device());
  const int M = x.size(0), K = x.size(1), N = w.size(0);
  at::ScalarType odt = out_dtype_code == 0 ? at::kFloat : (out_dtype_code == 1 ? at::kBFloat16 : at::kHalf);
  Tensor y = torch::empty({M, N}, x.options().dtype(odt));
  int bias_code = 0;
  if (bias.has_value()) {
    check_cuda_contig(*bias, "bias");
    bias_code = dtype_code(*bias);
    TORCH_CHECK(bias->numel() == N);
  }
  const bool ok = mb::gemv_small_m(x.data_ptr(), w.data_ptr(), opt_ptr(bias), bias_code, y.data_ptr(), M, N, K,
                                   x.stride(0), w.stride(0), y.stride(0), (float)alpha, (int)act, dtype_code(x),
                                   (int)out_dtype_code, stream());
  if (!ok) return OptTensor();
  return y;
}

// ------------------------------------------------------------------ FFT long convolution
// x [..., L] contiguous -> half spectrum [..., N2/2 + 1, 2] (fp32 pairs) of the zero-padded row
Tensor rfft_rows(const Tensor& x, bool flip, int64_t packed) {
  check_cuda_contig(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  const int L = x.size(-1);
  TORCH_CHECK(mb::fftconv_supported(L), "rfft: length > 16384 is not supported by the native kernel");
  const long long rows = x.numel() / L;
  const int bins = (1 << mb::fftconv_logn(L)) / 2 + 1;
  auto shape = x.sizes().vec();
  shape.back() = bins;
  shape.push_back(2);
  Tensor out = torch::empty(shape, x.options().dtype(at::kFloat));
  mb::rfft_rows(x.data_ptr(), out.data_ptr<float>(), rows, L, flip, dtype_code(x), stream(), (int)packed);
  return out;
}

// spec [..., N2/2 + 1, 2] fp32 -> first L samples of the inverse real transform, [..., L] fp32
Tensor irfft_rows(const Tensor& spec, int64_t L, int64_t packed) {
  check_cuda_contig(spec, "spec");
  c10::cuda::CUDAGuard guard(spec.device());
  TORCH_CHECK(mb::fftconv_supported((int)L) && spec.scalar_type() == at::kFloat && spec.dim() >= 2 && spec.size(-1) == 2);
  const int bins = (1 << mb::fftconv_logn((int)L)) / 2 + 1;
  TORCH_CHECK(spec.size(-2) == bins, "spectrum must have N2/2 + 1 bins for this length");
  auto shape = spec.sizes().vec();
  shape.pop_back();
  shape.back() = L;
  Tensor out = torch::empty(shape, spec.options());
  mb::irfft_rows(spec.data_ptr<float>(), out.data_ptr<float>(), out.numel() / L, (int)L, stream(), (int)packed);
  return out;
}

// x [B, D, L], kf [D, N2/2 + 1, 2] -> y [B, D, L] = irfft(rfft(x) * kf (or conj kf))[:L]
Tensor fftconv_apply(const Tensor& x, const Tensor& kf, bool conj_k, int64_t packed) {
  check_cuda_contig(x, "x");
  check_cuda_contig(kf, "kf");
  c10::cuda::CUDAGuard guard(x.device());
  const int L = x.size(-1), D = x.size(-2);
  const int bins = (1 << mb::fftconv_logn(L)) / 2 + 1;
  TORCH_CHECK(mb::fftconv_supported(L) && kf.scalar_type() == at::kFloat && kf.numel() == (long long)D * bins * 2);
  Tensor y = torch::empty_like(x);
  mb::fftconv_rows(x.data_ptr(), kf.data_ptr<float>(), y.data_ptr(), x.numel() / L, L, D, conj_k, dtype_code(x),
                   stream(), (int)packed);
  return y;
}

// dk [D, L] fp32 = sum over batch of the correlation of dy with x
Tensor fftconv_dk(const Tensor& dy, const Tensor& x) {
  check_cuda_contig(dy, "dy");
  check_cuda_contig(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  const int L = x.size(-1), D = x.size(-2);
  TORCH_CHECK(mb::fftconv_logn(L) <= 14 && dy.sizes() == x.sizes() && dy.scalar_type() == x.scalar_type());
  const int bins = (1 << mb::fftconv_logn(L)) / 2 + 1;
  Tensor acc = torch::zeros({D, bins, 2}, x.options().dtype(at::kFloat));
  Tensor dk = torch::empty({D, L}, x.options().dtype(at::kFloat));
  mb::fftconv_dk(dy.data_ptr(), x.data_ptr(), acc.data_ptr<float>(), dk.data_ptr<float>(), x.numel() / L, L, D,
                 dtype_code(x), stream());
  return dk;
}

// ------------------------------------------------------------------ attention softmax (in place)
// s [..., L1, L2] with contiguous last dim and uniform row stride; returns lse [rows] (fp32)
Tensor attn_softmax_fwd(Tensor& s, int64_t L1, int64_t L2, bool causal, double drop_p, int64_t seed,
                        int64_t offset) {
  TORCH_CHECK(s.is_cuda() && s.stride(-1) == 1 && L2 <= 8192, "attention softmax: bad input");
  c10::cuda::CUDAGuard guard(s.device());
  const long long ld = s.stride(-2);
  const long long rows = s.numel() / s.size(-1);
  for (int d = 0; d + 2 < s.dim(); ++d) TORCH_CHECK(s.stride(d) == s.stride(d + 1) * s.size(d + 1), "rows must be evenly strided");
  Tensor lse = torch::empty({rows}, s.options().dtype(at::kFloat));
  mb::attn_softmax_fwd(s.data_ptr(), lse.data_ptr<float>(), rows, (int)L1, (int)L2, ld, causal, (float)drop_p,
                       (unsigned long long)seed, (unsigned long long)offset, dtype_code(s), stream());
  return lse;
}

void attn_softmax_bwd(const Tensor& p, Tensor& dp, int64_t L1, int64_t L2, bool causal) {
  TORCH_CHECK(p.is_cuda() && dp.is_cuda() && p.stride(-1) == 1 && dp.stride(-1) == 1);
  TORCH_CHECK(p.stride(-2) == dp.stride(-2) && p.scalar_type() == dp.scalar_type() && L2 <= 8192);
  c10::cuda::CUDAGuard guard(p.device());
  const long long rows = p.numel() / p.size(-1);
  mb::attn_softmax_bwd(p.data_ptr(), dp.data_ptr(), rows, (int)L1, (int)L2, p.stride(-2), causal, dtype_code(p),
                       stream());
}

// q [B, H, dk], k_buf [B, H, C, dk], v_buf [B, H, C, dv] (16-bit, contiguous), pos int64 device tensor [1] -> [B, H, dv]
Tensor decode_attention(const Tensor& q, const Tensor& k_buf, const Tensor& v_buf, const Tensor& pos, double scale) {
  check_cuda_contig(q, "q");
  check_cuda_contig(k_buf, "k_buf");
  check_cuda_contig(v_buf, "v_buf");
  c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(q.dim() == 3 && k_buf.dim() == 4 && v_buf.dim() == 4 && pos.is_cuda() && pos.scalar_type() == at::kLong);
  TORCH_CHECK(q.scalar_type() == at::kBFloat16 || q.scalar_type() == at::kHalf);
  TORCH_CHECK(k_buf.scalar_type() == q.scalar_type() && v_buf.scalar_type() == q.scalar_type());
  const int B = q.size(0), H = q.size(1), dk = q.size(2), C = k_buf.size(2), dv = v_buf.size(3);
  TORCH_CHECK(k_buf.size(0) == B && k_buf.size(1) == H && k_buf.size(3) == dk && v_buf.size(2) == C && dk % 8 == 0);
  TORCH_CHECK(C * 4 <= 200 * 1024, "key buffer too long for the score array in shared memory");
  Tensor out = torch::empty({B, H, dv}, q.options());
  mb::decode_attention(q.data_ptr(), k_buf.data_ptr(), v_buf.data_ptr(),
                       reinterpret_cast<const long long*>(pos.data_ptr<int64_t>()), out.data_ptr(), B * H,
                       C, dk, dv, (float)scale, dtype_code(q), stream());
  return out;
}

// dout, out [B, L, H, dv] (16-bit), rowsum [B, H, L] fp32 -> (dout / rowsum, delta [B, H, L] = dout . out)
std::tuple<Tensor, Tensor> attn_bwd_prep(const Tensor& dout, const Tensor& out, const Tensor& rowsum) {
  check_cuda_contig(dout, "dout");
  check_cuda_contig(out, "out");
  check_cuda_contig(rowsum, "rowsum");
  c10::cuda::CUDAGuard guard(dout.device());
  TORCH_CHECK(dout.dim() == 4 && dout.sizes() == out.sizes() && dout.scalar_type() == out.scalar_type());
  TORCH_CHECK(dout.scalar_type() == at::kBFloat16 || dout.scalar_type() == at::kHalf);
  const int B = dout.size(0), L = dout.size(1), H = dout.size(2), dv = dout.size(3);
  TORCH_CHECK(dv % 8 == 0 && rowsum.scalar_type() == at::kFloat && rowsum.numel() == (int64_t)B * H * L);
  Tensor dos = torch::empty_like(dout);
  Tensor delta = torch::empty({B, H, L}, rowsum.options());
  mb::attn_bwd_prep(dout.data_ptr(), out.data_ptr(), rowsum.data_ptr<float>(), dos.data_ptr(), delta.data_ptr<float>(),
                    B, L, H, dv, dtype_code(dout), stream());
  return {dos, delta};
}

// ------------------------------------------------------------------ SequenceNorm pieces, dropout, CEMA coefficients
// sums over valid time steps per (b, h): (sum u, sum u*v) or (sum u, sum u^2) when v is None
std::tuple<Tensor, Tensor> time_sums(const Tensor& u, const OptTensor& v, const OptTensor& mask, bool length_last) {
  check_cuda_contig(u, "u");
  c10::cuda::CUDAGuard guard(u.device());
  TORCH_CHECK(u.dim() == 3);
  const int B = u.size(0), L = length_last ? u.size(2) : u.size(1), H = length_last ? u.size(1) : u.size(2);
  auto f32 = u.options().dtype(at::kFloat);
  Tensor s1 = torch::empty({B, H}, f32), s2 = torch::empty({B, H}, f32);
  if (v.has_value()) check_cuda_contig(*v, "v");
  mb::time_sums(u.data_ptr(), opt_ptr(v), mask.has_value() ? mask->data_ptr<bool>() : nullptr, s1.data_ptr<float>(),
                s2.data_ptr<float>(), B, L, H, length_last, dtype_code(u), stream());
  return {s1, s2};
}

// out = a[b,h] * p + c[b,h] * q + d[b,h], zero on padded steps
Tensor affine_apply(const Tensor& p, const OptTensor& q, const Tensor& a, const OptTensor& c, const Tensor& d,
                    const OptTensor& mask, bool length_last) {
  check_cuda_contig(p, "p");
  c10::cuda::CUDAGuard guard(p.device());
  const int B = p.size(0), L = length_last ? p.size(2) : p.size(1), H = length_last ? p.size(1) : p.size(2);
  TORCH_CHECK(a.scalar_type() == at::kFloat && d.scalar_type() == at::kFloat && a.is_contiguous() && d.is_contiguous());
  TORCH_CHECK(q.has_value() == c.has_value());
  Tensor out = torch::empty_like(p);
  mb::affine_apply(p.data_ptr(), opt_ptr(q), a.data_ptr<float>(), c.has_value() ? c->data_ptr<float>() : nullptr,
                   d.data_ptr<float>(), mask.has_value() ? mask->data_ptr<bool>() : nullptr, out.data_ptr(), B, L, H,
                   length_last, dtype_code(p), stream());
  return out;
}

Tensor dropout(const Tensor& x, double p, int64_t seed, int64_t offset) {
  check_cuda_contig(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor out = torch::empty_like(x);
  mb::dropout_apply(x.data_ptr(), out.data_ptr(), x.numel(), (float)p, (unsigned long long)seed,
                    (unsigned long long)offset, dtype_code(x), stream());
  return out;
}

// p [D,N] f32, logq / gamma [D,N,2] f32, h [B,D,N,2] f32 or None -> (k [D,L], bias [B,D,L] or None)
std::tuple<Tensor, OptTensor> ema_parameters_fwd(const Tensor& p, const Tensor& logq, const Tensor& gamma,
                                                 const OptTensor& h, int64_t L) {
  check_cuda_contig(p, "p");
  check_cuda_contig(logq, "logq");
  check_cuda_contig(gamma, "gamma");
  c10::cuda::CUDAGuard guard(p.device());
  const int D = p.size(0), N = p.size(1);
  const int B = h.has_value() ? h->size(0) : 0;
  Tensor k = torch::empty({D, L}, p.options());
  OptTensor bias;
  if (h.has_value()) { check_cuda_contig(*h, "h"); bias = torch::empty({B, D, L}, p.options()); }
  mb::ema_parameters_fwd(p.data_ptr<float>(), logq.data_ptr<float>(), gamma.data_ptr<float>(),
                         h.has_value() ? h->data_ptr<float>() : nullptr, k.data_ptr<float>(),
                         bias.has_value() ? bias->data_ptr<float>() : nullptr, B, D, N, (int)L, stream());
  return {k, bias};
}

// returns dp [D,N], dq [D,N,2], dgamma [D,N,2], dh [B,D,N,2] or None
std::vector<OptTensor> ema_parameters_bwd(const OptTensor& dk, const OptTensor& dbias, const Tensor& p,
                                          const Tensor& logq, const Tensor& gamma, const OptTensor& h, int64_t L) {
  c10::cuda::CUDAGuard guard(p.device());
  const int D = p.size(0), N = p.size(1);
  const int B = h.has_value() ? h->size(0) : 0;
  Tensor dp = torch::empty_like(p), dq = torch::empty_like(logq), dg = torch::empty_like(gamma);
  OptTensor dh;
  if (h.has_value()) dh = torch::zeros_like(*h);
  if (dk.has_value()) check_cuda_contig(*dk, "dk");
  if (dbias.has_value()) check_cuda_contig(*dbias, "dbias");
  mb::ema_parameters_bwd(dk.has_value() ? dk->data_ptr<float>() : nullptr,
                         dbias.has_value() ? dbias->data_ptr<float>() : nullptr, p.data_ptr<float>(),
                         logq.data_ptr<float>(), gamma.data_ptr<float>(), h.has_value() ? h->data_ptr<float>() : nullptr,
                         dp.data_ptr<float>(), dq.data_ptr<float>(), dg.data_ptr<float>(),
                         dh.has_value() ? dh->data_ptr<float>() : nullptr, B, D, N, (int)L, stream());
  return {dp, dq, dg, dh};
}

// ------------------------------------------------------------------ peer-memory communication
// Peer addresses are passed as integers (they come from the symmetric-memory rendezvous and are not
// tensors of this process).  `counter` / `err` are small device tensors owned by the caller.
// Device-side address of a pinned host tensor (what a kernel must use to write to it); 0 if the
// memory is not mapped into the device's address space.
int64_t pinned_device_ptr(const Tensor& t) {
  TORCH_CHECK(!t.is_cuda() && t.is_pinned(), "expects a pinned host tensor");
  void* dptr = nullptr;
  if (cudaHostGetDevicePointer(&dptr, t.data_ptr(), 0) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return reinterpret_cast<int64_t>(dptr);
}

// `abort`: the device's abort record (int32[kCommAbortWords], see comm_kernels.cu)
int* abort_ptr(Tensor& abort) {
  TORCH_CHECK(abort.is_cuda() && abort.scalar_type() == at::kInt && abort.is_contiguous() &&
              abort.numel() >= mb::kCommAbortWords, "abort record must be a CUDA int32 tensor of 16 words");
  return abort.data_ptr<int>();
}

void p2p_send(const Tensor& src, int64_t remote_dst, int64_t nbytes, int64_t remote_flag, int64_t seq,
              int64_t local_ack, int64_t need_ack, Tensor& counter, int64_t timeout_ns, Tensor& abort, int64_t rank,
              int64_t dir) {
  check_cuda_contig(src, "src");
  c10::cuda::CUDAGuard guard(src.device());
  TORCH_CHECK(nbytes % 16 == 0 && nbytes <= (int64_t)(src.numel() * src.element_size()), "payload must be whole 16-byte words");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(src.data_ptr()) % 16 == 0 && remote_dst % 16 == 0);
  mb::p2p_send(src.data_ptr(), reinterpret_cast<void*>(remote_dst), nbytes, reinterpret_cast<unsigned int*>(remote_flag),
               (unsigned int)seq, reinterpret_cast<const unsigned int*>(local_ack), (unsigned int)need_ack,
               reinterpret_cast<unsigned int*>(counter.data_ptr<int>()), (unsigned long long)timeout_ns,
               abort_ptr(abort), (int)rank, (int)dir, stream());
}

void p2p_recv(Tensor& dst, int64_t local_slot, int64_t nbytes, int64_t local_flag, int64_t seq, int64_t remote_ack,
              Tensor& counter, int64_t timeout_ns, Tensor& abort, int64_t rank, int64_t dir, bool poison) {
  check_cuda_contig(dst, "dst");
  c10::cuda::CUDAGuard guard(dst.device());
  TORCH_CHECK(nbytes % 16 == 0 && nbytes <= (int64_t)(dst.numel() * dst.element_size()));
  TORCH_CHECK(reinterpret_cast<uintptr_t>(dst.data_ptr()) % 16 == 0 && local_slot % 16 == 0);
  mb::p2p_recv(dst.data_ptr(), reinterpret_cast<void*>(local_slot), nbytes,
               reinterpret_cast<const unsigned int*>(local_flag), (unsigned int)seq,
               reinterpret_cast<unsigned int*>(remote_ack), reinterpret_cast<unsigned int*>(counter.data_ptr<int>()),
               (unsigned long long)timeout_ns, abort_ptr(abort), (int)rank, (int)dir, poison, stream());
}

// pads: int64 device tensor with the address of every rank's signal pad
void peer_barrier(const Tensor& pads, int64_t rank, int64_t epoch, int64_t timeout_ns, Tensor& abort, int64_t tag) {
  check_cuda_contig(pads, "pads");
  c10::cuda::CUDAGuard guard(pads.device());
  TORCH_CHECK(pads.scalar_type() == at::kLong && pads.numel() <= 32);
  mb::peer_barrier(reinterpret_cast<unsigned int* const*>(pads.data_ptr<int64_t>()), (int)rank, (int)pads.numel(),
                   (unsigned int)epoch, (unsigned long long)timeout_ns, abort_ptr(abort), (int)tag, stream());
}

// Sum over the group (gather = false) or concatenation along the last dimension (gather = true) of a
// small contiguous 16-bit tensor; `counter` (int32[1]) is the device-side epoch.  Captures in a CUDA graph.
Tensor small_collective(const Tensor& x, const Tensor& bufs, const Tensor& pads, Tensor& counter, int64_t rank,
                        int64_t slot_bytes, bool gather, int64_t timeout_ns, Tensor& abort) {
  check_cuda_contig(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t world = bufs.numel();
  const int64_t nbytes = x.numel() * x.element_size();
  TORCH_CHECK(x.element_size() == 2 && nbytes % 16 == 0 && nbytes <= slot_bytes && slot_bytes % 16 == 0,
              "small_collective: 16-bit tensor of a multiple of 16 bytes, at most one slot");
  TORCH_CHECK(bufs.scalar_type() == at::kLong && pads.scalar_type() == at::kLong && pads.numel() == world && world <= 32);
  TORCH_CHECK(counter.is_cuda() && counter.scalar_type() == at::kInt);
  const int64_t last = x.size(-1);
  const int64_t rows = x.numel() / last;
  if (gather) TORCH_CHECK((last * 2) % 16 == 0, "small_collective: rows of a multiple of 16 bytes");
  std::vector<int64_t> shape(x.sizes().begin(), x.sizes().end());
  if (gather) shape.back() = last * world;
  Tensor out = torch::empty(shape, x.options());
  mb::small_collective(x.data_ptr(), out.data_ptr(), reinterpret_cast<void* const*>(bufs.data_ptr<int64_t>()),
                       reinterpret_cast<unsigned int* const*>(pads.data_ptr<int64_t>()),
                       reinterpret_cast<unsigned int*>(counter.data_ptr<int>()), (int)rank, (int)world, nbytes,
                       slot_bytes, (int)rows, gather, dtype_code(x), (unsigned long long)timeout_ns, abort_ptr(abort),
                       stream());
  return out;
}

// bufs: int64 device tensor with the address of every rank's copy of the buffer (same byte offset everywhere)
const int* opt_abort(const OptTensor& abort) {
  if (!abort.has_value()) return nullptr;
  TORCH_CHECK(abort->is_cuda() && abort->scalar_type() == at::kInt && abort->numel() >= 1);
  return abort->data_ptr<int>();
}

void allreduce_sumsq(const Tensor& bufs, int64_t rank, int64_t nbytes, double scale, const OptTensor& sumsq,
                     int64_t dtype, const OptTensor& abort) {
  check_cuda_contig(bufs, "bufs");
  c10::cuda::CUDAGuard guard(bufs.device());
  TORCH_CHECK(bufs.scalar_type() == at::kLong && nbytes % 16 == 0);
  if (sumsq.has_value()) TORCH_CHECK(sumsq->scalar_type() == at::kDouble && sumsq->numel() == 1);
  mb::allreduce_sumsq(reinterpret_cast<void* const*>(bufs.data_ptr<int64_t>()), (int)rank, (int)bufs.numel(), nbytes,
                      (float)scale, sumsq.has_value() ? sumsq->data_ptr<double>() : nullptr, (int)dtype, opt_abort(abort),
                      stream());
}

// piece table of per-parameter sharding: int64 [P, 3] on the device (see comm_kernels.cu)
const long long* table_ptr(const OptTensor& table, int* npieces) {
  *npieces = 0;
  if (!table.has_value()) return nullptr;
  TORCH_CHECK(table->is_cuda() && table->scalar_type() == at::kLong && table->is_contiguous() && table->dim() == 2 &&
              table->size(1) == 3, "piece table must be a contiguous CUDA int64 [P, 3] tensor");
  TORCH_CHECK(table->size(0) <= mb::piece_table_limit(), "more parameters in one unit than the kernels' piece table holds");
  *npieces = (int)table->size(0);
  return reinterpret_cast<const long long*>(table->data_ptr<int64_t>());
}

// full (natural order) <- piece r of every parameter from peer_shards[r], for every rank r
void gather_pull(Tensor& full, const Tensor& peer_shards, const Tensor& table, int64_t listed_numel,
                 const OptTensor& abort, int64_t shard_numel) {
  check_cuda_contig(full, "full");
  check_cuda_contig(peer_shards, "peer_shards");
  c10::cuda::CUDAGuard guard(full.device());
  TORCH_CHECK(peer_shards.scalar_type() == at::kLong && peer_shards.numel() <= 32);
  int npieces = 0;
  const long long* tab = table_ptr(table, &npieces);
  TORCH_CHECK(reinterpret_cast<uintptr_t>(full.data_ptr()) % 16 == 0);
  const int64_t listed = listed_numel;          // world * sum of the listed pieces, known to the caller
  mb::gather_pull(full.data_ptr(), reinterpret_cast<const void* const*>(peer_shards.data_ptr<int64_t>()),
                  (int)peer_shards.numel(), tab, npieces, listed, (int)full.element_size(), opt_abort(abort),
                  shard_numel, full.numel(), stream());
}

void reduce_scatter_sumsq(const Tensor& bufs, int64_t rank, int64_t in_dtype, double scale, Tensor& out,
                          const OptTensor& sumsq, bool accumulate, const OptTensor& abort, const OptTensor& table) {
  check_cuda_contig(bufs, "bufs");
  check_cuda_contig(out, "out");
  c10::cuda::CUDAGuard guard(out.device());
  TORCH_CHECK(bufs.scalar_type() == at::kLong);
  int npieces = 0;
  const long long* tab = table_ptr(table, &npieces);
  mb::reduce_scatter_sumsq(reinterpret_cast<const void* const*>(bufs.data_ptr<int64_t>()), (int)rank,
                           (int)bufs.numel(), out.numel(), (float)scale, out.data_ptr(),
                           sumsq.has_value() ? sumsq->data_ptr<double>() : nullptr, accumulate, (int)in_dtype,
                           dtype_code(out), opt_abort(abort), tab, npieces, stream());
}

// bufs: int64 device tensor of every rank's staging address; p / m / v fp32 shards updated in place
void reduce_scatter_adamw(const Tensor& bufs, int64_t rank, int64_t in_dtype, double scale, Tensor& p, Tensor& m,
                          Tensor& v, const OptTensor& low, const OptTensor& sumsq, double lr, double beta1,
                          double beta2, double eps, double wd, int64_t step, const OptTensor& abort,
                          const OptTensor& table) {
  int npieces = 0;
  const long long* tab = table_ptr(table, &npieces);
  check_cuda_contig(bufs, "bufs");
  check_cuda_contig(p, "p");
  check_cuda_contig(m, "m");
  check_cuda_contig(v, "v");
  c10::cuda::CUDAGuard guard(p.device());
  TORCH_CHECK(bufs.scalar_type() == at::kLong && p.scalar_type() == at::kFloat && m.scalar_type() == at::kFloat &&
              v.scalar_type() == at::kFloat && m.numel() == p.numel() && v.numel() == p.numel());
  if (low.has_value()) TORCH_CHECK(low->is_contiguous() && low->numel() == p.numel());
  if (sumsq.has_value()) TORCH_CHECK(sumsq->scalar_type() == at::kDouble && sumsq->numel() == 1);
  const bool ok = mb::reduce_scatter_adamw(
      reinterpret_cast<const void* const*>(bufs.data_ptr<int64_t>()), (int)rank, (int)bufs.numel(), p.numel(),
      (float)scale, p.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(),
      low.has_value() ? low->data_ptr() : nullptr, sumsq.has_value() ? sumsq->data_ptr<double>() : nullptr, (float)lr,
      (float)beta1, (float)beta2, (float)eps, (float)wd, (int)step, (int)in_dtype,
      low.has_value() ? dtype_code(*low) : (int)in_dtype, opt_abort(abort), tab, npieces, stream());
  TORCH_CHECK(ok, "reduce_scatter_adamw: shard must be a multiple of 8 elements, 16-bit gradients, at most 8 ranks");
}

// out = sum of `world` consecutive slots of out.numel() elements each
void reduce_slots(const Tensor& slots, Tensor& out, int64_t world) {
  check_cuda_contig(slots, "slots");
  check_cuda_contig(out, "out");
  c10::cuda::CUDAGuard guard(out.device());
  TORCH_CHECK(slots.scalar_type() == out.scalar_type() && slots.numel() >= out.numel() * world);
  mb::reduce_slots(slots.data_ptr(), out.data_ptr(), out.numel(), (int)world, dtype_code(out), stream());
}

}  // namespace

// Every operator below launches kernels on the current stream.  `checked(fn)` wraps a binding so that
// a failed launch (bad configuration, a sticky error of an earlier kernel) surfaces as a Python
// exception at the call that hit it instead of at some later synchronisation point.
template <typename R, typename... A>
auto checked(R (*fn)(A...)) {
  return [fn](A... args) -> R {
    if constexpr (std::is_void_v<R>) {
      fn(args...);
      C10_CUDA_KERNEL_LAUNCH_CHECK();
    } else {
      R out = fn(args...);
      C10_CUDA_KERNEL_LAUNCH_CHECK();
      return out;
    }
  };
}

void register_cpu_ops(pybind11::module& m);      // cpu_ops.cpp
void register_cpu_bwd_ops(pybind11::module& m);  // cpu_ops_bwd.cpp

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  register_cpu_ops(m);
  register_cpu_bwd_ops(m);
  m.def("rms_norm_fwd", checked(&rms_norm_fwd));
  m.def("rms_norm_bwd", checked(&rms_norm_bwd));
  m.def("colsum", checked(&colsum));
  m.def("layer_norm_fwd", checked(&layer_norm_fwd));
  m.def("layer_norm_bwd", checked(&layer_norm_bwd));
  m.def("timestep_norm_fwd", checked(&timestep_norm_fwd));
  m.def("timestep_norm_bwd", checked(&timestep_norm_bwd));
  m.def("cema_fwd", checked(&cema_fwd));
  m.def("cema_bwd", checked(&cema_bwd));
  m.def("swiglu_fwd", checked(&swiglu_fwd));
  m.def("swiglu_bwd", checked(&swiglu_bwd));
  m.def("silu_bwd", checked(&silu_bwd));
  m.def("rotary", checked(&rotary));
  m.def("qk_rotary_fwd", checked(&qk_rotary_fwd));
  m.def("qk_rotary_bwd", checked(&qk_rotary_bwd));
  m.def("cross_entropy_fwd", checked(&cross_entropy_fwd));
  m.def("cross_entropy_bwd", checked(&cross_entropy_bwd));
  m.def("adamw_step", checked(&adamw_step));
  m.def("sum_squares", checked(&sum_squares));
  m.def("scale_by_ptr", checked(&scale_by_ptr));
  m.def("clip_coef", checked(&clip_coef));
  m.def("gemm", checked(&gemm), py::arg("A"), py::arg("B"), py::arg("out"), py::arg("bias"), py::arg("act"), py::arg("a_mn"),
        py::arg("b_mn"), py::arg("want_preact"), py::arg("out_dtype"), py::arg("mode"), py::arg("alpha"), py::arg("err"),
        py::arg("a_part_ptrs") = std::vector<int64_t>(), py::arg("a_first") = 0,
        py::arg("c_part_ptrs") = std::vector<int64_t>(), py::arg("accumulate") = false,
        py::arg("b_gather_ptrs") = std::vector<int64_t>(), py::arg("b_gather_rank") = 0, py::arg("epi_kind") = 0,
        py::arg("row_in") = py::none(), py::arg("row_in2") = py::none(), py::arg("row_out") = py::none(),
        py::arg("aux") = py::none(), py::arg("causal_off") = 0);
  m.def("gemm_gather_supported", [](int64_t M, int64_t N, int64_t K, int64_t world) {
    return mb::gemm_gather_supported((int)M, (int)N, (int)K, (int)world);
  });
  m.def("gemv_small_m", checked(&gemv_small_m));
  m.def("rfft_rows", checked(&rfft_rows), py::arg("x"), py::arg("flip"), py::arg("packed") = -1);
  m.def("irfft_rows", checked(&irfft_rows), py::arg("spec"), py::arg("L"), py::arg("packed") = -1);
  m.def("fftconv_apply", checked(&fftconv_apply), py::arg("x"), py::arg("kf"), py::arg("conj_k"), py::arg("packed") = -1);
  m.def("fftconv_dk", checked(&fftconv_dk));
  m.def("reduce_slots", checked(&reduce_slots));
  m.def("reduce_scatter_sumsq", checked(&reduce_scatter_sumsq), py::arg("bufs"), py::arg("rank"), py::arg("in_dtype"),
        py::arg("scale"), py::arg("out"), py::arg("sumsq"), py::arg("accumulate"), py::arg("abort") = py::none(),
        py::arg("table") = py::none());
  m.def("gather_pull", checked(&gather_pull), py::arg("full"), py::arg("peer_shards"), py::arg("table"),
        py::arg("listed_numel"), py::arg("abort") = py::none(), py::arg("shard_numel") = 0);
  m.def("reduce_scatter_adamw", checked(&reduce_scatter_adamw), py::arg("bufs"), py::arg("rank"), py::arg("in_dtype"),
        py::arg("scale"), py::arg("p"), py::arg("m"), py::arg("v"), py::arg("low"), py::arg("sumsq"), py::arg("lr"),
        py::arg("beta1"), py::arg("beta2"), py::arg("eps"), py::arg("wd"), py::arg("step"),
        py::arg("abort") = py::none(), py::arg("table") = py::none());
  m.def("time_sums", checked(&time_sums));
  m.def("affine_apply", checked(&affine_apply));
  m.def("dropout", checked(&dropout));
  m.def("ema_parameters_fwd", checked(&ema_parameters_fwd));
  m.def("ema_parameters_bwd", checked(&ema_parameters_bwd));
  m.def("attn_softmax_fwd", checked(&attn_softmax_fwd));
  m.def("attn_softmax_bwd", checked(&attn_softmax_bwd));
  m.def("attn_bwd_prep", checked(&attn_bwd_prep));
  m.def("decode_attention", checked(&decode_attention));
  m.def("p2p_send", checked(&p2p_send));
  m.def("p2p_recv", checked(&p2p_recv), py::arg("dst"), py::arg("local_slot"), py::arg("nbytes"), py::arg("local_flag"),
        py::arg("seq"), py::arg("remote_ack"), py::arg("counter"), py::arg("timeout_ns"), py::arg("abort"),
        py::arg("rank"), py::arg("dir"), py::arg("poison") = false);
  m.def("peer_barrier", checked(&peer_barrier));
  m.def("small_collective", checked(&small_collective));
  m.def("gemm_set_cta_pairs", [](bool on) { mb::gemm_set_cta_pairs(on); });
  m.def("gemm_pair_max_active_clusters", []() { return mb::gemm_pair_max_active_clusters(); });
  m.def("allreduce_sumsq", checked(&allreduce_sumsq), py::arg("bufs"), py::arg("rank"), py::arg("nbytes"),
        py::arg("scale"), py::arg("sumsq"), py::arg("dtype"), py::arg("abort") = py::none());
  m.attr("COMM_ABORT_WORDS") = (int)mb::kCommAbortWords;
  m.def("pinned_device_ptr", &pinned_device_ptr);
  m.def("piece_table_limit", []() { return mb::piece_table_limit(); });
}
