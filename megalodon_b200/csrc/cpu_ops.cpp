// Host (CPU) implementations of the forward passes of the operator families the reference also has on
// the CPU (TimestepNorm, SequenceNorm, ema_parameters, ema_hidden, plus the fused CEMA layer), for
// inference and data preparation on machines without a GPU.  The reference ships C++ CPU code for the same families
// (csrc/ops/timestep_norm.cc:23-450, ema_hidden.cc:15-159, ema_parameters.cc:17-188); here both are
// plain sequential scans over time, parallel over (batch, group) or (batch, feature), fp64 state.
// Gradients on CPU go through the PyTorch statements in ops/reference.py.
#include <torch/extension.h>

#include <ATen/Parallel.h>

#include <cmath>
#include <complex>
#include <tuple>
#include <vector>

namespace mb_cpu {

using torch::Tensor;

// x [B, L, H] fp32; prev_count [B] int64; prev_mean / prev_var [B, G]; gamma / beta [H]; mask [B, L] bool or
// undefined.  Returns (y, count, mean, var) with the semantics of the CUDA kernels: each step's group mean
// and variance enter the running population with weight one, padded steps give zeros and change nothing.
std::tuple<Tensor, Tensor, Tensor, Tensor> timestep_norm_fwd(const Tensor& x, const Tensor& prev_count,
                                                             const Tensor& prev_mean, const Tensor& prev_var,
                                                             const Tensor& gamma, double gamma_offset,
                                                             const Tensor& beta, const c10::optional<Tensor>& mask,
                                                             int64_t G, double eps) {
  TORCH_CHECK(!x.is_cuda() && x.dim() == 3 && x.scalar_type() == at::kFloat, "x must be a CPU fp32 [B, L, H] tensor");
  const Tensor xc = x.contiguous();
  const int64_t B = x.size(0), L = x.size(1), H = x.size(2);
  TORCH_CHECK(G > 0 && H % G == 0);
  const int64_t Dg = H / G;
  const Tensor pm = prev_mean.to(at::kDouble).contiguous(), pv = prev_var.to(at::kDouble).contiguous();
  const Tensor pc = prev_count.to(at::kLong).contiguous();
  const Tensor gm = gamma.to(at::kFloat).contiguous(), bt = beta.to(at::kFloat).contiguous();
  Tensor mk;
  if (mask.has_value()) mk = mask->to(at::kBool).contiguous();
  Tensor y = torch::empty_like(xc);
  Tensor mean_out = torch::empty({B, G}, pm.options()), var_out = torch::empty({B, G}, pm.options());
  Tensor count_out = pc.clone();
  const float* xp = xc.data_ptr<float>();
  float* yp = y.data_ptr<float>();
  const float* gp = gm.data_ptr<float>();
  const float* bp = bt.data_ptr<float>();
  const bool* mp = mk.defined() ? mk.data_ptr<bool>() : nullptr;
  const double* pmp = pm.data_ptr<double>();
  const double* pvp = pv.data_ptr<double>();
  const int64_t* pcp = pc.data_ptr<int64_t>();
  double* mo = mean_out.data_ptr<double>();
  double* vo = var_out.data_ptr<double>();
  int64_t* co = count_out.data_ptr<int64_t>();
  at::parallel_for(0, B * G, 1, [&](int64_t lo, int64_t hi) {
    for (int64_t bg = lo; bg < hi; ++bg) {
      const int64_t b = bg / G, g = bg % G;
      const double u0 = pmp[bg], v0 = pvp[bg];
      double n = (double)pcp[b];
      double s1 = n * u0, s2 = n * (v0 + u0 * u0);
      double mean = u0, var = v0;
      for (int64_t t = 0; t < L; ++t) {
        const float* row = xp + (b * L + t) * H + g * Dg;
        float* out = yp + (b * L + t) * H + g * Dg;
        if (mp != nullptr && mp[b * L + t]) {
          for (int64_t k = 0; k < Dg; ++k) out[k] = 0.f;
          continue;
        }
        double s = 0.0;
        for (int64_t k = 0; k < Dg; ++k) s += row[k];
        const double u = s / (double)Dg;
        double q = 0.0;
        for (int64_t k = 0; k < Dg; ++k) {
          const double d = row[k] - u;
          q += d * d;
        }
        const double v = q / (double)Dg;
        n += 1.0;
        s1 += u;
        s2 += v + u * u;
        mean = s1 / n;
        var = std::max(s2 / n - mean * mean, 0.0);
        const double rstd = 1.0 / std::sqrt(var + eps);
        for (int64_t k = 0; k < Dg; ++k) {
          const int64_t j = g * Dg + k;
          out[k] = (float)((row[k] - mean) * rstd * ((double)gp[j] + gamma_offset) + (double)bp[j]);
        }
      }
      mo[bg] = mean;
      vo[bg] = var;
      if (g == 0) co[b] = (int64_t)(n + 0.5);
    }
  });
  return {y, count_out, mean_out.to(prev_mean.scalar_type()), var_out.to(prev_var.scalar_type())};
}

// x [B, L, D] fp32; p [D, N] fp32; q, gamma [D, N] complex64; omega [D]; hx [B, D, N] complex64 or undefined.
// h_t = q h_{t-1} + p x_t,  y_t = Re(sum_n gamma_n h_t,n) + omega x_t.  Returns (y, h_last [B, D, N]).
std::tuple<Tensor, Tensor> cema_fwd(const Tensor& x, const Tensor& p, const Tensor& q, const Tensor& gamma,
                                    const Tensor& omega, const c10::optional<Tensor>& hx) {
  TORCH_CHECK(!x.is_cuda() && x.dim() == 3 && x.scalar_type() == at::kFloat, "x must be a CPU fp32 [B, L, D] tensor");
  const Tensor xc = x.contiguous();
  const int64_t B = x.size(0), L = x.size(1), D = x.size(2);
  const Tensor pc = p.reshape({D, -1}).to(at::kFloat).contiguous();
  const int64_t N = pc.size(1);
  const Tensor qc = q.reshape({D, N}).to(at::kComplexFloat).contiguous();
  const Tensor gc = gamma.reshape({D, N}).to(at::kComplexFloat).contiguous();
  const Tensor oc = omega.reshape({D}).to(at::kFloat).contiguous();
  Tensor hc;
  if (hx.has_value()) hc = hx->to(at::kComplexFloat).contiguous();
  Tensor y = torch::empty_like(xc);
  Tensor h_last = torch::empty({B, D, N}, qc.options());
  const float* xp = xc.data_ptr<float>();
  float* yp = y.data_ptr<float>();
  const float* pp = pc.data_ptr<float>();
  const auto* qp = qc.data_ptr<c10::complex<float>>();
  const auto* gp = gc.data_ptr<c10::complex<float>>();
  const float* op = oc.data_ptr<float>();
  const auto* hp = hc.defined() ? hc.data_ptr<c10::complex<float>>() : nullptr;
  auto* ho = h_last.data_ptr<c10::complex<float>>();
  at::parallel_for(0, B * D, 1, [&](int64_t lo, int64_t hi) {
    std::vector<std::complex<double>> h(N);
    for (int64_t bd = lo; bd < hi; ++bd) {
      const int64_t b = bd / D, d = bd % D;
      for (int64_t n = 0; n < N; ++n)
        h[n] = hp != nullptr ? std::complex<double>(hp[bd * N + n].real(), hp[bd * N + n].imag())
                             : std::complex<double>(0.0, 0.0);
      for (int64_t t = 0; t < L; ++t) {
        const double xv = xp[(b * L + t) * D + d];
        double acc = 0.0;
        for (int64_t n = 0; n < N; ++n) {
          const std::complex<double> qq(qp[d * N + n].real(), qp[d * N + n].imag());
          const std::complex<double> gg(gp[d * N + n].real(), gp[d * N + n].imag());
          h[n] = qq * h[n] + (double)pp[d * N + n] * xv;
          acc += (gg * h[n]).real();
        }
        yp[(b * L + t) * D + d] = (float)(acc + (double)op[d] * xv);
      }
      for (int64_t n = 0; n < N; ++n) ho[bd * N + n] = c10::complex<float>((float)h[n].real(), (float)h[n].imag());
    }
  });
  return {y, h_last};
}

// x [B, L, H] (or [B, H, L] when length_last) fp32; statistics over the non-padded steps per (batch, feature)
// or, with G > 0, per (batch, group of H / G features).  Padded steps give zeros.
Tensor sequence_norm_fwd(const Tensor& x, const Tensor& gamma, const Tensor& beta, const c10::optional<Tensor>& mask,
                         int64_t G, double eps, bool length_last) {
  TORCH_CHECK(!x.is_cuda() && x.dim() == 3 && x.scalar_type() == at::kFloat, "x must be a CPU fp32 3-D tensor");
  const Tensor xc = x.contiguous();
  const int64_t B = x.size(0), L = length_last ? x.size(2) : x.size(1), H = length_last ? x.size(1) : x.size(2);
  const int64_t groups = G > 0 ? G : H;
  TORCH_CHECK(H % groups == 0);
  const int64_t Dg = H / groups;
  const Tensor gm = gamma.to(at::kFloat).contiguous(), bt = beta.to(at::kFloat).contiguous();
  Tensor mk;
  if (mask.has_value()) mk = mask->to(at::kBool).contiguous();
  Tensor y = torch::empty_like(xc);
  const float* xp = xc.data_ptr<float>();
  float* yp = y.data_ptr<float>();
  const float* gp = gm.data_ptr<float>();
  const float* bp = bt.data_ptr<float>();
  const bool* mp = mk.defined() ? mk.data_ptr<bool>() : nullptr;
  auto at_ = [&](int64_t b, int64_t t, int64_t h) { return length_last ? (b * H + h) * L + t : (b * L + t) * H + h; };
  at::parallel_for(0, B * groups, 1, [&](int64_t lo, int64_t hi) {
    for (int64_t bg = lo; bg < hi; ++bg) {
      const int64_t b = bg / groups, g = bg % groups;
      double n = 0.0, s = 0.0;
      for (int64_t t = 0; t < L; ++t) {
        if (mp != nullptr && mp[b * L + t]) continue;
        n += 1.0;
        for (int64_t k = 0; k < Dg; ++k) s += xp[at_(b, t, g * Dg + k)];
      }
      const double cnt = std::max(n, 1.0) * (double)Dg;
      const double mean = s / cnt;
      double q = 0.0;
      for (int64_t t = 0; t < L; ++t) {
        if (mp != nullptr && mp[b * L + t]) continue;
        for (int64_t k = 0; k < Dg; ++k) {
          const double d = xp[at_(b, t, g * Dg + k)] - mean;
          q += d * d;
        }
      }
      const double rstd = 1.0 / std::sqrt(q / cnt + eps);
      for (int64_t t = 0; t < L; ++t) {
        const bool pad = mp != nullptr && mp[b * L + t];
        for (int64_t k = 0; k < Dg; ++k) {
          const int64_t h = g * Dg + k;
          const int64_t i = at_(b, t, h);
          yp[i] = pad ? 0.f : (float)((xp[i] - mean) * rstd * (double)gp[h] + (double)bp[h]);
        }
      }
    }
  });
  return y;
}

// k[d, j] = Re sum_n p gamma q^j (j < L);  b[b, d, j] = Re sum_n gamma q^(j+1) h (only with hx).
// p [D, N] real, q / gamma [D, N] complex, hx [B, D, N] complex or undefined.
std::tuple<Tensor, c10::optional<Tensor>> ema_parameters_fwd(const Tensor& p, const Tensor& q, const Tensor& gamma,
                                                             const c10::optional<Tensor>& hx, int64_t L) {
  TORCH_CHECK(!p.is_cuda());
  const int64_t D = p.size(0);
  const Tensor pc = p.reshape({D, -1}).to(at::kDouble).contiguous();
  const int64_t N = pc.size(1);
  const Tensor qc = q.reshape({D, N}).to(at::kComplexDouble).contiguous();
  const Tensor gc = gamma.reshape({D, N}).to(at::kComplexDouble).contiguous();
  Tensor hc;
  int64_t B = 0;
  if (hx.has_value()) {
    hc = hx->to(at::kComplexDouble).contiguous();
    B = hc.size(0);
  }
  Tensor k = torch::empty({D, L}, pc.options().dtype(at::kFloat));
  Tensor bias;
  if (B > 0) bias = torch::empty({B, D, L}, k.options());
  const double* pp = pc.data_ptr<double>();
  const auto* qp = qc.data_ptr<c10::complex<double>>();
  const auto* gp = gc.data_ptr<c10::complex<double>>();
  const auto* hp = hc.defined() ? hc.data_ptr<c10::complex<double>>() : nullptr;
  float* kp = k.data_ptr<float>();
  float* bp = bias.defined() ? bias.data_ptr<float>() : nullptr;
  at::parallel_for(0, D, 1, [&](int64_t lo, int64_t hi) {
    std::vector<std::complex<double>> pw(N);
    for (int64_t d = lo; d < hi; ++d) {
      for (int64_t n = 0; n < N; ++n) pw[n] = {1.0, 0.0};        // q^j
      for (int64_t j = 0; j < L; ++j) {
        double acc = 0.0;
        for (int64_t n = 0; n < N; ++n) {
          const std::complex<double> g(gp[d * N + n].real(), gp[d * N + n].imag());
          acc += (pp[d * N + n] * g * pw[n]).real();
        }
        kp[d * L + j] = (float)acc;
        for (int64_t n = 0; n < N; ++n)
          pw[n] *= std::complex<double>(qp[d * N + n].real(), qp[d * N + n].imag());
        // pw now holds q^(j+1): the power the carried state is multiplied by at output j
        for (int64_t b = 0; b < B; ++b) {
          double ab = 0.0;
          for (int64_t n = 0; n < N; ++n) {
            const std::complex<double> g(gp[d * N + n].real(), gp[d * N + n].imag());
            const auto& hh = hp[(b * D + d) * N + n];
            ab += (g * pw[n] * std::complex<double>(hh.real(), hh.imag())).real();
          }
          bp[(b * D + d) * L + j] = (float)ab;
        }
      }
    }
  });
  if (B > 0) return {k, bias};
  return {k, c10::nullopt};
}

// last state h' = p sum_j q^(L-1-j) x_j + q^L h;  x [B, D, L] fp32 -> [B, D, N] complex64
Tensor ema_hidden_fwd(const Tensor& x, const Tensor& p, const Tensor& q, const c10::optional<Tensor>& hx) {
  TORCH_CHECK(!x.is_cuda() && x.dim() == 3);
  const Tensor xc = x.to(at::kFloat).contiguous();
  const int64_t B = x.size(0), D = x.size(1), L = x.size(2);
  const Tensor pc = p.reshape({D, -1}).to(at::kDouble).contiguous();
  const int64_t N = pc.size(1);
  const Tensor qc = q.reshape({D, N}).to(at::kComplexDouble).contiguous();
  Tensor hc;
  if (hx.has_value()) hc = hx->to(at::kComplexDouble).contiguous();
  Tensor out = torch::empty({B, D, N}, xc.options().dtype(at::kComplexFloat));
  const float* xp = xc.data_ptr<float>();
  const double* pp = pc.data_ptr<double>();
  const auto* qp = qc.data_ptr<c10::complex<double>>();
  const auto* hp = hc.defined() ? hc.data_ptr<c10::complex<double>>() : nullptr;
  auto* op = out.data_ptr<c10::complex<float>>();
  at::parallel_for(0, B * D, 1, [&](int64_t lo, int64_t hi) {
    for (int64_t bd = lo; bd < hi; ++bd) {
      const int64_t d = bd % D;
      for (int64_t n = 0; n < N; ++n) {
        const std::complex<double> qq(qp[d * N + n].real(), qp[d * N + n].imag());
        std::complex<double> h = hp != nullptr ? std::complex<double>(hp[bd * N + n].real(), hp[bd * N + n].imag())
                                               : std::complex<double>(0.0, 0.0);
        for (int64_t t = 0; t < L; ++t) h = qq * h + pp[d * N + n] * (double)xp[bd * L + t];
        op[bd * N + n] = c10::complex<float>((float)h.real(), (float)h.imag());
      }
    }
  });
  return out;
}

}  // namespace mb_cpu

void register_cpu_ops(pybind11::module& m) {
  m.def("cpu_timestep_norm_fwd", &mb_cpu::timestep_norm_fwd);
  m.def("cpu_cema_fwd", &mb_cpu::cema_fwd);
  m.def("cpu_sequence_norm_fwd", &mb_cpu::sequence_norm_fwd);
  m.def("cpu_ema_parameters_fwd", &mb_cpu::ema_parameters_fwd);
  m.def("cpu_ema_hidden_fwd", &mb_cpu::ema_hidden_fwd);
}
