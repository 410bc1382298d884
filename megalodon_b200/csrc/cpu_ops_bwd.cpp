// Host (CPU) backward passes of TimestepNorm, SequenceNorm, ema_parameters and ema_hidden, so that the
// CPU gradients are not only the PyTorch statements of ops/reference.py (the reference ships C++ CPU
// backward code for the same families: csrc/ops/timestep_norm.cc:318-450, sequence_norm.cc,
// ema_parameters.cc:119-188, ema_hidden.cc:15-159).  Sequential scans over time in fp64, parallel over
// (batch, group) or (feature); written from the recurrences, not from the reference's loops.
#include <torch/extension.h>

#include <ATen/Parallel.h>

#include <cmath>
#include <complex>
#include <tuple>
#include <vector>

namespace mb_cpu {

using torch::Tensor;
using cdouble = std::complex<double>;

// Grouped TimestepNorm.  dy [B, L, H], dmean / dvar [B, G] (gradients of the returned statistics, may be
// undefined), x [B, L, H] fp32, prev_count [B], prev_mean / prev_var [B, G], gamma [H] (+ gamma_offset),
// mask [B, L] or undefined.  Returns (dx, dprev_mean, dprev_var, dgamma, dbeta).
//
// Forward per (b, g): the step's group mean gu and variance gv enter the running population (n, u, v)
// with weight one: n' = n + 1, u' = u + (gu - u) / n', v' = (n v + gv) / n' + n (gu - u)^2 / n'^2;
// y = (x - u') r gamma + beta with r = 1 / sqrt(v' + eps).  The backward pass walks the steps in
// reverse with the adjoints (ub, vb) of the running (u, v).
std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> timestep_norm_bwd(
    const Tensor& dy, const c10::optional<Tensor>& dmean, const c10::optional<Tensor>& dvar, const Tensor& x,
    const Tensor& prev_count, const Tensor& prev_mean, const Tensor& prev_var, const Tensor& gamma,
    double gamma_offset, const c10::optional<Tensor>& mask, int64_t G, double eps) {
  TORCH_CHECK(!x.is_cuda() && x.dim() == 3 && x.scalar_type() == at::kFloat, "x must be a CPU fp32 [B, L, H] tensor");
  const Tensor xc = x.contiguous(), dyc = dy.to(at::kFloat).contiguous();
  const int64_t B = x.size(0), L = x.size(1), H = x.size(2);
  TORCH_CHECK(G > 0 && H % G == 0);
  const int64_t Dg = H / G;
  const Tensor pm = prev_mean.to(at::kDouble).contiguous(), pv = prev_var.to(at::kDouble).contiguous();
  const Tensor pc = prev_count.to(at::kLong).contiguous();
  const Tensor gm = gamma.to(at::kDouble).contiguous();
  Tensor mk, dm, dv;
  if (mask.has_value()) mk = mask->to(at::kBool).contiguous();
  if (dmean.has_value()) dm = dmean->to(at::kDouble).contiguous();
  if (dvar.has_value()) dv = dvar->to(at::kDouble).contiguous();
  Tensor dx = torch::zeros_like(xc);
  auto f64 = pm.options();
  Tensor dpm = torch::zeros({B, G}, f64), dpv = torch::zeros({B, G}, f64);
  Tensor dgam_b = torch::zeros({B, H}, f64), dbet_b = torch::zeros({B, H}, f64);
  const float* xp = xc.data_ptr<float>();
  const float* gp = dyc.data_ptr<float>();
  float* dxp = dx.data_ptr<float>();
  const double* gam = gm.data_ptr<double>();
  const bool* mp = mk.defined() ? mk.data_ptr<bool>() : nullptr;
  at::parallel_for(0, B * G, 1, [&](int64_t lo, int64_t hi) {
    std::vector<double> cu(L), cr(L), gux(L), cn(L);
    for (int64_t bg = lo; bg < hi; ++bg) {
      const int64_t b = bg / G, g = bg % G;
      // forward statistics, kept per step
      double n = (double)pc.data_ptr<int64_t>()[b], u = pm.data_ptr<double>()[bg], v = pv.data_ptr<double>()[bg];
      for (int64_t t = 0; t < L; ++t) {
        cn[t] = -1.0;
        if (mp != nullptr && mp[b * L + t]) continue;
        const float* row = xp + (b * L + t) * H + g * Dg;
        double s = 0.0;
        for (int64_t k = 0; k < Dg; ++k) s += row[k];
        const double gu = s / (double)Dg;
        double q = 0.0;
        for (int64_t k = 0; k < Dg; ++k) q += (row[k] - gu) * (row[k] - gu);
        const double gv = q / (double)Dg;
        const double n1 = n + 1.0, c1 = n / n1, c2 = 1.0 / n1, d = gu - u;
        v = c1 * v + c2 * gv + c1 * c2 * d * d;
        u = u + c2 * d;
        n = n1;
        cu[t] = u; cr[t] = 1.0 / std::sqrt(v + eps); gux[t] = gu; cn[t] = n;
      }
      double ub = dm.defined() ? dm.data_ptr<double>()[bg] : 0.0;
      double vb = dv.defined() ? dv.data_ptr<double>()[bg] : 0.0;
      double* dga = dgam_b.data_ptr<double>() + b * H + g * Dg;
      double* dbe = dbet_b.data_ptr<double>() + b * H + g * Dg;
      // mean of the population before step t: the previous unmasked step's, or the carried one
      std::vector<double> before(L);
      double last = pm.data_ptr<double>()[bg];
      for (int64_t t = 0; t < L; ++t) {
        before[t] = last;
        if (cn[t] > 0.0) last = cu[t];
      }
      for (int64_t t = L - 1; t >= 0; --t) {
        if (cn[t] < 0.0) continue;
        const float* row = xp + (b * L + t) * H + g * Dg;
        const float* grow = gp + (b * L + t) * H + g * Dg;
        float* drow = dxp + (b * L + t) * H + g * Dg;
        const double m0 = cn[t], c1 = (m0 - 1.0) / m0, c2 = 1.0 / m0, r = cr[t], um = cu[t], ux = gux[t];
        double ds = 0.0, db = 0.0;
        for (int64_t k = 0; k < Dg; ++k) {
          const double w = gam[g * Dg + k] + gamma_offset, gy = grow[k];
          ds += gy * (row[k] - um) * w;
          db += gy * w;
          dga[k] += gy * (row[k] - um) * r;
          dbe[k] += gy;
        }
        const double du = ub - r * db, dvv = vb - 0.5 * r * r * r * ds;
        const double delta = ux - before[t];
        const double dux = c2 * du + 2.0 * c1 * c2 * dvv * delta, dvx = c2 * dvv;
        for (int64_t k = 0; k < Dg; ++k) {
          const double w = gam[g * Dg + k] + gamma_offset;
          drow[k] = (float)(grow[k] * r * w + (dux + 2.0 * dvx * (row[k] - ux)) / (double)Dg);
        }
        ub = c1 * du - 2.0 * c1 * c2 * dvv * delta;
        vb = c1 * dvv;
      }
      dpm.data_ptr<double>()[bg] = ub;
      dpv.data_ptr<double>()[bg] = vb;
    }
  });
  return {dx, dpm.to(at::kFloat), dpv.to(at::kFloat), dgam_b.sum(0).to(at::kFloat), dbet_b.sum(0).to(at::kFloat)};
}

// SequenceNorm (whole-sequence statistics per (batch, feature) or, with G > 0, per (batch, group)), layouts
// [B, L, H] and [B, H, L].  With u, r the mean and reciprocal standard deviation over the cnt unmasked values
// of a (batch, group):  dx = r gamma dy + (du + 2 (x - u) dv) / cnt,  du = -r sum(dy gamma),
// dv = -r^3 / 2 sum(dy gamma (x - u)).  Returns (dx, dgamma [H], dbeta [H]).
std::tuple<Tensor, Tensor, Tensor> sequence_norm_bwd(const Tensor& dy, const Tensor& x, const Tensor& gamma,
                                                     const c10::optional<Tensor>& mask, int64_t G, double eps,
                                                     bool length_last) {
  TORCH_CHECK(!x.is_cuda() && x.dim() == 3 && x.scalar_type() == at::kFloat, "x must be a CPU fp32 3-D tensor");
  const Tensor xc = x.contiguous(), dyc = dy.to(at::kFloat).contiguous();
  const int64_t B = x.size(0), L = length_last ? x.size(2) : x.size(1), H = length_last ? x.size(1) : x.size(2);
  const int64_t groups = G > 0 ? G : H;
  TORCH_CHECK(H % groups == 0);
  const int64_t Dg = H / groups;
  const Tensor gm = gamma.to(at::kDouble).contiguous();
  Tensor mk;
  if (mask.has_value()) mk = mask->to(at::kBool).contiguous();
  Tensor dx = torch::zeros_like(xc);
  Tensor dgam_b = torch::zeros({B, H}, gm.options()), dbet_b = torch::zeros({B, H}, gm.options());
  const float* xp = xc.data_ptr<float>();
  const float* gp = dyc.data_ptr<float>();
  float* dxp = dx.data_ptr<float>();
  const double* gam = gm.data_ptr<double>();
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
      const double u = s / cnt;
      double q = 0.0;
      for (int64_t t = 0; t < L; ++t) {
        if (mp != nullptr && mp[b * L + t]) continue;
        for (int64_t k = 0; k < Dg; ++k) {
          const double d = xp[at_(b, t, g * Dg + k)] - u;
          q += d * d;
        }
      }
      const double r = 1.0 / std::sqrt(q / cnt + eps);
      double sg = 0.0, sgx = 0.0;
      for (int64_t t = 0; t < L; ++t) {
        if (mp != nullptr && mp[b * L + t]) continue;
        for (int64_t k = 0; k < Dg; ++k) {
          const int64_t h = g * Dg + k, i = at_(b, t, h);
          const double gy = gp[i], xm = xp[i] - u;
          sg += gy * gam[h];
          sgx += gy * gam[h] * xm;
          dgam_b.data_ptr<double>()[b * H + h] += gy * xm * r;
          dbet_b.data_ptr<double>()[b * H + h] += gy;
        }
      }
      const double du = -r * sg, dv = -0.5 * r * r * r * sgx;
      for (int64_t t = 0; t < L; ++t) {
        if (mp != nullptr && mp[b * L + t]) continue;
        for (int64_t k = 0; k < Dg; ++k) {
          const int64_t h = g * Dg + k, i = at_(b, t, h);
          dxp[i] = (float)(gp[i] * r * gam[h] + (du + 2.0 * (xp[i] - u) * dv) / cnt);
        }
      }
    }
  });
  return {dx, dgam_b.sum(0).to(at::kFloat), dbet_b.sum(0).to(at::kFloat)};
}

static inline cdouble cd(const c10::complex<double>& z) { return {z.real(), z.imag()}; }

// Gradients of k[d, j] = Re sum_n p gamma q^j and bias[b, d, j] = Re sum_n gamma q^(j+1) h w.r.t. p (real),
// q, gamma and h (complex).  For a real loss and a complex parameter z the returned tensor is
// dL/dRe(z) + i dL/dIm(z) (PyTorch's convention), which for L = Re(c z) is conj(c).
// dk [D, L], dbias [B, D, L] or undefined.  Returns (dp [D, N], dq, dgamma [D, N] complex, dh [B, D, N] or undefined).
std::tuple<Tensor, Tensor, Tensor, c10::optional<Tensor>> ema_parameters_bwd(
    const Tensor& dk, const c10::optional<Tensor>& dbias, const Tensor& p, const Tensor& q, const Tensor& gamma,
    const c10::optional<Tensor>& hx) {
  TORCH_CHECK(!p.is_cuda());
  const int64_t D = p.size(0), L = dk.size(-1);
  const Tensor pc = p.reshape({D, -1}).to(at::kDouble).contiguous();
  const int64_t N = pc.size(1);
  const Tensor qc = q.reshape({D, N}).to(at::kComplexDouble).contiguous();
  const Tensor gc = gamma.reshape({D, N}).to(at::kComplexDouble).contiguous();
  const Tensor dkc = dk.to(at::kDouble).contiguous();
  Tensor hc, dbc;
  int64_t B = 0;
  if (hx.has_value() && dbias.has_value()) {
    hc = hx->to(at::kComplexDouble).contiguous();
    dbc = dbias->to(at::kDouble).contiguous();
    B = hc.size(0);
  }
  auto c128 = qc.options();
  Tensor dp = torch::zeros({D, N}, pc.options()), dq = torch::zeros({D, N}, c128), dg = torch::zeros({D, N}, c128);
  Tensor dh;
  if (B > 0) dh = torch::zeros({B, D, N}, c128);
  const double* pp = pc.data_ptr<double>();
  const auto* qp = qc.data_ptr<c10::complex<double>>();
  const auto* gp = gc.data_ptr<c10::complex<double>>();
  at::parallel_for(0, D * N, 1, [&](int64_t lo, int64_t hi) {
    for (int64_t dn = lo; dn < hi; ++dn) {
      const int64_t d = dn / N;
      const cdouble qq = cd(qp[dn]), gg = cd(gp[dn]);
      const double pv = pp[dn];
      // S1 = sum_j dk_j j q^(j-1), S2 = sum_j dk_j q^j
      cdouble s1 = 0.0, s2 = 0.0, pw = 1.0, pw_prev = 0.0;
      const double* dkr = dkc.data_ptr<double>() + d * L;
      for (int64_t j = 0; j < L; ++j) {
        s2 += dkr[j] * pw;
        if (j > 0) s1 += dkr[j] * (double)j * pw_prev;
        pw_prev = pw;
        pw *= qq;
      }
      double dpv = (s2 * gg).real();
      cdouble dqv = std::conj(s1 * pv * gg), dgv = std::conj(s2 * pv);
      for (int64_t b = 0; b < B; ++b) {
        const cdouble hh = cd(hc.data_ptr<c10::complex<double>>()[(b * D + d) * N + (dn % N)]);
        const double* dbr = dbc.data_ptr<double>() + (b * D + d) * L;
        // T1 = sum_j db_j (j+1) q^j, T2 = sum_j db_j q^(j+1)
        cdouble t1 = 0.0, t2 = 0.0, w = 1.0;
        for (int64_t j = 0; j < L; ++j) {
          t1 += dbr[j] * (double)(j + 1) * w;
          w *= qq;
          t2 += dbr[j] * w;
        }
        dqv += std::conj(t1 * gg * hh);
        dgv += std::conj(t2 * hh);
        const cdouble dhv = std::conj(t2 * gg);
        dh.data_ptr<c10::complex<double>>()[(b * D + d) * N + (dn % N)] = c10::complex<double>(dhv.real(), dhv.imag());
      }
      dp.data_ptr<double>()[dn] = dpv;
      dq.data_ptr<c10::complex<double>>()[dn] = c10::complex<double>(dqv.real(), dqv.imag());
      dg.data_ptr<c10::complex<double>>()[dn] = c10::complex<double>(dgv.real(), dgv.imag());
    }
  });
  c10::optional<Tensor> dh_out;
  if (B > 0) dh_out = dh.to(at::kComplexFloat);
  return {dp.to(at::kFloat), dq.to(at::kComplexFloat), dg.to(at::kComplexFloat), dh_out};
}

// Gradients of the last state h' = p sum_j q^(L-1-j) x_j + q^L h.  dh_out [B, D, N] complex (PyTorch convention:
// dL/dRe + i dL/dIm), x [B, D, L].  Returns (dx [B, D, L], dp [D, N], dq [D, N] complex, dh [B, D, N] or undefined).
std::tuple<Tensor, Tensor, Tensor, c10::optional<Tensor>> ema_hidden_bwd(const Tensor& dh_out, const Tensor& x,
                                                                         const Tensor& p, const Tensor& q,
                                                                         const c10::optional<Tensor>& hx) {
  TORCH_CHECK(!x.is_cuda() && x.dim() == 3);
  const Tensor xc = x.to(at::kDouble).contiguous();
  const int64_t B = x.size(0), D = x.size(1), L = x.size(2);
  const Tensor pc = p.reshape({D, -1}).to(at::kDouble).contiguous();
  const int64_t N = pc.size(1);
  const Tensor qc = q.reshape({D, N}).to(at::kComplexDouble).contiguous();
  const Tensor gc = dh_out.to(at::kComplexDouble).contiguous();
  Tensor hc;
  if (hx.has_value()) hc = hx->to(at::kComplexDouble).contiguous();
  Tensor dx = torch::zeros({B, D, L}, xc.options());
  Tensor dp_b = torch::zeros({B, D, N}, xc.options()), dq_b = torch::zeros({B, D, N}, qc.options());
  Tensor dh;
  if (hc.defined()) dh = torch::zeros({B, D, N}, qc.options());
  at::parallel_for(0, B * D, 1, [&](int64_t lo, int64_t hi) {
    for (int64_t bd = lo; bd < hi; ++bd) {
      const int64_t d = bd % D;
      const double* xr = xc.data_ptr<double>() + bd * L;
      double* dxr = dx.data_ptr<double>() + bd * L;
      for (int64_t n = 0; n < N; ++n) {
        const cdouble qq = cd(qc.data_ptr<c10::complex<double>>()[d * N + n]);
        const double pv = pc.data_ptr<double>()[d * N + n];
        // with c = conj(dh_out): L = Re(c h') up to a constant, so dL/dx_j = Re(c p q^(L-1-j)), ...
        const cdouble c = std::conj(cd(gc.data_ptr<c10::complex<double>>()[bd * N + n]));
        cdouble pw = 1.0, pw_prev = 0.0, sx = 0.0, sxd = 0.0;     // q^m, q^(m-1) with m = L-1-j
        for (int64_t j = L - 1; j >= 0; --j) {
          const int64_t m = L - 1 - j;
          dxr[j] += (c * pv * pw).real();
          sx += xr[j] * pw;
          if (m > 0) sxd += xr[j] * (double)m * pw_prev;
          pw_prev = pw;
          pw *= qq;
        }
        // pw = q^L, pw_prev = q^(L-1)
        const cdouble h0 = hc.defined() ? cd(hc.data_ptr<c10::complex<double>>()[bd * N + n]) : cdouble(0.0);
        dp_b.data_ptr<double>()[bd * N + n] = (c * sx).real();
        const cdouble dqv = std::conj(c * (pv * sxd + (double)L * pw_prev * h0));
        dq_b.data_ptr<c10::complex<double>>()[bd * N + n] = c10::complex<double>(dqv.real(), dqv.imag());
        if (dh.defined()) {
          const cdouble dhv = std::conj(c * pw);
          dh.data_ptr<c10::complex<double>>()[bd * N + n] = c10::complex<double>(dhv.real(), dhv.imag());
        }
      }
    }
  });
  c10::optional<Tensor> dh_o;
  if (dh.defined()) dh_o = dh.to(at::kComplexFloat);
  return {dx.to(at::kFloat), dp_b.sum(0).to(at::kFloat), dq_b.sum(0).to(at::kComplexFloat), dh_o};
}

// Backward of the fused complex-EMA layer (cpu_ops.cpp: cema_fwd): h_t = q h_{t-1} + p x_t,
// y_t = Re(sum_n gamma_n h_t,n) + omega x_t, last state h_L returned.  dy [B, L, D]; dh_last [B, D, N] complex
// or undefined; x [B, L, D] fp32; p [D, N]; q, gamma [D, N] complex64; omega [D]; hx [B, D, N] or undefined.
// Gradients of complex tensors are d/dRe + i d/dIm, as autograd hands them around.  The adjoint of the state
// obeys lambda_t = conj(gamma) dy_t + conj(q) lambda_{t+1} (lambda_L also takes dh_last), and
//   dx_t = sum_n p_n Re(lambda_t,n) + omega dy_t      dp_n = sum_t x_t Re(lambda_t,n)
//   dq_n = sum_t lambda_t,n conj(h_{t-1},n)           dgamma_n = sum_t dy_t conj(h_t,n)
//   domega = sum_t dy_t x_t                           dhx_n = conj(q_n) lambda_1,n
// The states of one (batch, feature) row are kept from a forward sweep (L * N complex doubles).
// Returns (dx, dp, dq, dgamma, domega, dhx or undefined).
std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor, c10::optional<Tensor>> cema_bwd(
    const Tensor& dy, const c10::optional<Tensor>& dh_last, const Tensor& x, const Tensor& p, const Tensor& q,
    const Tensor& gamma, const Tensor& omega, const c10::optional<Tensor>& hx) {
  TORCH_CHECK(!x.is_cuda() && x.dim() == 3 && x.scalar_type() == at::kFloat, "x must be a CPU fp32 [B, L, D] tensor");
  const Tensor xc = x.contiguous(), dyc = dy.to(at::kFloat).contiguous();
  const int64_t B = x.size(0), L = x.size(1), D = x.size(2);
  const Tensor pc = p.reshape({D, -1}).to(at::kDouble).contiguous();
  const int64_t N = pc.size(1);
  const Tensor qc = q.reshape({D, N}).to(at::kComplexDouble).contiguous();
  const Tensor gc = gamma.reshape({D, N}).to(at::kComplexDouble).contiguous();
  const Tensor oc = omega.reshape({D}).to(at::kDouble).contiguous();
  Tensor hc, gl;
  if (hx.has_value()) hc = hx->to(at::kComplexDouble).contiguous();
  if (dh_last.has_value()) gl = dh_last->to(at::kComplexDouble).contiguous();
  Tensor dx = torch::empty({B, L, D}, xc.options());
  Tensor dp = torch::zeros({D, N}, pc.options());
  Tensor dq = torch::zeros({D, N}, qc.options());
  Tensor dg = torch::zeros({D, N}, qc.options());
  Tensor dom = torch::zeros({D}, oc.options());
  Tensor dhx;
  if (hc.defined()) dhx = torch::empty({B, D, N}, qc.options());
  const float* xp = xc.data_ptr<float>();
  const float* dyp = dyc.data_ptr<float>();
  float* dxp = dx.data_ptr<float>();
  const double* pp = pc.data_ptr<double>();
  const auto* qp = reinterpret_cast<const cdouble*>(qc.data_ptr<c10::complex<double>>());
  const auto* gp = reinterpret_cast<const cdouble*>(gc.data_ptr<c10::complex<double>>());
  const double* op = oc.data_ptr<double>();
  const cdouble* hp = hc.defined() ? reinterpret_cast<const cdouble*>(hc.data_ptr<c10::complex<double>>()) : nullptr;
  const cdouble* glp = gl.defined() ? reinterpret_cast<const cdouble*>(gl.data_ptr<c10::complex<double>>()) : nullptr;
  double* dpp = dp.data_ptr<double>();
  auto* dqp = reinterpret_cast<cdouble*>(dq.data_ptr<c10::complex<double>>());
  auto* dgp = reinterpret_cast<cdouble*>(dg.data_ptr<c10::complex<double>>());
  double* domp = dom.data_ptr<double>();
  cdouble* dhp = dhx.defined() ? reinterpret_cast<cdouble*>(dhx.data_ptr<c10::complex<double>>()) : nullptr;
  // one feature per task: its parameter gradients are summed over the batch without races
  at::parallel_for(0, D, 1, [&](int64_t lo, int64_t hi) {
    std::vector<cdouble> hist((L + 1) * N), lam(N);
    for (int64_t d = lo; d < hi; ++d) {
      for (int64_t b = 0; b < B; ++b) {
        const int64_t bd = b * D + d;
        for (int64_t n = 0; n < N; ++n) hist[n] = hp != nullptr ? hp[bd * N + n] : cdouble(0.0, 0.0);
        for (int64_t t = 0; t < L; ++t) {
          const double xv = xp[(b * L + t) * D + d];
          for (int64_t n = 0; n < N; ++n)
            hist[(t + 1) * N + n] = qp[d * N + n] * hist[t * N + n] + pp[d * N + n] * xv;
        }
        for (int64_t n = 0; n < N; ++n) lam[n] = glp != nullptr ? glp[bd * N + n] : cdouble(0.0, 0.0);
        for (int64_t t = L - 1; t >= 0; --t) {
          const double g = dyp[(b * L + t) * D + d];
          const double xv = xp[(b * L + t) * D + d];
          double acc = op[d] * g;
          for (int64_t n = 0; n < N; ++n) {
            const int64_t i = d * N + n;
            lam[n] += std::conj(gp[i]) * g;                       // lambda_{t+1}: adjoint of h_{t+1} (1-based)
            acc += pp[i] * lam[n].real();
            dpp[i] += xv * lam[n].real();
            dqp[i] += lam[n] * std::conj(hist[t * N + n]);
            dgp[i] += g * std::conj(hist[(t + 1) * N + n]);
            lam[n] = std::conj(qp[i]) * lam[n];                   // carried to the previous step
          }
          dxp[(b * L + t) * D + d] = (float)acc;
          domp[d] += g * xv;
        }
        if (dhp != nullptr)
          for (int64_t n = 0; n < N; ++n) dhp[bd * N + n] = lam[n];
      }
    }
  });
  c10::optional<Tensor> dhx_o;
  if (dhx.defined()) dhx_o = dhx.to(at::kComplexFloat);
  return {dx, dp.to(at::kFloat), dq.to(at::kComplexFloat), dg.to(at::kComplexFloat), dom.to(at::kFloat), dhx_o};
}

}  // namespace mb_cpu

void register_cpu_bwd_ops(pybind11::module& m) {
  m.def("cpu_cema_bwd", &mb_cpu::cema_bwd);
  m.def("cpu_timestep_norm_bwd", &mb_cpu::timestep_norm_bwd);
  m.def("cpu_sequence_norm_bwd", &mb_cpu::sequence_norm_bwd);
  m.def("cpu_ema_parameters_bwd", &mb_cpu::ema_parameters_bwd);
  m.def("cpu_ema_hidden_bwd", &mb_cpu::ema_hidden_bwd);
}
