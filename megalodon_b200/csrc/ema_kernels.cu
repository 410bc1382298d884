// Stand-alone CEMA coefficient operators (API parity with the reference's
// `ema_parameters_fwd/bwd`, csrc/ops/ema_parameters_kernel.cu): the convolution
// kernel k[d, j] = Re sum_n p gamma q^j and the carried-state bias
// b[b, d, j] = Re sum_n gamma q^(j+1) h, with their gradients.  The model's hot
// path does not use them (the fused scan in cema_kernels.cu needs neither); they
// serve callers that want the explicit kernel, e.g. `fftconv`.
//
// q^j is evaluated as exp(j log q) per term, so no power table is stored.
#include "common.cuh"
#include "kernels.h"

namespace mb {
namespace {

__device__ __forceinline__ cfloat cexp_scaled(cfloat logq, float j) {
  const float mag = __expf(logq.re * j);
  float s, c;
  sincosf(logq.im * j, &s, &c);
  return {mag * c, mag * s};
}

// one thread per (d, j)
__global__ void ema_weight_fwd_kernel(const float* __restrict__ p, const cfloat* __restrict__ logq,
                                      const cfloat* __restrict__ gamma, float* __restrict__ k, int D, int N, int L) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)D * L) return;
  const int d = (int)(i / L), j = (int)(i % L);
  float acc = 0.f;
  for (int n = 0; n < N; ++n) {
    const cfloat e = cexp_scaled(logq[d * N + n], (float)j);
    const cfloat g = gamma[d * N + n];
    acc += p[d * N + n] * (g.re * e.re - g.im * e.im);
  }
  k[i] = acc;
}

// one thread per (b, d, j)
__global__ void ema_bias_fwd_kernel(const cfloat* __restrict__ logq, const cfloat* __restrict__ gamma,
                                    const cfloat* __restrict__ h, float* __restrict__ bias, int B, int D, int N,
                                    int L) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)B * D * L) return;
  const int j = (int)(i % L);
  const long long bd = i / L;
  const int d = (int)(bd % D);
  float acc = 0.f;
  for (int n = 0; n < N; ++n) {
    const cfloat e = cexp_scaled(logq[d * N + n], (float)(j + 1));
    const cfloat gh = cmul(gamma[d * N + n], h[bd * N + n]);
    acc += gh.re * e.re - gh.im * e.im;
  }
  bias[i] = acc;
}

// one CTA per feature d
__global__ void ema_params_bwd_kernel(const float* __restrict__ dk, const float* __restrict__ dbias,
                                      const float* __restrict__ p, const cfloat* __restrict__ logq,
                                      const cfloat* __restrict__ gamma, const cfloat* __restrict__ h,
                                      float* __restrict__ dp, cfloat* __restrict__ dq, cfloat* __restrict__ dgamma,
                                      cfloat* __restrict__ dh, int B, int D, int N, int L) {
  __shared__ float scratch[32];
  const int d = blockIdx.x;
  for (int n = 0; n < N; ++n) {
    const cfloat lq = logq[d * N + n];
    const cfloat g = gamma[d * N + n];
    const float pn = p[d * N + n];
    // S1 = sum_j dk_j j q^(j-1),  S2 = sum_j dk_j q^j
    cfloat s1 = {0.f, 0.f}, s2 = {0.f, 0.f};
    if (dk != nullptr) {
      for (int j = threadIdx.x; j < L; j += blockDim.x) {
        const float w = dk[(long long)d * L + j];
        const cfloat e2 = cexp_scaled(lq, (float)j);
        s2.re += w * e2.re;
        s2.im += w * e2.im;
        if (j > 0) {
          const cfloat e1 = cexp_scaled(lq, (float)(j - 1));
          s1.re += w * j * e1.re;
          s1.im += w * j * e1.im;
        }
      }
    }
    s1.re = block_sum(s1.re, scratch);
    s1.im = block_sum(s1.im, scratch);
    s2.re = block_sum(s2.re, scratch);
    s2.im = block_sum(s2.im, scratch);
    float out_dp = s2.re * g.re - s2.im * g.im;                 // Re(S2 gamma)
    cfloat pg = {pn * g.re, pn * g.im};
    cfloat out_dq = cconj(cmul(s1, pg));                        // conj(S1 p gamma)
    cfloat out_dg = {s2.re * pn, -s2.im * pn};                  // conj(S2 p)
    if (dbias != nullptr && h != nullptr) {
      for (int b = 0; b < B; ++b) {
        const long long bd = (long long)b * D + d;
        cfloat t1 = {0.f, 0.f}, t2 = {0.f, 0.f};                // T1 = sum db (j+1) q^j, T2 = sum db q^(j+1)
        for (int j = threadIdx.x; j < L; j += blockDim.x) {
          const float w = dbias[bd * L + j];
          const cfloat e1 = cexp_scaled(lq, (float)j);
          const cfloat e2 = cexp_scaled(lq, (float)(j + 1));
          t1.re += w * (j + 1) * e1.re;
          t1.im += w * (j + 1) * e1.im;
          t2.re += w * e2.re;
          t2.im += w * e2.im;
        }
        t1.re = block_sum(t1.re, scratch);
        t1.im = block_sum(t1.im, scratch);
        t2.re = block_sum(t2.re, scratch);
        t2.im = block_sum(t2.im, scratch);
        const cfloat hv = h[bd * N + n];
        out_dq = cadd(out_dq, cconj(cmul(t1, cmul(g, hv))));
        out_dg = cadd(out_dg, cconj(cmul(t2, hv)));
        if (threadIdx.x == 0) dh[bd * N + n] = cconj(cmul(t2, g));
      }
    }
    if (threadIdx.x == 0) {
      dp[d * N + n] = out_dp;
      dq[d * N + n] = out_dq;
      dgamma[d * N + n] = out_dg;
    }
  }
}

}  // namespace

void ema_parameters_fwd(const float* p, const float* logq, const float* gamma, const float* h, float* k,
                        float* bias, int B, int D, int N, int L, cudaStream_t st) {
  const long long n1 = (long long)D * L;
  ema_weight_fwd_kernel<<<div_up(n1, 256), 256, 0, st>>>(p, (const cfloat*)logq, (const cfloat*)gamma, k, D, N, L);
  if (h != nullptr && bias != nullptr) {
    const long long n2 = (long long)B * D * L;
    ema_bias_fwd_kernel<<<div_up(n2, 256), 256, 0, st>>>((const cfloat*)logq, (const cfloat*)gamma, (const cfloat*)h,
                                                         bias, B, D, N, L);
  }
}

void ema_parameters_bwd(const float* dk, const float* dbias, const float* p, const float* logq, const float* gamma,
                        const float* h, float* dp, float* dq, float* dgamma, float* dh, int B, int D, int N, int L,
                        cudaStream_t st) {
  ema_params_bwd_kernel<<<D, 256, 0, st>>>(dk, dbias, p, (const cfloat*)logq, (const cfloat*)gamma, (const cfloat*)h,
                                           dp, (cfloat*)dq, (cfloat*)dgamma, (cfloat*)dh, B, D, N, L);
}

}  // namespace mb
