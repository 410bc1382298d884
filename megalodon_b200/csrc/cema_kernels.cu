// Complex exponential moving average (CEMA) as a segmented linear scan.
//
//   h_t = q h_{t-1} + p x_t          (N complex states per feature)
//   y_t = Re(sum_n gamma_n h_t,n) + omega x_t
//
// The reference evaluates this as an FFT convolution with a kernel built from
// q^j plus a bias from the carried state plus a separate kernel for the last
// state (ema_parameters + fftconv + ema_hidden; csrc/ops/ema_parameters_kernel.cu,
// fftconv_kernel.cu, ema_hidden_kernel.cu).  With N = 16 the recurrence costs
// O(L N) = about the same arithmetic as two length-2L FFTs, needs no transposed
// layout (threads own consecutive features of the channels-last activations, so
// loads are coalesced), never materialises a spectrum, and produces the carried
// state exactly and for free.  So here the whole layer is three small kernels:
//
//   A: per (batch, segment, feature)  end state of the segment from a zero start
//   B: per (batch, feature, n)        sequential combine over segments -> incoming state
//   C: per (batch, segment, feature)  rerun the segment from its incoming state, emit y
//
// Backward runs the adjoint recurrence (reverse time) for dx, dp, domega, dh_prev
// and a forward recurrence on (h, u = dh/dq) for dgamma and dq.
//
// Work split: a feature's N states are divided over NSPLIT adjacent lanes
// (NPT = N / NSPLIT states each); the sum over n for y / dx is one shuffle.
#include "common.cuh"
#include "kernels.h"

namespace mb {
namespace {

constexpr int kCemaThreads = 256;
constexpr int kPf = 1;   // time steps whose inputs are fetched together (larger values cost registers and ran slower)

template <int NPT>
struct Coef {
  float p[NPT];
  cfloat q[NPT];
  cfloat g[NPT];
};

template <int NPT, int NSPLIT>
__device__ __forceinline__ void load_coef(Coef<NPT>& c, const float* p, const cfloat* q, const cfloat* g,
                                          int d, int split, int N) {
#pragma unroll
  for (int i = 0; i < NPT; ++i) {
    const int n = split * NPT + i;
    c.p[i] = p[d * N + n];
    c.q[i] = q[d * N + n];
    c.g[i] = g[d * N + n];
  }
}

template <int NSPLIT>
__device__ __forceinline__ float split_sum(float v) {
#pragma unroll
  for (int o = NSPLIT / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ cfloat cpow_int(cfloat q, int n) {
  cfloat r = {1.f, 0.f};
  cfloat base = q;
  while (n > 0) {
    if (n & 1) r = cmul(r, base);
    base = cmul(base, base);
    n >>= 1;
  }
  return r;
}

// index into the [B, S, N, D] carry buffers
__device__ __forceinline__ long long cidx(int b, int s, int n, int d, int S, int N, int D) {
  return (((long long)b * S + s) * N + n) * D + d;
}

struct Geo {
  int B, L, D, N, S, Ts;
};

#define CEMA_THREAD_SETUP()                                                    \
  const int tix = blockIdx.x * blockDim.x + threadIdx.x;                       \
  const int d = tix / NSPLIT;                                                  \
  const int split = tix % NSPLIT;                                              \
  const int s = blockIdx.y;                                                    \
  const int b = blockIdx.z;                                                    \
  const bool live = d < geo.D;                                                 \
  const int dd = live ? d : 0;                                                 \
  const int t0 = s * geo.Ts;                                                   \
  const int t1 = min(geo.L, t0 + geo.Ts);

// ------------------------------------------------------------------ forward
template <typename T, int NPT, int NSPLIT>
__global__ void cema_fwd_local(const T* __restrict__ x, const float* __restrict__ p,
                               const cfloat* __restrict__ q, const cfloat* __restrict__ g,
                               cfloat* __restrict__ carry, Geo geo) {
  CEMA_THREAD_SETUP();
  Coef<NPT> c;
  load_coef<NPT, NSPLIT>(c, p, q, g, dd, split, geo.N);
  cfloat h[NPT];
#pragma unroll
  for (int i = 0; i < NPT; ++i) h[i] = {0.f, 0.f};
  const T* xp = x + (long long)b * geo.L * geo.D + dd;
  for (int tb = t0; tb < t1; tb += kPf) {
    float xs[kPf];
#pragma unroll
    for (int j = 0; j < kPf; ++j) xs[j] = tb + j < t1 ? to_f(xp[(long long)(tb + j) * geo.D]) : 0.f;
#pragma unroll
    for (int j = 0; j < kPf; ++j) {
      if (tb + j >= t1) break;
      const float xv = xs[j];
#pragma unroll
      for (int i = 0; i < NPT; ++i) {
        const cfloat hn = cmul(c.q[i], h[i]);
        h[i] = {hn.re + c.p[i] * xv, hn.im};
      }
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < NPT; ++i) carry[cidx(b, s, split * NPT + i, d, geo.S, geo.N, geo.D)] = h[i];
  }
}

// One thread per (b, n, d): carry[b, s] (end state from zero) -> incoming state of segment s.
// `conj_q` runs the adjoint (segments visited from last to first).
__global__ void cema_combine(cfloat* __restrict__ carry, const cfloat* __restrict__ q,
                             const cfloat* __restrict__ init /* [B, D, N] or null */,
                             cfloat* __restrict__ final_out /* [B, D, N] or null */, Geo geo, bool reverse) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long per_b = (long long)geo.N * geo.D;
  if (i >= per_b * geo.B) return;
  const int b = (int)(i / per_b);
  const int n = (int)((i % per_b) / geo.D);
  const int d = (int)(i % geo.D);
  cfloat qq = q[d * geo.N + n];
  if (reverse) qq = cconj(qq);
  const cfloat q_full = cpow_int(qq, geo.Ts);
  const int last_len = geo.L - (geo.S - 1) * geo.Ts;
  const cfloat q_last = cpow_int(qq, last_len);
  cfloat H = init ? init[((long long)b * geo.D + d) * geo.N + n] : cfloat{0.f, 0.f};
  for (int k = 0; k < geo.S; ++k) {
    const int s = reverse ? geo.S - 1 - k : k;
    const long long idx = cidx(b, s, n, d, geo.S, geo.N, geo.D);
    if (k == geo.S - 1 && final_out == nullptr) {   // nobody needs the state after the last visited segment
      carry[idx] = H;
      break;
    }
    const cfloat c = carry[idx];
    carry[idx] = H;
    H = cadd(cmul(s == geo.S - 1 ? q_last : q_full, H), c);
  }
  if (final_out) final_out[((long long)b * geo.D + d) * geo.N + n] = H;
}

template <typename T, int NPT, int NSPLIT>
__global__ void cema_fwd_final(const T* __restrict__ x, const float* __restrict__ p,
                               const cfloat* __restrict__ q, const cfloat* __restrict__ g,
                               const float* __restrict__ omega, const cfloat* __restrict__ incoming,
                               const cfloat* __restrict__ hx, T* __restrict__ y,
                               cfloat* __restrict__ h_last, Geo geo) {
  CEMA_THREAD_SETUP();
  Coef<NPT> c;
  load_coef<NPT, NSPLIT>(c, p, q, g, dd, split, geo.N);
  cfloat h[NPT];
#pragma unroll
  for (int i = 0; i < NPT; ++i) {
    const int n = split * NPT + i;
    if (incoming != nullptr) h[i] = incoming[cidx(b, s, n, dd, geo.S, geo.N, geo.D)];
    else if (hx != nullptr) h[i] = hx[((long long)b * geo.D + dd) * geo.N + n];
    else h[i] = {0.f, 0.f};
  }
  const float om = omega[dd];
  const long long base = (long long)b * geo.L * geo.D + dd;
  for (int tb = t0; tb < t1; tb += kPf) {
    float xs[kPf];
#pragma unroll
    for (int j = 0; j < kPf; ++j) xs[j] = tb + j < t1 ? to_f(x[base + (long long)(tb + j) * geo.D]) : 0.f;
#pragma unroll
    for (int j = 0; j < kPf; ++j) {
      const int t = tb + j;
      if (t >= t1) break;
      const float xv = xs[j];
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < NPT; ++i) {
        const cfloat hn = cmul(c.q[i], h[i]);
        h[i] = {hn.re + c.p[i] * xv, hn.im};
        acc += c.g[i].re * h[i].re - c.g[i].im * h[i].im;
      }
      acc = split_sum<NSPLIT>(acc);
      if (live && split == 0) y[base + (long long)t * geo.D] = from_f<T>(acc + om * xv);
    }
  }
  if (h_last != nullptr && live && s == geo.S - 1) {
#pragma unroll
    for (int i = 0; i < NPT; ++i) h_last[((long long)b * geo.D + d) * geo.N + split * NPT + i] = h[i];
  }
}

// ------------------------------------------------------------------ backward: adjoint (reverse time)
// state s_n = conj(q_n) * lambda_{t+1,n};  lambda_t = s + conj(gamma) dy_t
template <typename T, int NPT, int NSPLIT>
__global__ void cema_bwd_rev_local(const T* __restrict__ dy, const float* __restrict__ p,
                                   const cfloat* __restrict__ q, const cfloat* __restrict__ g,
                                   cfloat* __restrict__ carry, Geo geo) {
  CEMA_THREAD_SETUP();
  Coef<NPT> c;
  load_coef<NPT, NSPLIT>(c, p, q, g, dd, split, geo.N);
  cfloat st[NPT];
#pragma unroll
  for (int i = 0; i < NPT; ++i) st[i] = {0.f, 0.f};
  const long long base = (long long)b * geo.L * geo.D + dd;
  for (int tb = t1 - 1; tb >= t0; tb -= kPf) {
    float gs[kPf];
#pragma unroll
    for (int j = 0; j < kPf; ++j) gs[j] = tb - j >= t0 ? to_f(dy[base + (long long)(tb - j) * geo.D]) : 0.f;
#pragma unroll
    for (int j = 0; j < kPf; ++j) {
      if (tb - j < t0) break;
      const float gy = gs[j];
#pragma unroll
      for (int i = 0; i < NPT; ++i) {
        const cfloat lam = {st[i].re + c.g[i].re * gy, st[i].im - c.g[i].im * gy};
        st[i] = cmul(cconj(c.q[i]), lam);
      }
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < NPT; ++i) carry[cidx(b, s, split * NPT + i, d, geo.S, geo.N, geo.D)] = st[i];
  }
}

template <typename T, int NPT, int NSPLIT>
__global__ void cema_bwd_rev_final(const T* __restrict__ dy, const T* __restrict__ x,
                                   const float* __restrict__ p, const cfloat* __restrict__ q,
                                   const cfloat* __restrict__ g, const float* __restrict__ omega,
                                   const cfloat* __restrict__ incoming, const cfloat* __restrict__ dh_last,
                                   T* __restrict__ dx, float* __restrict__ dp, float* __restrict__ domega,
                                   cfloat* __restrict__ dhx, Geo geo) {
  CEMA_THREAD_SETUP();
  Coef<NPT> c;
  load_coef<NPT, NSPLIT>(c, p, q, g, dd, split, geo.N);
  cfloat st[NPT];
  float acc_p[NPT];
#pragma unroll
  for (int i = 0; i < NPT; ++i) {
    const int n = split * NPT + i;
    if (incoming != nullptr) st[i] = incoming[cidx(b, s, n, dd, geo.S, geo.N, geo.D)];
    else if (dh_last != nullptr) st[i] = dh_last[((long long)b * geo.D + dd) * geo.N + n];
    else st[i] = {0.f, 0.f};
    acc_p[i] = 0.f;
  }
  const float om = omega[dd];
  float acc_om = 0.f;
  const long long base = (long long)b * geo.L * geo.D + dd;
  for (int tb = t1 - 1; tb >= t0; tb -= kPf) {
    float gs[kPf], xs[kPf];
#pragma unroll
    for (int j = 0; j < kPf; ++j) {
      const bool in = tb - j >= t0;
      gs[j] = in ? to_f(dy[base + (long long)(tb - j) * geo.D]) : 0.f;
      xs[j] = in ? to_f(x[base + (long long)(tb - j) * geo.D]) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < kPf; ++j) {
      const int t = tb - j;
      if (t < t0) break;
      const float gy = gs[j], xv = xs[j];
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < NPT; ++i) {
        const cfloat lam = {st[i].re + c.g[i].re * gy, st[i].im - c.g[i].im * gy};
        acc += c.p[i] * lam.re;
        acc_p[i] += lam.re * xv;
        st[i] = cmul(cconj(c.q[i]), lam);
      }
      acc = split_sum<NSPLIT>(acc);
      acc_om += gy * xv;
      if (live && split == 0) dx[base + (long long)t * geo.D] = from_f<T>(acc + om * gy);
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < NPT; ++i) atomicAdd(dp + d * geo.N + split * NPT + i, acc_p[i]);
    if (split == 0) atomicAdd(domega + d, acc_om);
    if (dhx != nullptr && s == 0 && incoming == nullptr) {
      // single-segment case: the combine kernel did not run, finish here
#pragma unroll
      for (int i = 0; i < NPT; ++i) dhx[((long long)b * geo.D + d) * geo.N + split * NPT + i] = st[i];
    }
  }
}

// ------------------------------------------------------------------ backward: forward-time pass on (h, u = dh/dq)
template <typename T, int NPT, int NSPLIT>
__global__ void cema_bwd_fwd_local(const T* __restrict__ x, const float* __restrict__ p,
                                   const cfloat* __restrict__ q, const cfloat* __restrict__ g,
                                   cfloat* __restrict__ carry_h, cfloat* __restrict__ carry_u, Geo geo) {
  CEMA_THREAD_SETUP();
  Coef<NPT> c;
  load_coef<NPT, NSPLIT>(c, p, q, g, dd, split, geo.N);
  cfloat h[NPT], u[NPT];
#pragma unroll
  for (int i = 0; i < NPT; ++i) h[i] = u[i] = {0.f, 0.f};
  const long long base = (long long)b * geo.L * geo.D + dd;
  for (int tb = t0; tb < t1; tb += kPf) {
    float xs[kPf];
#pragma unroll
    for (int j = 0; j < kPf; ++j) xs[j] = tb + j < t1 ? to_f(x[base + (long long)(tb + j) * geo.D]) : 0.f;
#pragma unroll
    for (int j = 0; j < kPf; ++j) {
      if (tb + j >= t1) break;
      const float xv = xs[j];
#pragma unroll
      for (int i = 0; i < NPT; ++i) {
        u[i] = cadd(cmul(c.q[i], u[i]), h[i]);
        const cfloat hn = cmul(c.q[i], h[i]);
        h[i] = {hn.re + c.p[i] * xv, hn.im};
      }
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
      const long long idx = cidx(b, s, split * NPT + i, d, geo.S, geo.N, geo.D);
      carry_h[idx] = h[i];
      carry_u[idx] = u[i];
    }
  }
}

// per (b, n, d): incoming (h, u) of every segment; adds the last-state term of dq
__global__ void cema_bwd_fwd_combine(cfloat* __restrict__ carry_h, cfloat* __restrict__ carry_u,
                                     const cfloat* __restrict__ q, const cfloat* __restrict__ hx,
                                     const cfloat* __restrict__ dh_last, float* __restrict__ dq, Geo geo) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long per_b = (long long)geo.N * geo.D;
  if (i >= per_b * geo.B) return;
  const int b = (int)(i / per_b);
  const int n = (int)((i % per_b) / geo.D);
  const int d = (int)(i % geo.D);
  const cfloat qq = q[d * geo.N + n];
  const int last_len = geo.L - (geo.S - 1) * geo.Ts;
  const cfloat qT = cpow_int(qq, geo.Ts), qTm1 = cpow_int(qq, geo.Ts - 1);
  const cfloat qL = cpow_int(qq, last_len), qLm1 = cpow_int(qq, last_len - 1);
  cfloat H = hx ? hx[((long long)b * geo.D + d) * geo.N + n] : cfloat{0.f, 0.f};
  cfloat U = {0.f, 0.f};
  for (int s = 0; s < geo.S; ++s) {
    const long long idx = cidx(b, s, n, d, geo.S, geo.N, geo.D);
    const cfloat ch = carry_h[idx], cu = carry_u[idx];
    carry_h[idx] = H;
    carry_u[idx] = U;
    const bool last = s == geo.S - 1;
    const int len = last ? last_len : geo.Ts;
    const cfloat a = last ? qL : qT, am1 = last ? qLm1 : qTm1;
    cfloat lh = cmul(am1, H);
    lh = {lh.re * len, lh.im * len};
    U = cadd(cadd(cmul(a, U), lh), cu);
    H = cadd(cmul(a, H), ch);
  }
  if (dh_last != nullptr) {
    // dL/dq += g_last * conj(u_{L-1})
    const cfloat gl = dh_last[((long long)b * geo.D + d) * geo.N + n];
    const cfloat v = cmul(gl, cconj(U));
    atomicAdd(dq + 2 * (d * geo.N + n), v.re);
    atomicAdd(dq + 2 * (d * geo.N + n) + 1, v.im);
  }
}

template <typename T, int NPT, int NSPLIT>
__global__ void cema_bwd_fwd_final(const T* __restrict__ dy, const T* __restrict__ x,
                                   const float* __restrict__ p, const cfloat* __restrict__ q,
                                   const cfloat* __restrict__ g, const cfloat* __restrict__ inc_h,
                                   const cfloat* __restrict__ inc_u, const cfloat* __restrict__ hx,
                                   const cfloat* __restrict__ dh_last, float* __restrict__ dgamma,
                                   float* __restrict__ dq, Geo geo) {
  CEMA_THREAD_SETUP();
  Coef<NPT> c;
  load_coef<NPT, NSPLIT>(c, p, q, g, dd, split, geo.N);
  cfloat h[NPT], u[NPT], ag[NPT], aq[NPT];
#pragma unroll
  for (int i = 0; i < NPT; ++i) {
    const int n = split * NPT + i;
    if (inc_h != nullptr) {
      const long long idx = cidx(b, s, n, dd, geo.S, geo.N, geo.D);
      h[i] = inc_h[idx];
      u[i] = inc_u[idx];
    } else {
      h[i] = hx ? hx[((long long)b * geo.D + dd) * geo.N + n] : cfloat{0.f, 0.f};
      u[i] = {0.f, 0.f};
    }
    ag[i] = aq[i] = {0.f, 0.f};
  }
  const long long base = (long long)b * geo.L * geo.D + dd;
  for (int tb = t0; tb < t1; tb += kPf) {
    float xs[kPf], gs[kPf];
#pragma unroll
    for (int j = 0; j < kPf; ++j) {
      const bool in = tb + j < t1;
      xs[j] = in ? to_f(x[base + (long long)(tb + j) * geo.D]) : 0.f;
      gs[j] = in ? to_f(dy[base + (long long)(tb + j) * geo.D]) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < kPf; ++j) {
      if (tb + j >= t1) break;
      const float xv = xs[j], gy = gs[j];
#pragma unroll
      for (int i = 0; i < NPT; ++i) {
        u[i] = cadd(cmul(c.q[i], u[i]), h[i]);
        const cfloat hn = cmul(c.q[i], h[i]);
        h[i] = {hn.re + c.p[i] * xv, hn.im};
        // dgamma += conj(h) dy ; dq += (conj(gamma) dy) conj(u)
        ag[i].re += h[i].re * gy;
        ag[i].im -= h[i].im * gy;
        const cfloat cg = {c.g[i].re * gy, -c.g[i].im * gy};
        const cfloat v = cmul(cg, cconj(u[i]));
        aq[i].re += v.re;
        aq[i].im += v.im;
      }
    }
  }
  if (inc_h == nullptr && dh_last != nullptr) {
    // single-segment case (the combine kernel did not run): dq += g_last * conj(u_{L-1})
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
      const cfloat gl = dh_last[((long long)b * geo.D + dd) * geo.N + split * NPT + i];
      const cfloat v = cmul(gl, cconj(u[i]));
      aq[i].re += v.re;
      aq[i].im += v.im;
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
      const int o = 2 * (d * geo.N + split * NPT + i);
      atomicAdd(dgamma + o, ag[i].re);
      atomicAdd(dgamma + o + 1, ag[i].im);
      atomicAdd(dq + o, aq[i].re);
      atomicAdd(dq + o + 1, aq[i].im);
    }
  }
}


// ================================================================== tiled variants (16-bit activations)
// Same three-kernel structure, restructured for the FMA pipes, which bound this
// op (N complex states per element, about ten FMAs per state and time step):
//
//   * activations move through shared memory in tiles of kTT time steps x 128
//     features (cp.async, kStages deep), so the recurrence never waits on a
//     global load, and outputs leave through a staged tile with 16-byte stores;
//   * the state is kept as h / p, which turns "q h + p x" into two FMAs per
//     component with x as the addend; p is folded into gamma (c = gamma p) and
//     multiplied back when a state leaves the kernel.  |p| is floored at 1e-20 so
//     the division of an incoming state is always finite;
//   * the adjoint's local pass runs on mu = lambda / conj(gamma) (zero start, so
//     nothing is divided), and the forward-time pass accumulates G = sum dy h/p
//     and U = sum dy u/p, from which dgamma = conj(p G), dq = conj(gamma p U).
//
// A CTA owns 128 features of one segment: 128 * NSPLIT threads.
constexpr int kTT = 16;
constexpr int kStages = 4;
constexpr int kTileFeat = 128;
constexpr int kTileElems = kTT * kTileFeat;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned int s = (unsigned int)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;     // 0: nothing is read, the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ float p_floor(float p) { return copysignf(fmaxf(fabsf(p), 1e-20f), p); }

// Walks the time steps [t0, t1) of batch row b for features [f0, f0 + 128) in tiles, forward or
// reverse in time, and calls step(in0_t, in1_t) for this thread's feature at every step; the value
// it returns is written to `out` (by the split-0 lane) when HAS_OUT.
template <typename T, int NIN, bool HAS_OUT, bool REVERSE, int NSPLIT, typename Step>
__device__ __forceinline__ void tiled_scan(const T* __restrict__ in0, const T* __restrict__ in1, T* __restrict__ out,
                                           const Geo& geo, int b, int t0, int t1, int f0, T* smem_in, T* smem_out,
                                           Step&& step) {
  constexpr int NT = kTileFeat * NSPLIT;
  constexpr int kChunks = kTileElems / 8;            // 16-byte chunks per tile
  const int tid = threadIdx.x;
  const int fl = tid / NSPLIT;
  const int split = tid % NSPLIT;
  const int nt = (t1 - t0 + kTT - 1) / kTT;
  const long long row0 = (long long)b * geo.L;

  auto tile_base = [&](int k) { return t0 + (REVERSE ? nt - 1 - k : k) * kTT; };
  auto issue = [&](int k) {
    if (k < nt) {
      const int tb = tile_base(k);
      const int stage = k % kStages;
      for (int c = tid; c < kChunks; c += NT) {
        const int r = c >> 4, cc = c & 15;
        const int t = tb + r, f = f0 + cc * 8;
        const bool ok = t < t1 && f < geo.D;
        const long long off = ok ? (row0 + t) * geo.D + f : 0;
        cp_async16(smem_in + stage * kTileElems + r * kTileFeat + cc * 8, in0 + off, ok);
        if (NIN == 2)
          cp_async16(smem_in + (kStages + stage) * kTileElems + r * kTileFeat + cc * 8, in1 + off, ok);
      }
    }
    cp_async_commit();     // an empty group keeps the wait_group arithmetic uniform
  };
  auto store_out = [&](int k) {
    const int tb = tile_base(k);
    const T* src = smem_out + (k & 1) * kTileElems;
    for (int c = tid; c < kChunks; c += NT) {
      const int r = c >> 4, cc = c & 15;
      const int t = tb + r, f = f0 + cc * 8;
      if (t < t1 && f < geo.D)
        *reinterpret_cast<uint4*>(out + (row0 + t) * geo.D + f) =
            *reinterpret_cast<const uint4*>(src + r * kTileFeat + cc * 8);
    }
  };

#pragma unroll
  for (int k = 0; k < kStages - 1; ++k) issue(k);
  for (int k = 0; k < nt; ++k) {
    cp_async_wait<kStages - 2>();
    __syncthreads();                 // tile k has landed for everyone; everyone is done with tile k-1
    issue(k + kStages - 1);          // refills the stage tile k-1 used
    if (HAS_OUT && k > 0) store_out(k - 1);
    const int tb = tile_base(k);
    const int nvalid = min(kTT, t1 - tb);
    const T* x0 = smem_in + (k % kStages) * kTileElems + fl;
    const T* x1 = smem_in + (kStages + k % kStages) * kTileElems + fl;
    T* os = smem_out + (k & 1) * kTileElems + fl;
    if (nvalid == kTT) {
#pragma unroll
      for (int jj = 0; jj < kTT; ++jj) {
        const int j = REVERSE ? kTT - 1 - jj : jj;
        const float a0 = to_f(x0[j * kTileFeat]);
        const float a1 = NIN == 2 ? to_f(x1[j * kTileFeat]) : 0.f;
        const float o = step(a0, a1);
        if (HAS_OUT && split == 0) os[j * kTileFeat] = from_f<T>(o);
      }
    } else {
      for (int jj = 0; jj < kTT; ++jj) {
        const int j = REVERSE ? kTT - 1 - jj : jj;
        if (j >= nvalid) continue;
        const float a0 = to_f(x0[j * kTileFeat]);
        const float a1 = NIN == 2 ? to_f(x1[j * kTileFeat]) : 0.f;
        const float o = step(a0, a1);
        if (HAS_OUT && split == 0) os[j * kTileFeat] = from_f<T>(o);
      }
    }
  }
  if (HAS_OUT && nt > 0) {
    __syncthreads();
    store_out(nt - 1);
  }
}

#define CEMA_TILE_SETUP()                                       \
  const int fl = threadIdx.x / NSPLIT;                          \
  const int split = threadIdx.x % NSPLIT;                       \
  const int f0 = blockIdx.x * kTileFeat;                        \
  const int d = f0 + fl;                                        \
  const int s = blockIdx.y;                                     \
  const int b = blockIdx.z;                                     \
  const bool live = d < geo.D;                                  \
  const int dd = live ? d : 0;                                  \
  const int t0 = s * geo.Ts;                                    \
  const int t1 = min(geo.L, t0 + geo.Ts);

// h <- q h + x  (h kept as h / p)
#define CEMA_ADVANCE(h, qq, xv)                                          \
  do {                                                                   \
    const float re_ = fmaf(qq.re, h.re, fmaf(-qq.im, h.im, xv));         \
    h.im = fmaf(qq.re, h.im, qq.im * h.re);                              \
    h.re = re_;                                                          \
  } while (0)

template <typename T, int NSPLIT>
__global__ void __launch_bounds__(kTileFeat* NSPLIT)
cema_fwd_local_t(const T* __restrict__ x, const float* __restrict__ p, const cfloat* __restrict__ q,
                 cfloat* __restrict__ carry, Geo geo) {
  constexpr int NPT = 8;
  __shared__ __align__(16) T sm_in[kStages * kTileElems];
  CEMA_TILE_SETUP();
  cfloat qq[NPT], h[NPT];
#pragma unroll
  for (int i = 0; i < NPT; ++i) {
    qq[i] = q[dd * geo.N + split * NPT + i];
    h[i] = {0.f, 0.f};
  }
  tiled_scan<T, 1, false, false, NSPLIT>(x, nullptr, nullptr, geo, b, t0, t1, f0, sm_in, nullptr,
                                         [&](float xv, float) {
#pragma unroll
                                           for (int i = 0; i < NPT; ++i) CEMA_ADVANCE(h[i], qq[i], xv);
                                           return 0.f;
                                         });
  if (live) {
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
      const int n = split * NPT + i;
      const float pp = p[d * geo.N + n];
      carry[cidx(b, s, n, d, geo.S, geo.N, geo.D)] = {pp * h[i].re, pp * h[i].im};
    }
  }
}

template <typename T, int NSPLIT>
__global__ void __launch_bounds__(kTileFeat* NSPLIT)
cema_fwd_final_t(const T* __restrict__ x, const float* __restrict__ p, const cfloat* __restrict__ q,
                 const cfloat* __restrict__ g, const float* __restrict__ omega,
                 const cfloat* __restrict__ incoming, const cfloat* __restrict__ hx, T* __restrict__ y,
                 cfloat* __restrict__ h_last, Geo geo) {
  constexpr int NPT = 8;
  __shared__ __align__(16) T sm_in[kStages * kTileElems];
  __shared__ __align__(16) T sm_out[2 * kTileElems];
  CEMA_TILE_SETUP();
  cfloat qq[NPT], c[NPT], h[NPT];
  float pe[NPT];
#pragma unroll
  for (int i = 0; i < NPT; ++i) {
    const int n = split * NPT + i;
    qq[i] = q[dd * geo.N + n];
    pe[i] = p_floor(p[dd * geo.N + n]);
    const cfloat gg = g[dd * geo.N + n];
    c[i] = {gg.re * pe[i], gg.im * pe[i]};
    cfloat hin = {0.f, 0.f};
    if (incoming != nullptr) hin = incoming[cidx(b, s, n, dd, geo.S, geo.N, geo.D)];
    else if (hx != nullptr) hin = hx[((long long)b * geo.D + dd) * geo.N + n];
    h[i] = {hin.re / pe[i], hin.im / pe[i]};
  }
  const float om = omega[dd];
  tiled_scan<T, 1, true, false, NSPLIT>(x, nullptr, y, geo, b, t0, t1, f0, sm_in, sm_out, [&](float xv, float) {
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
      CEMA_ADVANCE(h[i], qq[i], xv);
      acc = fmaf(c[i].re, h[i].re, fmaf(-c[i].im, h[i].im, acc));
    }
    return split_sum<NSPLIT>(acc) + om * xv;
  });
  if (h_last != nullptr && live && s == geo.S - 1) {
#pragma unroll
    for (int i = 0; i < NPT; ++i)
      h_last[((long long)b * geo.D + d) * geo.N + split * NPT + i] = {pe[i] * h[i].re, pe[i] * h[i].im};
  }
}

// adjoint, local: mu_t = dy_t + conj(q) mu_{t+1} from zero; carry = conj(q) conj(gamma) mu_{t0}
template <typename T, int NSPLIT>
__global__ void __launch_bounds__(kTileFeat* NSPLIT)
cema_bwd_rev_local_t(const T* __restrict__ dy, const cfloat* __restrict__ q, const cfloat* __restrict__ g,
                     cfloat* __restrict__ carry, Geo geo) {
  constexpr int NPT = 8;
  __shared__ __align__(16) T sm_in[kStages * kTileElems];
  CEMA_TILE_SETUP();
  cfloat qc[NPT], m[NPT];
#pragma unroll
  for (int i = 0; i < NPT; ++i) {
    qc[i] = cconj(q[dd * geo.N + split * NPT + i]);
    m[i] = {0.f, 0.f};
  }
  tiled_scan<T, 1, false, true, NSPLIT>(dy, nullptr, nullptr, geo, b, t0, t1, f0, sm_in, nullptr,
                                        [&](float gy, float) {
#pragma unroll
                                          for (int i = 0; i < NPT; ++i) CEMA_ADVANCE(m[i], qc[i], gy);
                                          return 0.f;
                                        });
  if (live) {
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
      const int n = split * NPT + i;
      const cfloat lam = cmul(cconj(g[d * geo.N + n]), m[i]);
      carry[cidx(b, s, n, d, geo.S, geo.N, geo.D)] = cmul(qc[i], lam);
    }
  }
}

// adjoint, final: state st = p conj(q) lambda_{t+1};  Lambda_t = st + conj(c) dy_t (c = gamma p)
template <typename T, int NSPLIT>
__global__ void __launch_bounds__(kTileFeat* NSPLIT)
cema_bwd_rev_final_t(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ p,
                     const cfloat* __restrict__ q, const cfloat* __restrict__ g, const float* __restrict__ omega,
                     const cfloat* __restrict__ incoming, const cfloat* __restrict__ dh_last, T* __restrict__ dx,
                     float* __restrict__ dp, float* __restrict__ domega, cfloat* __restrict__ dhx, Geo geo) {
  constexpr int NPT = 8;
  __shared__ __align__(16) T sm_in[2 * kStages * kTileElems];
  __shared__ __align__(16) T sm_out[2 * kTileElems];
  CEMA_TILE_SETUP();
  cfloat qq[NPT], c[NPT], st[NPT];
  float pe[NPT], acc_p[NPT];
#pragma unroll
  for (int i = 0; i < NPT; ++i) {
    const int n = split * NPT + i;
    qq[i] = q[dd * geo.N + n];
    pe[i] = p_floor(p[dd * geo.N + n]);
    const cfloat gg = g[dd * geo.N + n];
    c[i] = {gg.re * pe[i], gg.im * pe[i]};
    cfloat in = {0.f, 0.f};
    if (incoming != nullptr) in = incoming[cidx(b, s, n, dd, geo.S, geo.N, geo.D)];
    else if (dh_last != nullptr) in = dh_last[((long long)b * geo.D + dd) * geo.N + n];
    st[i] = {in.re * pe[i], in.im * pe[i]};
    acc_p[i] = 0.f;
  }
  const float om = omega[dd];
  float acc_om = 0.f;
  tiled_scan<T, 2, true, true, NSPLIT>(dy, x, dx, geo, b, t0, t1, f0, sm_in, sm_out, [&](float gy, float xv) {
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
      const float lre = fmaf(c[i].re, gy, st[i].re);
      const float lim = fmaf(-c[i].im, gy, st[i].im);
      acc += lre;
      acc_p[i] = fmaf(lre, xv, acc_p[i]);
      st[i].re = fmaf(qq[i].re, lre, qq[i].im * lim);       // conj(q) * Lambda
      st[i].im = fmaf(qq[i].re, lim, -qq[i].im * lre);
    }
    acc_om = fmaf(gy, xv, acc_om);
    return split_sum<NSPLIT>(acc) + om * gy;
  });
  if (live) {
#pragma unroll
    for (int i = 0; i < NPT; ++i) atomicAdd(dp + d * geo.N + split * NPT + i, acc_p[i] / pe[i]);
    if (split == 0) atomicAdd(domega + d, acc_om);
    if (dhx != nullptr && s == 0 && incoming == nullptr) {
      // single-segment case: the combine kernel did not run, finish here
#pragma unroll
      for (int i = 0; i < NPT; ++i)
        dhx[((long long)b * geo.D + d) * geo.N + split * NPT + i] = {st[i].re / pe[i], st[i].im / pe[i]};
    }
  }
}

// forward-time pass, local: end states of (h, u = dh/dq) from zero
template <typename T, int NSPLIT>
__global__ void __launch_bounds__(kTileFeat* NSPLIT)
cema_bwd_fwd_local_t(const T* __restrict__ x, const float* __restrict__ p, const cfloat* __restrict__ q,
                     cfloat* __restrict__ carry_h, cfloat* __restrict__ carry_u, Geo geo) {
  constexpr int NPT = 8;
  __shared__ __align__(16) T sm_in[kStages * kTileElems];
  CEMA_TILE_SETUP();
  cfloat qq[NPT], h[NPT], u[NPT];
#pragma unroll
  for (int i = 0; i < NPT; ++i) {
    qq[i] = q[dd * geo.N + split * NPT + i];
    h[i] = u[i] = {0.f, 0.f};
  }
  tiled_scan<T, 1, false, false, NSPLIT>(x, nullptr, nullptr, geo, b, t0, t1, f0, sm_in, nullptr,
                                         [&](float xv, float) {
#pragma unroll
                                           for (int i = 0; i < NPT; ++i) {
                                             const float ure = fmaf(qq[i].re, u[i].re, fmaf(-qq[i].im, u[i].im, h[i].re));
                                             u[i].im = fmaf(qq[i].re, u[i].im, fmaf(qq[i].im, u[i].re, h[i].im));
                                             u[i].re = ure;
                                             CEMA_ADVANCE(h[i], qq[i], xv);
                                           }
                                           return 0.f;
                                         });
  if (live) {
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
      const int n = split * NPT + i;
      const float pp = p[d * geo.N + n];
      const long long idx = cidx(b, s, n, d, geo.S, geo.N, geo.D);
      carry_h[idx] = {pp * h[i].re, pp * h[i].im};
      carry_u[idx] = {pp * u[i].re, pp * u[i].im};
    }
  }
}

// forward-time pass, final: G = sum dy h/p, U = sum dy u/p  ->  dgamma += conj(p G), dq += conj(gamma p U)
template <typename T, int NSPLIT>
__global__ void __launch_bounds__(kTileFeat* NSPLIT)
cema_bwd_fwd_final_t(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ p,
                     const cfloat* __restrict__ q, const cfloat* __restrict__ g, const cfloat* __restrict__ inc_h,
                     const cfloat* __restrict__ inc_u, const cfloat* __restrict__ hx,
                     const cfloat* __restrict__ dh_last, float* __restrict__ dgamma, float* __restrict__ dq,
                     Geo geo) {
  constexpr int NPT = 8;
  __shared__ __align__(16) T sm_in[2 * kStages * kTileElems];
  CEMA_TILE_SETUP();
  cfloat qq[NPT], h[NPT], u[NPT], G[NPT], U[NPT];
#pragma unroll
  for (int i = 0; i < NPT; ++i) {
    const int n = split * NPT + i;
    qq[i] = q[dd * geo.N + n];
    const float pe = p_floor(p[dd * geo.N + n]);
    cfloat hin = {0.f, 0.f}, uin = {0.f, 0.f};
    if (inc_h != nullptr) {
      const long long idx = cidx(b, s, n, dd, geo.S, geo.N, geo.D);
      hin = inc_h[idx];
      uin = inc_u[idx];
    } else if (hx != nullptr) {
      hin = hx[((long long)b * geo.D + dd) * geo.N + n];
    }
    h[i] = {hin.re / pe, hin.im / pe};
    u[i] = {uin.re / pe, uin.im / pe};
    G[i] = U[i] = {0.f, 0.f};
  }
  tiled_scan<T, 2, false, false, NSPLIT>(x, dy, nullptr, geo, b, t0, t1, f0, sm_in, nullptr,
                                         [&](float xv, float gy) {
#pragma unroll
                                           for (int i = 0; i < NPT; ++i) {
                                             const float ure = fmaf(qq[i].re, u[i].re, fmaf(-qq[i].im, u[i].im, h[i].re));
                                             u[i].im = fmaf(qq[i].re, u[i].im, fmaf(qq[i].im, u[i].re, h[i].im));
                                             u[i].re = ure;
                                             CEMA_ADVANCE(h[i], qq[i], xv);
                                             G[i].re = fmaf(h[i].re, gy, G[i].re);
                                             G[i].im = fmaf(h[i].im, gy, G[i].im);
                                             U[i].re = fmaf(u[i].re, gy, U[i].re);
                                             U[i].im = fmaf(u[i].im, gy, U[i].im);
                                           }
                                           return 0.f;
                                         });
  if (live) {
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
      const int n = split * NPT + i;
      const float pe = p_floor(p[d * geo.N + n]);
      const cfloat gg = g[d * geo.N + n];
      const cfloat cu = cmul({gg.re * pe, gg.im * pe}, U[i]);
      cfloat aq = {cu.re, -cu.im};
      if (inc_h == nullptr && dh_last != nullptr) {
        // single-segment case (the combine kernel did not run): dq += g_last * conj(u_{L-1})
        const cfloat gl = dh_last[((long long)b * geo.D + d) * geo.N + n];
        const cfloat v = cmul(gl, {pe * u[i].re, -pe * u[i].im});
        aq.re += v.re;
        aq.im += v.im;
      }
      const int o = 2 * (d * geo.N + n);
      atomicAdd(dgamma + o, pe * G[i].re);
      atomicAdd(dgamma + o + 1, -pe * G[i].im);
      atomicAdd(dq + o, aq.re);
      atomicAdd(dq + o + 1, aq.im);
    }
  }
}

// Segment length for the tiled kernels: the longest (<= 512 steps, so the fewest redundant
// local passes and pipeline ramps) for which all CTAs of the final kernel fit in a whole
// number of waves.  Never below kCemaSegLen, which sizes the carry buffers.
template <typename K>
int plan_seg_len(K final_kernel, int threads, int B, int L, int D) {
  if (L <= kCemaSegLen) return kCemaSegLen;
  int per_sm = 1;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, final_kernel, threads, 0) != cudaSuccess || per_sm < 1)
    per_sm = 1;
  const long long slots = 148LL * per_sm;
  const long long fb = (long long)div_up(D, kTileFeat) * B;
  for (int k = 1; k <= 64; ++k) {
    const long long S = k * slots / fb;
    if (S < 1) continue;
    const int ts = (int)(((L + S - 1) / S + 15) / 16 * 16);
    if (ts > 512) continue;
    return ts < kCemaSegLen ? kCemaSegLen : ts;
  }
  return kCemaSegLen;
}

inline Geo make_geo(int B, int L, int D, int N, int ts) { return Geo{B, L, D, N, (L + ts - 1) / ts, ts}; }

inline bool tiled_ok(int D, int N, int x_dtype) {
  return x_dtype != kF32 && D % 8 == 0 && (N == 8 || N == 16 || N == 32);
}

void pick_split(int N, int& npt, int& nsplit) {
  if (N % 8 == 0) { npt = 8; nsplit = N / 8; }
  else if (N % 4 == 0) { npt = 4; nsplit = N / 4; }
  else if (N % 2 == 0) { npt = 2; nsplit = N / 2; }
  else { npt = 1; nsplit = N; }
}

#define CEMA_SWITCH(N, ...)                                                                  \
  do {                                                                                       \
    int npt_, nsplit_;                                                                       \
    pick_split(N, npt_, nsplit_);                                                            \
    if (npt_ == 8 && nsplit_ == 1) { constexpr int NPT = 8, NSPLIT = 1; __VA_ARGS__; }       \
    else if (npt_ == 8 && nsplit_ == 2) { constexpr int NPT = 8, NSPLIT = 2; __VA_ARGS__; }  \
    else if (npt_ == 8 && nsplit_ == 4) { constexpr int NPT = 8, NSPLIT = 4; __VA_ARGS__; }  \
    else if (npt_ == 4 && nsplit_ == 1) { constexpr int NPT = 4, NSPLIT = 1; __VA_ARGS__; }  \
    else if (npt_ == 2 && nsplit_ == 1) { constexpr int NPT = 2, NSPLIT = 1; __VA_ARGS__; }  \
    else { constexpr int NPT = 1, NSPLIT = 1; __VA_ARGS__; }                                 \
  } while (0)



#define CEMA_TILED_SWITCH(N, ...)                                      \
  do {                                                                 \
    if ((N) == 8) { constexpr int NSPLIT = 1; __VA_ARGS__; }           \
    else if ((N) == 16) { constexpr int NSPLIT = 2; __VA_ARGS__; }     \
    else { constexpr int NSPLIT = 4; __VA_ARGS__; }                    \
  } while (0)

}  // namespace

bool cema_supported_ndim(int N) { return N == 1 || N == 2 || N == 4 || N == 8 || N == 16 || N == 32; }

int cema_num_segments(int L) { return (L + kCemaSegLen - 1) / kCemaSegLen; }

void cema_fwd(const void* x, const float* p, const float* q, const float* gamma, const float* omega,
              const float* hx, void* y, float* h_last, float* carry, int B, int L, int D, int N,
              int x_dtype, cudaStream_t st) {
  Geo geo{B, L, D, N, cema_num_segments(L), kCemaSegLen};
  const cfloat* qc = (const cfloat*)q;
  const cfloat* gc = (const cfloat*)gamma;
  if (tiled_ok(D, N, x_dtype)) {
    MB_DISPATCH_16BIT(x_dtype, {
      using T = scalar_t;
      CEMA_TILED_SWITCH(N, {
        geo = make_geo(B, L, D, N, plan_seg_len(cema_fwd_final_t<T, NSPLIT>, kTileFeat * NSPLIT, B, L, D));
        dim3 grid(div_up(D, kTileFeat), geo.S, B);
        const cfloat* incoming = nullptr;
        if (geo.S > 1) {
          // the end state of the last segment is never needed (fwd_final produces h_last)
          dim3 grid_a(grid.x, geo.S - 1, B);
          cema_fwd_local_t<T, NSPLIT><<<grid_a, kTileFeat * NSPLIT, 0, st>>>((const T*)x, p, qc, (cfloat*)carry, geo);
          const long long n = (long long)B * N * D;
          cema_combine<<<div_up(n, 256), 256, 0, st>>>((cfloat*)carry, qc, (const cfloat*)hx, nullptr, geo, false);
          incoming = (const cfloat*)carry;
        }
        cema_fwd_final_t<T, NSPLIT><<<grid, kTileFeat * NSPLIT, 0, st>>>(
            (const T*)x, p, qc, gc, omega, incoming, (const cfloat*)hx, (T*)y, (cfloat*)h_last, geo);
      });
    });
    return;
  }
  MB_DISPATCH_DTYPE(x_dtype, {
    using T = scalar_t;
    CEMA_SWITCH(N, {
      dim3 grid(div_up((long long)D * NSPLIT, kCemaThreads), geo.S, B);
      const cfloat* incoming = nullptr;
      if (geo.S > 1) {
        cema_fwd_local<T, NPT, NSPLIT><<<grid, kCemaThreads, 0, st>>>((const T*)x, p, qc, gc, (cfloat*)carry, geo);
        const long long n = (long long)B * N * D;
        cema_combine<<<div_up(n, 256), 256, 0, st>>>((cfloat*)carry, qc, (const cfloat*)hx, nullptr, geo, false);
        incoming = (const cfloat*)carry;
      }
      cema_fwd_final<T, NPT, NSPLIT><<<grid, kCemaThreads, 0, st>>>(
          (const T*)x, p, qc, gc, omega, incoming, (const cfloat*)hx, (T*)y, (cfloat*)h_last, geo);
    });
  });
}

void cema_bwd(const void* dy, const void* x, const float* p, const float* q, const float* gamma,
              const float* omega, const float* hx, const float* dh_last, void* dx, float* dp, float* dq,
              float* dgamma, float* domega, float* dhx, float* carry_a, float* carry_b, int B, int L,
              int D, int N, int x_dtype, cudaStream_t st) {
  Geo geo{B, L, D, N, cema_num_segments(L), kCemaSegLen};
  const cfloat* qc = (const cfloat*)q;
  const cfloat* gc = (const cfloat*)gamma;
  const long long nbd = (long long)B * N * D;
  if (tiled_ok(D, N, x_dtype)) {
    MB_DISPATCH_16BIT(x_dtype, {
      using T = scalar_t;
      CEMA_TILED_SWITCH(N, {
        const int nthr = kTileFeat * NSPLIT;
        geo = make_geo(B, L, D, N, plan_seg_len(cema_bwd_fwd_final_t<T, NSPLIT>, nthr, B, L, D));
        dim3 grid(div_up(D, kTileFeat), geo.S, B);
        const cfloat* inc = nullptr;
        if (geo.S > 1) {
          cema_bwd_rev_local_t<T, NSPLIT><<<grid, nthr, 0, st>>>((const T*)dy, qc, gc, (cfloat*)carry_a, geo);
          cema_combine<<<div_up(nbd, 256), 256, 0, st>>>((cfloat*)carry_a, qc, (const cfloat*)dh_last,
                                                         (cfloat*)dhx, geo, true);
          inc = (const cfloat*)carry_a;
        }
        cema_bwd_rev_final_t<T, NSPLIT><<<grid, nthr, 0, st>>>(
            (const T*)dy, (const T*)x, p, qc, gc, omega, inc, (const cfloat*)dh_last, (T*)dx, dp, domega,
            (cfloat*)dhx, geo);
        const cfloat* inc_h = nullptr;
        const cfloat* inc_u = nullptr;
        if (geo.S > 1) {
          cema_bwd_fwd_local_t<T, NSPLIT><<<grid, nthr, 0, st>>>((const T*)x, p, qc, (cfloat*)carry_a,
                                                                (cfloat*)carry_b, geo);
          cema_bwd_fwd_combine<<<div_up(nbd, 256), 256, 0, st>>>((cfloat*)carry_a, (cfloat*)carry_b, qc,
                                                                 (const cfloat*)hx, (const cfloat*)dh_last, dq, geo);
          inc_h = (const cfloat*)carry_a;
          inc_u = (const cfloat*)carry_b;
        }
        cema_bwd_fwd_final_t<T, NSPLIT><<<grid, nthr, 0, st>>>(
            (const T*)dy, (const T*)x, p, qc, gc, inc_h, inc_u, (const cfloat*)hx, (const cfloat*)dh_last,
            dgamma, dq, geo);
      });
    });
    return;
  }
  MB_DISPATCH_DTYPE(x_dtype, {
    using T = scalar_t;
    CEMA_SWITCH(N, {
      dim3 grid(div_up((long long)D * NSPLIT, kCemaThreads), geo.S, B);
      // adjoint pass
      const cfloat* inc = nullptr;
      if (geo.S > 1) {
        cema_bwd_rev_local<T, NPT, NSPLIT><<<grid, kCemaThreads, 0, st>>>((const T*)dy, p, qc, gc, (cfloat*)carry_a, geo);
        cema_combine<<<div_up(nbd, 256), 256, 0, st>>>((cfloat*)carry_a, qc, (const cfloat*)dh_last,
                                                       (cfloat*)dhx, geo, true);
        inc = (const cfloat*)carry_a;
      }
      cema_bwd_rev_final<T, NPT, NSPLIT><<<grid, kCemaThreads, 0, st>>>(
          (const T*)dy, (const T*)x, p, qc, gc, omega, inc, (const cfloat*)dh_last, (T*)dx, dp, domega,
          (cfloat*)dhx, geo);
      // forward-time pass for dgamma, dq
      const cfloat* inc_h = nullptr;
      const cfloat* inc_u = nullptr;
      if (geo.S > 1) {
        cema_bwd_fwd_local<T, NPT, NSPLIT><<<grid, kCemaThreads, 0, st>>>((const T*)x, p, qc, gc, (cfloat*)carry_a,
                                                                        (cfloat*)carry_b, geo);
        cema_bwd_fwd_combine<<<div_up(nbd, 256), 256, 0, st>>>((cfloat*)carry_a, (cfloat*)carry_b, qc,
                                                               (const cfloat*)hx, (const cfloat*)dh_last, dq, geo);
        inc_h = (const cfloat*)carry_a;
        inc_u = (const cfloat*)carry_b;
      }
      cema_bwd_fwd_final<T, NPT, NSPLIT><<<grid, kCemaThreads, 0, st>>>(
          (const T*)dy, (const T*)x, p, qc, gc, inc_h, inc_u, (const cfloat*)hx, (const cfloat*)dh_last,
          dgamma, dq, geo);
    });
  });
}

}  // namespace mb
