// TimestepNorm: group normalisation with statistics that are cumulative over
// time (position t is normalised by the mean/variance of all positions <= t of
// its sequence, seeded with carried statistics).
//
// Semantics follow the reference's CPU implementation
// (csrc/ops/timestep_norm.cc:218-450): at step t the D = H/G features of a group
// give one sample (gu, gv) of weight one that is merged into the running
// population (count, mean, var); padded steps output zero and do not advance
// the statistics.
//
// Design (differs from the reference's Welford-state Blelloch scan): merging
// populations is associative, so the running moments are prefix sums of the
// first and second moments.  Those are accumulated in fp64, which makes the
// closed form as accurate as the compensated fp32 Welford recurrence while
// letting a (group x segment) thread block scan a sequence in two short passes.
//
//   forward : group_stats -> scan -> apply
//   backward: group_grads -> reverse affine scan -> apply (+ dgamma / dbeta)
//
// The backward recurrence on (d mean, d var) is affine with a 2x2 upper
// triangular matrix with equal diagonal, a family closed under composition, so
// the reverse scan composes (a, b, o1, o2) quadruples per segment.
#include "common.cuh"
#include "kernels.h"

namespace mb {
namespace {

constexpr int kSeg = 32;  // segments per sequence in the scan kernels (threadIdx.y)

template <typename T, int LPG>
__global__ void tsn_group_stats_kernel(const T* __restrict__ x, float* __restrict__ gu,
                                       float* __restrict__ gv, long long rows, int H, int G) {
  const int Dg = H / G;
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long grp = gid / LPG;  // (row, g) flattened
  const int l = (int)(gid % LPG);
  const bool live = grp < rows * G;
  const T* p = x + (live ? grp : 0) * Dg;  // groups are contiguous: row*H + g*Dg == grp*Dg
  float s = 0.f;
  if (live)
    for (int k = l; k < Dg; k += LPG) s += to_f(p[k]);
  s = subwarp_sum<LPG>(s);
  const float mean = s / Dg;
  float q = 0.f;
  if (live)
    for (int k = l; k < Dg; k += LPG) {
      const float d = to_f(p[k]) - mean;
      q += d * d;
    }
  q = subwarp_sum<LPG>(q);
  if (live && l == 0) {
    gu[grp] = mean;
    gv[grp] = q / Dg;
  }
}

// grid (ceil(G/32), B), block (32, kSeg)
template <typename T>
__global__ void tsn_scan_kernel(const float* __restrict__ gu, const float* __restrict__ gv,
                                const bool* __restrict__ mask, const long long* __restrict__ prev_count,
                                const T* __restrict__ prev_mean, const T* __restrict__ prev_var,
                                float* __restrict__ cummean, float* __restrict__ cumrstd,
                                long long* __restrict__ count_out, T* __restrict__ mean_out,
                                T* __restrict__ var_out, int L, int G, float eps) {
  __shared__ double sh_n[kSeg][32], sh_a[kSeg][32], sh_b[kSeg][32];
  const int b = blockIdx.y;
  const int g = blockIdx.x * 32 + threadIdx.x;
  const int s = threadIdx.y;
  const bool live = g < G;
  const int Ls = (L + kSeg - 1) / kSeg;
  const int t0 = min(L, s * Ls), t1 = min(L, t0 + Ls);
  const float* gub = gu + (long long)b * L * G;
  const float* gvb = gv + (long long)b * L * G;
  const bool* mb_ = mask ? mask + (long long)b * L : nullptr;

  double n = 0, a = 0, c = 0;
  if (live) {
    for (int t = t0; t < t1; ++t) {
      if (mb_ && mb_[t]) continue;
      const double u = gub[(long long)t * G + g], v = gvb[(long long)t * G + g];
      n += 1.0;
      a += u;
      c += v + u * u;
    }
  }
  sh_n[s][threadIdx.x] = n;
  sh_a[s][threadIdx.x] = a;
  sh_b[s][threadIdx.x] = c;
  __syncthreads();
  if (!live) return;
  const double n0 = (double)prev_count[b];
  const double u0 = to_f(prev_mean[(long long)b * G + g]);
  const double v0 = to_f(prev_var[(long long)b * G + g]);
  double cn = n0, s1 = n0 * u0, s2 = n0 * (v0 + u0 * u0);
  for (int k = 0; k < s; ++k) {
    cn += sh_n[k][threadIdx.x];
    s1 += sh_a[k][threadIdx.x];
    s2 += sh_b[k][threadIdx.x];
  }
  double mean = cn > 0.5 ? s1 / cn : u0;
  double var = cn > 0.5 ? fmax(s2 / cn - mean * mean, 0.0) : v0;
  float* cm = cummean + (long long)b * L * G;
  float* cr = cumrstd + (long long)b * L * G;
  for (int t = t0; t < t1; ++t) {
    if (!(mb_ && mb_[t])) {
      const double u = gub[(long long)t * G + g], v = gvb[(long long)t * G + g];
      cn += 1.0;
      s1 += u;
      s2 += v + u * u;
      mean = s1 / cn;
      var = fmax(s2 / cn - mean * mean, 0.0);
    }
    // padded steps keep the running values, so cummean[t-1] is always the
    // state *before* step t (the backward pass relies on that)
    cm[(long long)t * G + g] = (float)mean;
    cr[(long long)t * G + g] = (float)(1.0 / sqrt(var + (double)eps));
  }
  if (s == kSeg - 1) {
    mean_out[(long long)b * G + g] = from_f<T>((float)mean);
    var_out[(long long)b * G + g] = from_f<T>((float)var);
    if (g == 0) count_out[b] = (long long)(cn + 0.5);
  }
}

template <typename T, typename W>
__global__ void tsn_apply_kernel(const T* __restrict__ x, const float* __restrict__ cummean,
                                 const float* __restrict__ cumrstd, const W* __restrict__ gamma,
                                 float gamma_offset, const W* __restrict__ beta,
                                 const bool* __restrict__ mask, T* __restrict__ y, long long rows, int H,
                                 int G) {
  const int Dg = H / G;
  const long long total = rows * H;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / H;
    const int j = (int)(i - row * H);
    float out = 0.f;
    if (!(mask && mask[row])) {
      const long long sg = row * G + j / Dg;
      out = (to_f(x[i]) - cummean[sg]) * cumrstd[sg] * (to_f(gamma[j]) + gamma_offset) + to_f(beta[j]);
    }
    y[i] = from_f<T>(out);
  }
}

// ----------------------------------------------------------------------------- backward
template <typename T, typename W, int LPG>
__global__ void tsn_group_grads_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                       const float* __restrict__ cummean, const W* __restrict__ gamma,
                                       float gamma_offset, float* __restrict__ ux, float* __restrict__ ds,
                                       float* __restrict__ db, long long rows, int H, int G) {
  const int Dg = H / G;
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long grp = gid / LPG;
  const int l = (int)(gid % LPG);
  const bool live = grp < rows * G;
  const long long base = (live ? grp : 0) * Dg;
  const int g = (int)((live ? grp : 0) % G);
  const float u = cummean[live ? grp : 0];
  float sx = 0.f, s1 = 0.f, s2 = 0.f;
  if (live)
    for (int k = l; k < Dg; k += LPG) {
      const float xv = to_f(x[base + k]);
      const float gw = to_f(dy[base + k]) * (to_f(gamma[g * Dg + k]) + gamma_offset);
      sx += xv;
      s1 += gw * (xv - u);
      s2 += gw;
    }
  sx = subwarp_sum<LPG>(sx);
  s1 = subwarp_sum<LPG>(s1);
  s2 = subwarp_sum<LPG>(s2);
  if (live && l == 0) {
    ux[grp] = sx / Dg;
    ds[grp] = s1;
    db[grp] = s2;
  }
}

struct Affine {  // [u; v] -> [[a, b], [0, a]] [u; v] + [o1; o2]
  double a, b, o1, o2;
};
__device__ __forceinline__ Affine affine_identity() { return {1.0, 0.0, 0.0, 0.0}; }
// result = second o first  (apply `first`, then `second`)
__device__ __forceinline__ Affine affine_compose(const Affine& second, const Affine& first) {
  return {second.a * first.a, second.a * first.b + second.b * first.a,
          second.a * first.o1 + second.b * first.o2 + second.o1, second.a * first.o2 + second.o2};
}

template <typename T>
__global__ void tsn_bwd_scan_kernel(const float* __restrict__ ux, const float* __restrict__ ds,
                                    const float* __restrict__ db, const float* __restrict__ cummean,
                                    const float* __restrict__ cumrstd, const bool* __restrict__ mask,
                                    const long long* __restrict__ count_final,
                                    const T* __restrict__ prev_mean, const T* __restrict__ dmean_out,
                                    const T* __restrict__ dvar_out, float* __restrict__ dux,
                                    float* __restrict__ dvx, T* __restrict__ dprev_mean,
                                    T* __restrict__ dprev_var, int L, int G) {
  __shared__ double sh[4][kSeg][32];
  __shared__ int sh_valid[kSeg];
  const int b = blockIdx.y;
  const int g = blockIdx.x * 32 + threadIdx.x;
  const int s = threadIdx.y;
  const bool live = g < G;
  const int Ls = (L + kSeg - 1) / kSeg;
  const int t0 = min(L, s * Ls), t1 = min(L, t0 + Ls);
  const bool* mb_ = mask ? mask + (long long)b * L : nullptr;
  const long long off = (long long)b * L * G;

  // number of valid steps in each segment (needed to recover the running count)
  if (threadIdx.x == 0) {
    int nv = 0;
    for (int t = t0; t < t1; ++t) nv += !(mb_ && mb_[t]);
    sh_valid[s] = nv;
  }
  __syncthreads();
  // count *including* the last step of this segment
  long long cnt_end = count_final[b];
  for (int k = kSeg - 1; k > s; --k) cnt_end -= sh_valid[k];

  const double pm = live ? (double)to_f(prev_mean[(long long)b * G + g]) : 0.0;

  auto step_map = [&](int t, double m0) -> Affine {
    const long long i = off + (long long)t * G + g;
    const double c1 = (m0 - 1.0) / m0, c2 = 1.0 / m0;
    const double prev_u = t == 0 ? pm : (double)cummean[i - G];
    const double delta = (double)ux[i] - prev_u;
    const double r = cumrstd[i];
    const double r3ds = r * r * r * (double)ds[i];
    Affine m;
    m.a = c1;
    m.b = -2.0 * c1 * c2 * delta;
    m.o1 = -c1 * r * (double)db[i] + c1 * c2 * delta * r3ds;
    m.o2 = -0.5 * c1 * r3ds;
    return m;
  };

  Affine seg = affine_identity();
  if (live) {
    long long m0 = cnt_end;
    for (int t = t1 - 1; t >= t0; --t) {
      if (mb_ && mb_[t]) continue;
      seg = affine_compose(step_map(t, (double)m0), seg);
      --m0;
    }
  }
  sh[0][s][threadIdx.x] = seg.a;
  sh[1][s][threadIdx.x] = seg.b;
  sh[2][s][threadIdx.x] = seg.o1;
  sh[3][s][threadIdx.x] = seg.o2;
  __syncthreads();
  if (!live) return;

  double u = to_f(dmean_out[(long long)b * G + g]);
  double v = to_f(dvar_out[(long long)b * G + g]);
  for (int k = kSeg - 1; k > s; --k) {
    const double a = sh[0][k][threadIdx.x], bb = sh[1][k][threadIdx.x];
    const double nu = a * u + bb * v + sh[2][k][threadIdx.x];
    v = a * v + sh[3][k][threadIdx.x];
    u = nu;
  }
  long long m0 = cnt_end;
  for (int t = t1 - 1; t >= t0; --t) {
    const long long i = off + (long long)t * G + g;
    if (mb_ && mb_[t]) {
      dux[i] = 0.f;
      dvx[i] = 0.f;
      continue;
    }
    const double md = (double)m0;
    const double c1 = (md - 1.0) / md, c2 = 1.0 / md;
    const double prev_u = t == 0 ? pm : (double)cummean[i - G];
    const double delta = (double)ux[i] - prev_u;
    const double r = cumrstd[i];
    const double du = u - r * (double)db[i];
    const double dv = v - 0.5 * r * r * r * (double)ds[i];
    dux[i] = (float)(c2 * du + 2.0 * c1 * c2 * dv * delta);
    dvx[i] = (float)(c2 * dv);
    u = c1 * du - 2.0 * c1 * c2 * dv * delta;
    v = c1 * dv;
    --m0;
  }
  if (s == 0) {
    dprev_mean[(long long)b * G + g] = from_f<T>((float)u);
    dprev_var[(long long)b * G + g] = from_f<T>((float)v);
  }
}

constexpr int kBwdCols = 32;
constexpr int kBwdThreads = 256;   // block size of tsn_bwd_apply_kernel

// One CTA walks a strip of rows; thread t owns columns t, t+blockDim, ...
template <typename T, typename W>
__global__ void tsn_bwd_apply_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                     const float* __restrict__ cummean, const float* __restrict__ cumrstd,
                                     const float* __restrict__ ux, const float* __restrict__ dux,
                                     const float* __restrict__ dvx, const W* __restrict__ gamma,
                                     float gamma_offset, const bool* __restrict__ mask, T* __restrict__ dx,
                                     float* __restrict__ dgamma, float* __restrict__ dbeta, long long rows,
                                     int H, int G) {
  const int Dg = H / G;
  const float inv_d = 1.f / Dg;
  float acc_g[kBwdCols], acc_b[kBwdCols];
#pragma unroll
  for (int i = 0; i < kBwdCols; ++i) acc_g[i] = acc_b[i] = 0.f;
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const bool pad = mask && mask[row];
#pragma unroll
    for (int i = 0; i < kBwdCols; ++i) {    // fixed trip count keeps the accumulators in registers
      const int j = threadIdx.x + i * kBwdThreads;
      if (j >= H) continue;
      const long long e = row * H + j;
      float out = 0.f;
      if (!pad) {
        const long long sg = row * G + j / Dg;
        const float g = to_f(dy[e]), xv = to_f(x[e]);
        const float r = cumrstd[sg], u = cummean[sg];
        out = g * r * (to_f(gamma[j]) + gamma_offset) + (dux[sg] + 2.f * dvx[sg] * (xv - ux[sg])) * inv_d;
        acc_g[i] += g * (xv - u) * r;
        acc_b[i] += g;
      }
      dx[e] = from_f<T>(out);
    }
  }
#pragma unroll
  for (int i = 0; i < kBwdCols; ++i) {
    const int j = threadIdx.x + i * kBwdThreads;
    if (j < H) {
      atomicAdd(dgamma + j, acc_g[i]);
      atomicAdd(dbeta + j, acc_b[i]);
    }
  }
}

int pick_lpg(int Dg) {
  int l = 1;
  while (l * 2 <= Dg && l < 32) l *= 2;
  return l;
}

#define LPG_SWITCH(lpg, ...)                          \
  switch (lpg) {                                      \
    case 1: { constexpr int LPG = 1; __VA_ARGS__; } break;   \
    case 2: { constexpr int LPG = 2; __VA_ARGS__; } break;   \
    case 4: { constexpr int LPG = 4; __VA_ARGS__; } break;   \
    case 8: { constexpr int LPG = 8; __VA_ARGS__; } break;   \
    case 16: { constexpr int LPG = 16; __VA_ARGS__; } break; \
    default: { constexpr int LPG = 32; __VA_ARGS__; } break; \
  }

}  // namespace

#define TSN_DISPATCH(xd, wd, ...)                                    \
  MB_DISPATCH_DTYPE(xd, {                                            \
    using T = scalar_t;                                              \
    if ((wd) == kF32) {                                              \
      using W = float;                                               \
      __VA_ARGS__;                                                   \
    } else {                                                         \
      using W = T;                                                   \
      __VA_ARGS__;                                                   \
    }                                                                \
  })

void timestep_norm_fwd(const void* x, const long long* prev_count, const void* prev_mean,
                       const void* prev_var, const void* gamma, float gamma_offset, const void* beta,
                       const bool* mask, void* y, long long* count_out, void* mean_out, void* var_out,
                       float* cummean, float* cumrstd, float* gu, float* gv, int B, int L, int H, int G,
                       float eps, int x_dtype, int w_dtype, cudaStream_t st) {
  const long long rows = (long long)B * L;
  const int lpg = pick_lpg(H / G);
  TSN_DISPATCH(x_dtype, w_dtype, {
    LPG_SWITCH(lpg, {
      const long long threads = rows * G * LPG;
      tsn_group_stats_kernel<T, LPG><<<div_up(threads, 256), 256, 0, st>>>((const T*)x, gu, gv, rows, H, G);
    });
    tsn_scan_kernel<T><<<dim3(div_up(G, 32), B), dim3(32, kSeg), 0, st>>>(
        gu, gv, mask, prev_count, (const T*)prev_mean, (const T*)prev_var, cummean, cumrstd, count_out,
        (T*)mean_out, (T*)var_out, L, G, eps);
    const int grid = (int)std::min<long long>(div_up(rows * H, 256), 148LL * 16);
    tsn_apply_kernel<T, W><<<grid, 256, 0, st>>>((const T*)x, cummean, cumrstd, (const W*)gamma,
                                                 gamma_offset, (const W*)beta, mask, (T*)y, rows, H, G);
  });
}

void timestep_norm_bwd(const void* dy, const void* dmean_out, const void* dvar_out, const void* x,
                       const void* prev_mean, const long long* count_final, const float* cummean,
                       const float* cumrstd, const void* gamma, float gamma_offset, const bool* mask,
                       void* dx, void* dprev_mean, void* dprev_var, float* dgamma, float* dbeta,
                       float* ux, float* ds, float* db, float* dux, float* dvx, int B, int L, int H, int G,
                       int x_dtype, int w_dtype, cudaStream_t st) {
  const long long rows = (long long)B * L;
  const int lpg = pick_lpg(H / G);
  TSN_DISPATCH(x_dtype, w_dtype, {
    LPG_SWITCH(lpg, {
      const long long threads = rows * G * LPG;
      tsn_group_grads_kernel<T, W, LPG><<<div_up(threads, 256), 256, 0, st>>>(
          (const T*)dy, (const T*)x, cummean, (const W*)gamma, gamma_offset, ux, ds, db, rows, H, G);
    });
    tsn_bwd_scan_kernel<T><<<dim3(div_up(G, 32), B), dim3(32, kSeg), 0, st>>>(
        ux, ds, db, cummean, cumrstd, mask, count_final, (const T*)prev_mean, (const T*)dmean_out,
        (const T*)dvar_out, dux, dvx, (T*)dprev_mean, (T*)dprev_var, L, G);
    const int grid = (int)std::min<long long>(rows, 148LL * 4);
    tsn_bwd_apply_kernel<T, W><<<grid, kBwdThreads, 0, st>>>((const T*)dy, (const T*)x, cummean, cumrstd, ux, dux,
                                                     dvx, (const W*)gamma, gamma_offset, mask, (T*)dx,
                                                     dgamma, dbeta, rows, H, G);
  });
}

}  // namespace mb
