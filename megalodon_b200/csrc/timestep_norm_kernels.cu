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

#include <initializer_list>

namespace mb {
namespace {

constexpr int kSegLen = 32;  // time steps per scan segment

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

// ---- forward scan in three small kernels over segments of kSegLen steps:
//   seg_sums   : (b, seg, g)  sums of (1, gu, gv + gu^2) over the segment's valid steps
//   seg_prefix : (b, g)       exclusive prefix over segments, seeded with the carried statistics
//   seg_apply  : (b, seg, g)  running mean / rstd inside the segment
// Threads are consecutive in g, so every access is coalesced, and no thread
// walks more than kSegLen (or L / kSegLen) dependent steps.
__global__ void tsn_seg_sums_kernel(const float* __restrict__ gu, const float* __restrict__ gv,
                                    const bool* __restrict__ mask, double* __restrict__ seg, int B, int L,
                                    int G, int nseg) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)B * nseg * G) return;
  const int g = (int)(i % G);
  const int sgi = (int)((i / G) % nseg);
  const int b = (int)(i / ((long long)G * nseg));
  const int t0 = sgi * kSegLen, t1 = min(L, t0 + kSegLen);
  const float* gub = gu + (long long)b * L * G + g;
  const float* gvb = gv + (long long)b * L * G + g;
  const bool* mb_ = mask ? mask + (long long)b * L : nullptr;
  double n = 0, a = 0, c = 0;
#pragma unroll 8
  for (int t = t0; t < t1; ++t) {
    const double u = gub[(long long)t * G], v = gvb[(long long)t * G];
    const double w = (mb_ && mb_[t]) ? 0.0 : 1.0;
    n += w;
    a += w * u;
    c += w * (v + u * u);
  }
  const long long total = (long long)B * nseg * G;
  seg[i] = n;
  seg[total + i] = a;
  seg[2 * total + i] = c;
}

template <typename T>
__global__ void tsn_seg_prefix_kernel(double* __restrict__ seg, const long long* __restrict__ prev_count,
                                      const T* __restrict__ prev_mean, const T* __restrict__ prev_var,
                                      long long* __restrict__ count_out, T* __restrict__ mean_out,
                                      T* __restrict__ var_out, int B, int G, int nseg) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= B * G) return;
  const int g = i % G, b = i / G;
  const long long total = (long long)B * nseg * G;
  const double n0 = (double)prev_count[b];
  const double u0 = to_f(prev_mean[i]), v0 = to_f(prev_var[i]);
  double cn = n0, s1 = n0 * u0, s2 = n0 * (v0 + u0 * u0);
#pragma unroll 4
  for (int k = 0; k < nseg; ++k) {
    const long long idx = ((long long)b * nseg + k) * G + g;
    const double dn = seg[idx], da = seg[total + idx], dc = seg[2 * total + idx];
    seg[idx] = cn;
    seg[total + idx] = s1;
    seg[2 * total + idx] = s2;
    cn += dn;
    s1 += da;
    s2 += dc;
  }
  double mean = u0, var = v0;
  if (cn > 0.5) {
    mean = s1 / cn;
    var = fmax(s2 / cn - mean * mean, 0.0);
  }
  mean_out[i] = from_f<T>((float)mean);
  var_out[i] = from_f<T>((float)var);
  if (g == 0) count_out[b] = (long long)(cn + 0.5);
}

template <typename T>
__global__ void tsn_seg_apply_kernel(const float* __restrict__ gu, const float* __restrict__ gv,
                                     const bool* __restrict__ mask, const double* __restrict__ seg,
                                     const T* __restrict__ prev_mean, const T* __restrict__ prev_var,
                                     float* __restrict__ cummean, float* __restrict__ cumrstd, int B, int L,
                                     int G, int nseg, float eps) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)B * nseg * G;
  if (i >= total) return;
  const int g = (int)(i % G);
  const int sgi = (int)((i / G) % nseg);
  const int b = (int)(i / ((long long)G * nseg));
  const int t0 = sgi * kSegLen, t1 = min(L, t0 + kSegLen);
  const long long off = (long long)b * L * G + g;
  const bool* mb_ = mask ? mask + (long long)b * L : nullptr;
  double cn = seg[i], s1 = seg[total + i], s2 = seg[2 * total + i];
  double mean = to_f(prev_mean[b * G + g]), var = to_f(prev_var[b * G + g]);
  if (cn > 0.5) {
    mean = s1 / cn;
    var = fmax(s2 / cn - mean * mean, 0.0);
  }
  for (int tb = t0; tb < t1; tb += 8) {
    float us[8], vs[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const bool in = tb + j < t1;
      us[j] = in ? gu[off + (long long)(tb + j) * G] : 0.f;
      vs[j] = in ? gv[off + (long long)(tb + j) * G] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int t = tb + j;
      if (t >= t1) break;
      if (!(mb_ && mb_[t])) {
        const double u = us[j], v = vs[j];
        cn += 1.0;
        s1 += u;
        s2 += v + u * u;
        mean = s1 / cn;
        var = fmax(s2 / cn - mean * mean, 0.0);
      }
      // padded steps keep the running values, so cummean[t-1] is always the
      // state *before* step t (the backward pass relies on that)
      cummean[off + (long long)t * G] = (float)mean;
      cumrstd[off + (long long)t * G] = (float)(1.0 / sqrt(var + (double)eps));
    }
  }
}

// ---- the same scan as ONE kernel when a sequence's segments fit one CTA (L <= 16384): a CTA owns GT
// groups of one batch row, thread (segment, group) keeps its kSegLen samples in registers, the exclusive
// prefix over segments runs in shared memory (log2(nseg) doubling steps), and the running statistics are
// written from the registers.  Three dependent launches and the round trip of the segment sums through
// global memory become one launch.
constexpr int kScanMaxThreads = 512;   // 128 registers per thread: the segment's samples stay in registers

template <typename T>
__global__ void __launch_bounds__(kScanMaxThreads)
tsn_scan_fused_kernel(const float* __restrict__ gu, const float* __restrict__ gv, const bool* __restrict__ mask,
                      const long long* __restrict__ prev_count, const T* __restrict__ prev_mean,
                      const T* __restrict__ prev_var, long long* __restrict__ count_out, T* __restrict__ mean_out,
                      T* __restrict__ var_out, float* __restrict__ cummean, float* __restrict__ cumrstd, int L, int G,
                      int nseg, int GT, float eps) {
  __shared__ double sh[3][kScanMaxThreads];
  const int tid = threadIdx.x;
  const int gl = tid % GT, sgi = tid / GT;
  const int g = blockIdx.x * GT + gl, b = blockIdx.y;
  const bool live = g < G;
  const int t0 = sgi * kSegLen, t1 = min(L, t0 + kSegLen);
  const long long off = (long long)b * L * G + (live ? g : 0);
  const bool* mb_ = mask ? mask + (long long)b * L : nullptr;
  float us[kSegLen], vs[kSegLen];
  unsigned valid = 0;   // bit j: step t0 + j exists and is not padded
  double n = 0, a = 0, c = 0;
#pragma unroll
  for (int j = 0; j < kSegLen; ++j) {
    const int t = t0 + j;
    const bool in = live && t < t1;
    us[j] = in ? gu[off + (long long)t * G] : 0.f;
    vs[j] = in ? gv[off + (long long)t * G] : 0.f;
    if (in && !(mb_ && mb_[t])) valid |= 1u << j;
  }
#pragma unroll
  for (int j = 0; j < kSegLen; ++j)
    if (valid >> j & 1u) {
      const double u = us[j], v = vs[j];
      n += 1.0;
      a += u;
      c += v + u * u;
    }
  sh[0][tid] = n;
  sh[1][tid] = a;
  sh[2][tid] = c;
  __syncthreads();
  for (int step = 1; step < nseg; step <<= 1) {   // inclusive prefix over segments, per group
    double tn = 0, ta = 0, tc = 0;
    if (sgi >= step) {
      tn = sh[0][tid - step * GT];
      ta = sh[1][tid - step * GT];
      tc = sh[2][tid - step * GT];
    }
    __syncthreads();
    if (sgi >= step) {
      sh[0][tid] += tn;
      sh[1][tid] += ta;
      sh[2][tid] += tc;
    }
    __syncthreads();
  }
  if (!live) return;
  const double n0 = (double)prev_count[b];
  const double u0 = to_f(prev_mean[b * G + g]), v0 = to_f(prev_var[b * G + g]);
  double cn = n0, s1 = n0 * u0, s2 = n0 * (v0 + u0 * u0);
  if (sgi == nseg - 1) {   // the sequence's final statistics
    const double fn = cn + sh[0][tid], f1 = s1 + sh[1][tid], f2 = s2 + sh[2][tid];
    double mean = u0, var = v0;
    if (fn > 0.5) {
      mean = f1 / fn;
      var = fmax(f2 / fn - mean * mean, 0.0);
    }
    mean_out[b * G + g] = from_f<T>((float)mean);
    var_out[b * G + g] = from_f<T>((float)var);
    if (g == 0) count_out[b] = (long long)(fn + 0.5);
  }
  if (sgi > 0) {
    cn += sh[0][tid - GT];
    s1 += sh[1][tid - GT];
    s2 += sh[2][tid - GT];
  }
  double mean = u0, var = v0;
  if (cn > 0.5) {
    mean = s1 / cn;
    var = fmax(s2 / cn - mean * mean, 0.0);
  }
#pragma unroll
  for (int j = 0; j < kSegLen; ++j) {
    const int t = t0 + j;
    if (t >= t1) break;
    if (valid >> j & 1u) {
      const double u = us[j], v = vs[j];
      cn += 1.0;
      s1 += u;
      s2 += v + u * u;
      mean = s1 / cn;
      var = fmax(s2 / cn - mean * mean, 0.0);
    }
    cummean[off + (long long)t * G] = (float)mean;
    cumrstd[off + (long long)t * G] = (float)(1.0 / sqrt(var + (double)eps));
  }
}

// groups per CTA of the fused scans: as many as keep the CTA near 512 threads (0: the sequence is too long)
inline int tsn_fused_groups(int nseg) {
  if (nseg > kScanMaxThreads) return 0;
  int gt = 1;
  while (gt * 2 * nseg <= kScanMaxThreads && gt < 32) gt *= 2;
  return gt;
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

// running count *including* step t
__device__ __forceinline__ double count_at(const int* cumvalid, long long first_count, int b, int L, int t) {
  return cumvalid ? (double)(first_count + cumvalid[(long long)b * L + t]) : (double)(first_count + t + 1);
}

// inclusive prefix count of non-padded steps, one thread per batch row (only used with a padding mask)
__global__ void tsn_cumvalid_kernel(const bool* __restrict__ mask, int* __restrict__ cumvalid, int B, int L) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  int c = 0;
  for (int t = 0; t < L; ++t) {
    c += mask[(long long)b * L + t] ? 0 : 1;
    cumvalid[(long long)b * L + t] = c;
  }
}

struct StepIn {
  const float *ux, *ds, *db, *cummean, *cumrstd;
};

__device__ __forceinline__ Affine tsn_step_map(const StepIn& in, long long i, int G, int t, double pm, double m0) {
  const double c1 = (m0 - 1.0) / m0, c2 = 1.0 / m0;
  const double prev_u = t == 0 ? pm : (double)in.cummean[i - G];
  const double delta = (double)in.ux[i] - prev_u;
  const double r = in.cumrstd[i];
  const double r3ds = r * r * r * (double)in.ds[i];
  Affine m;
  m.a = c1;
  m.b = -2.0 * c1 * c2 * delta;
  m.o1 = -c1 * r * (double)in.db[i] + c1 * c2 * delta * r3ds;
  m.o2 = -0.5 * c1 * r3ds;
  return m;
}

// (b, seg, g): composite map of the segment's valid steps, taken from its last step to its first
template <typename T>
__global__ void tsn_bwd_seg_maps_kernel(StepIn in, const bool* __restrict__ mask, const int* __restrict__ cumvalid,
                                        const long long* __restrict__ count_final,
                                        const T* __restrict__ prev_mean, double* __restrict__ maps, int B, int L,
                                        int G, int nseg) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)B * nseg * G;
  if (i >= total) return;
  const int g = (int)(i % G);
  const int sgi = (int)((i / G) % nseg);
  const int b = (int)(i / ((long long)G * nseg));
  const int t0 = sgi * kSegLen, t1 = min(L, t0 + kSegLen);
  const bool* mb_ = mask ? mask + (long long)b * L : nullptr;
  const long long first = count_final[b] - (cumvalid ? cumvalid[(long long)b * L + L - 1] : L);
  const double pm = to_f(prev_mean[b * G + g]);
  const long long off = (long long)b * L * G + g;
  Affine seg = affine_identity();
  for (int t = t1 - 1; t >= t0; --t) {
    if (mb_ && mb_[t]) continue;
    seg = affine_compose(tsn_step_map(in, off + (long long)t * G, G, t, pm, count_at(cumvalid, first, b, L, t)), seg);
  }
  maps[i] = seg.a;
  maps[total + i] = seg.b;
  maps[2 * total + i] = seg.o1;
  maps[3 * total + i] = seg.o2;
}

// (b, g): walk the segments from last to first; leaves each segment's incoming (u, v) in maps[0], maps[1]
template <typename T>
__global__ void tsn_bwd_seg_prefix_kernel(double* __restrict__ maps, const T* __restrict__ dmean_out,
                                          const T* __restrict__ dvar_out, T* __restrict__ dprev_mean,
                                          T* __restrict__ dprev_var, int B, int G, int nseg) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= B * G) return;
  const int g = i % G, b = i / G;
  const long long total = (long long)B * nseg * G;
  double u = to_f(dmean_out[i]), v = to_f(dvar_out[i]);
#pragma unroll 4
  for (int k = nseg - 1; k >= 0; --k) {
    const long long idx = ((long long)b * nseg + k) * G + g;
    const double a = maps[idx], bb = maps[total + idx], o1 = maps[2 * total + idx], o2 = maps[3 * total + idx];
    maps[idx] = u;
    maps[total + idx] = v;
    const double nu = a * u + bb * v + o1;
    v = a * v + o2;
    u = nu;
  }
  dprev_mean[i] = from_f<T>((float)u);
  dprev_var[i] = from_f<T>((float)v);
}

// (b, seg, g): replay the segment from its incoming state and emit d(ux), d(vx) per step
template <typename T>
__global__ void tsn_bwd_seg_apply_kernel(StepIn in, const bool* __restrict__ mask, const int* __restrict__ cumvalid,
                                         const long long* __restrict__ count_final,
                                         const T* __restrict__ prev_mean, const double* __restrict__ maps,
                                         float* __restrict__ dux, float* __restrict__ dvx, int B, int L, int G,
                                         int nseg) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)B * nseg * G;
  if (i >= total) return;
  const int g = (int)(i % G);
  const int sgi = (int)((i / G) % nseg);
  const int b = (int)(i / ((long long)G * nseg));
  const int t0 = sgi * kSegLen, t1 = min(L, t0 + kSegLen);
  const bool* mb_ = mask ? mask + (long long)b * L : nullptr;
  const long long first = count_final[b] - (cumvalid ? cumvalid[(long long)b * L + L - 1] : L);
  const double pm = to_f(prev_mean[b * G + g]);
  const long long off = (long long)b * L * G + g;
  double u = maps[i], v = maps[total + i];
  for (int t = t1 - 1; t >= t0; --t) {
    const long long e = off + (long long)t * G;
    if (mb_ && mb_[t]) {
      dux[e] = 0.f;
      dvx[e] = 0.f;
      continue;
    }
    const double md = count_at(cumvalid, first, b, L, t);
    const double c1 = (md - 1.0) / md, c2 = 1.0 / md;
    const double prev_u = t == 0 ? pm : (double)in.cummean[e - G];
    const double delta = (double)in.ux[e] - prev_u;
    const double r = in.cumrstd[e];
    const double du = u - r * (double)in.db[e];
    const double dv = v - 0.5 * r * r * r * (double)in.ds[e];
    dux[e] = (float)(c2 * du + 2.0 * c1 * c2 * dv * delta);
    dvx[e] = (float)(c2 * dv);
    u = c1 * du - 2.0 * c1 * c2 * dv * delta;
    v = c1 * dv;
  }
}

// The backward scan as ONE kernel under the same condition as the forward one: thread (segment, group)
// composes its segment's map, the suffix composition over segments runs in shared memory (the maps do not
// commute: the later segment's map is applied first), and the segment is replayed from its incoming state.
template <typename T>
__global__ void __launch_bounds__(kScanMaxThreads)
tsn_bwd_scan_fused_kernel(StepIn in, const bool* __restrict__ mask, const int* __restrict__ cumvalid,
                          const long long* __restrict__ count_final, const T* __restrict__ prev_mean,
                          const T* __restrict__ dmean_out, const T* __restrict__ dvar_out,
                          T* __restrict__ dprev_mean, T* __restrict__ dprev_var, float* __restrict__ dux,
                          float* __restrict__ dvx, int L, int G, int nseg, int GT) {
  __shared__ double sh[4][kScanMaxThreads];
  const int tid = threadIdx.x;
  const int gl = tid % GT, sgi = tid / GT;
  const int g = blockIdx.x * GT + gl, b = blockIdx.y;
  const bool live = g < G;
  const int t0 = sgi * kSegLen, t1 = min(L, t0 + kSegLen);
  const bool* mb_ = mask ? mask + (long long)b * L : nullptr;
  const long long first = count_final[b] - (cumvalid ? cumvalid[(long long)b * L + L - 1] : L);
  const double pm = live ? (double)to_f(prev_mean[b * G + g]) : 0.0;
  const long long off = (long long)b * L * G + (live ? g : 0);
  Affine seg = affine_identity();
  if (live)
    for (int t = t1 - 1; t >= t0; --t) {
      if (mb_ && mb_[t]) continue;
      seg = affine_compose(tsn_step_map(in, off + (long long)t * G, G, t, pm, count_at(cumvalid, first, b, L, t)), seg);
    }
  // position j = nseg - 1 - sgi counts the segments in the order the backward pass meets them
  const int j = nseg - 1 - sgi;
  const int slot = j * GT + gl;
  sh[0][slot] = seg.a;
  sh[1][slot] = seg.b;
  sh[2][slot] = seg.o1;
  sh[3][slot] = seg.o2;
  __syncthreads();
  for (int step = 1; step < nseg; step <<= 1) {   // inclusive: P[j] = M_j o M_{j-1} o ... o M_0
    Affine early = affine_identity(), late = affine_identity();
    if (j >= step) {
      const int e = slot - step * GT;
      early = {sh[0][e], sh[1][e], sh[2][e], sh[3][e]};
      late = {sh[0][slot], sh[1][slot], sh[2][slot], sh[3][slot]};
    }
    __syncthreads();
    if (j >= step) {
      const Affine r = affine_compose(late, early);
      sh[0][slot] = r.a;
      sh[1][slot] = r.b;
      sh[2][slot] = r.o1;
      sh[3][slot] = r.o2;
    }
    __syncthreads();
  }
  if (!live) return;
  const double iu = to_f(dmean_out[b * G + g]), iv = to_f(dvar_out[b * G + g]);
  if (sgi == 0) {   // every segment applied: the gradient of the carried statistics
    dprev_mean[b * G + g] = from_f<T>((float)(sh[0][slot] * iu + sh[1][slot] * iv + sh[2][slot]));
    dprev_var[b * G + g] = from_f<T>((float)(sh[0][slot] * iv + sh[3][slot]));
  }
  double u = iu, v = iv;
  if (j > 0) {
    const int e = slot - GT;
    u = sh[0][e] * iu + sh[1][e] * iv + sh[2][e];
    v = sh[0][e] * iv + sh[3][e];
  }
  for (int t = t1 - 1; t >= t0; --t) {
    const long long e = off + (long long)t * G;
    if (mb_ && mb_[t]) {
      dux[e] = 0.f;
      dvx[e] = 0.f;
      continue;
    }
    const double md = count_at(cumvalid, first, b, L, t);
    const double c1 = (md - 1.0) / md, c2 = 1.0 / md;
    const double prev_u = t == 0 ? pm : (double)in.cummean[e - G];
    const double delta = (double)in.ux[e] - prev_u;
    const double r = in.cumrstd[e];
    const double du = u - r * (double)in.db[e];
    const double dv = v - 0.5 * r * r * r * (double)in.ds[e];
    dux[e] = (float)(c2 * du + 2.0 * c1 * c2 * dv * delta);
    dvx[e] = (float)(c2 * dv);
    u = c1 * du - 2.0 * c1 * c2 * dv * delta;
    v = c1 * dv;
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

// ---------------------------------------------------------------- 16-byte variants of the four
// kernels that touch the activations.  A group of Dg features is read by VL = Dg / 8 adjacent lanes,
// one 8-element vector each, kept in registers (x is read once); needs Dg % 8 == 0, VL a power of
// two <= 32 and 32-byte aligned pointers.
template <typename T, int VL>
__global__ void tsn_group_stats_vec_kernel(const T* __restrict__ x, float* __restrict__ gu, float* __restrict__ gv,
                                           long long ngroups) {
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long grp = gid / VL;
  const int l = (int)(gid % VL);
  const bool live = grp < ngroups;
  float v[8];
  float s = 0.f;
  if (live) {
    load8(x + (grp * VL + l) * 8, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) s += v[j];
  }
  s = subwarp_sum<VL>(s);
  const float mean = s / (VL * 8);
  float q = 0.f;
  if (live) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float d = v[j] - mean;
      q = fmaf(d, d, q);
    }
  }
  q = subwarp_sum<VL>(q);
  if (live && l == 0) {
    gu[grp] = mean;
    gv[grp] = q / (VL * 8);
  }
}

template <typename T, typename W>
__global__ void tsn_apply_vec_kernel(const T* __restrict__ x, const float* __restrict__ cummean,
                                     const float* __restrict__ cumrstd, const W* __restrict__ gamma,
                                     float gamma_offset, const W* __restrict__ beta, const bool* __restrict__ mask,
                                     T* __restrict__ y, long long rows, int H, int G) {
  const int Dg = H / G;
  const int hv = H / 8;
  const long long total = rows * hv;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / hv;
    const int j0 = (int)(i - row * hv) * 8;
    float o[8];
    if (mask && mask[row]) {
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = 0.f;
    } else {
      const long long sg = row * G + j0 / Dg;
      const float u = cummean[sg], r = cumrstd[sg];
      float xv[8], gm[8], bt[8];
      load8(x + row * H + j0, xv);
      load8(gamma + j0, gm);
      load8(beta + j0, bt);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = fmaf((xv[j] - u) * r, gm[j] + gamma_offset, bt[j]);
    }
    store8(y + row * H + j0, o);
  }
}

template <typename T, typename W, int VL>
__global__ void tsn_group_grads_vec_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                           const float* __restrict__ cummean, const W* __restrict__ gamma,
                                           float gamma_offset, float* __restrict__ ux, float* __restrict__ ds,
                                           float* __restrict__ db, long long ngroups, int G) {
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long grp = gid / VL;
  const int l = (int)(gid % VL);
  const bool live = grp < ngroups;
  float sx = 0.f, s1 = 0.f, s2 = 0.f;
  if (live) {
    const int g = (int)(grp % G);
    const float u = cummean[grp];
    float xv[8], gy[8], gm[8];
    load8(x + (grp * VL + l) * 8, xv);
    load8(dy + (grp * VL + l) * 8, gy);
    load8(gamma + ((long long)g * VL + l) * 8, gm);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gw = gy[j] * (gm[j] + gamma_offset);
      sx += xv[j];
      s1 = fmaf(gw, xv[j] - u, s1);
      s2 += gw;
    }
  }
  sx = subwarp_sum<VL>(sx);
  s1 = subwarp_sum<VL>(s1);
  s2 = subwarp_sum<VL>(s2);
  if (live && l == 0) {
    ux[grp] = sx / (VL * 8);
    ds[grp] = s1;
    db[grp] = s2;
  }
}

// One CTA walks a strip of rows; thread t owns the 8-element column groups t, t + 256, ... (VPT of them)
template <typename T, typename W, int VPT>
__global__ void tsn_bwd_apply_vec_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                         const float* __restrict__ cummean, const float* __restrict__ cumrstd,
                                         const float* __restrict__ ux, const float* __restrict__ dux,
                                         const float* __restrict__ dvx, const W* __restrict__ gamma,
                                         float gamma_offset, const bool* __restrict__ mask, T* __restrict__ dx,
                                         float* __restrict__ dgamma, float* __restrict__ dbeta, long long rows,
                                         int H, int G, float* __restrict__ colsum_ws) {
  const int Dg = H / G;
  const int hv = H / 8;
  const float inv_d = 1.f / Dg;
  float acc_g[VPT][8], acc_b[VPT][8], gm[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * kBwdThreads;
    if (c < hv) {
      load8(gamma + c * 8, gm[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) gm[i][j] += gamma_offset;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) acc_g[i][j] = acc_b[i][j] = 0.f;
  }
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const bool pad = mask && mask[row];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * kBwdThreads;
      if (c >= hv) continue;
      const long long e = row * H + c * 8;
      float o[8];
      if (pad) {
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = 0.f;
      } else {
        const long long sg = row * G + (c * 8) / Dg;
        const float r = cumrstd[sg], u = cummean[sg], uxv = ux[sg];
        const float a = dux[sg] * inv_d, b2 = 2.f * dvx[sg] * inv_d;
        float gy[8], xv[8];
        load8(dy + e, gy);
        load8(x + e, xv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          o[j] = fmaf(gy[j] * r, gm[i][j], fmaf(b2, xv[j] - uxv, a));
          acc_g[i][j] = fmaf(gy[j] * r, xv[j] - u, acc_g[i][j]);
          acc_b[i][j] += gy[j];
        }
      }
      store8(dx + e, o);
    }
  }
  if (colsum_ws != nullptr) {   // one row of partial sums per CTA: [dgamma | dbeta]
    float* mine = colsum_ws + (long long)blockIdx.x * 2 * H;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * kBwdThreads;
      if (c < hv) {
        store8(mine + c * 8, acc_g[i]);
        store8(mine + H + c * 8, acc_b[i]);
      }
    }
    return;
  }
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * kBwdThreads;
    if (c < hv) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        atomicAdd(dgamma + c * 8 + j, acc_g[i][j]);
        atomicAdd(dbeta + c * 8 + j, acc_b[i][j]);
      }
    }
  }
}

inline bool tsn_vec_ok(int H, int G, std::initializer_list<const void*> ptrs) {
  const int Dg = H / G;
  const int vl = Dg / 8;
  if (Dg % 8 != 0 || vl > 32 || (vl & (vl - 1)) != 0 || H > kBwdThreads * 8 * 4) return false;
  for (const void* q : ptrs)
    if (q != nullptr && !aligned32(q)) return false;
  return true;
}

#define VL_SWITCH(vl, ...)                                   \
  switch (vl) {                                              \
    case 1: { constexpr int VL = 1; __VA_ARGS__; } break;    \
    case 2: { constexpr int VL = 2; __VA_ARGS__; } break;    \
    case 4: { constexpr int VL = 4; __VA_ARGS__; } break;    \
    case 8: { constexpr int VL = 8; __VA_ARGS__; } break;    \
    case 16: { constexpr int VL = 16; __VA_ARGS__; } break;  \
    default: { constexpr int VL = 32; __VA_ARGS__; } break;  \
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

int tsn_num_segments(int L) { return (L + kSegLen - 1) / kSegLen; }

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
                       float* cummean, float* cumrstd, float* gu, float* gv, double* seg_scratch, int B, int L,
                       int H, int G, float eps, int x_dtype, int w_dtype, cudaStream_t st) {
  const long long rows = (long long)B * L;
  const int lpg = pick_lpg(H / G);
  TSN_DISPATCH(x_dtype, w_dtype, {
    const bool vec = tsn_vec_ok(H, G, {x, y, gamma, beta});
    if (vec) {
      VL_SWITCH(H / G / 8, {
        const long long threads = rows * G * VL;
        tsn_group_stats_vec_kernel<T, VL><<<div_up(threads, 256), 256, 0, st>>>((const T*)x, gu, gv, rows * G);
      });
    } else {
      LPG_SWITCH(lpg, {
        const long long threads = rows * G * LPG;
        tsn_group_stats_kernel<T, LPG><<<div_up(threads, 256), 256, 0, st>>>((const T*)x, gu, gv, rows, H, G);
      });
    }
    const int nseg = tsn_num_segments(L);
    const long long nsg = (long long)B * nseg * G;
    const int gt = tsn_fused_groups(nseg);
    if (gt > 0 && B <= 65535) {
      tsn_scan_fused_kernel<T><<<dim3(div_up(G, gt), B), gt * nseg, 0, st>>>(
          gu, gv, mask, prev_count, (const T*)prev_mean, (const T*)prev_var, count_out, (T*)mean_out, (T*)var_out,
          cummean, cumrstd, L, G, nseg, gt, eps);
    } else {
    tsn_seg_sums_kernel<<<div_up(nsg, 256), 256, 0, st>>>(gu, gv, mask, seg_scratch, B, L, G, nseg);
    tsn_seg_prefix_kernel<T><<<div_up((long long)B * G, 128), 128, 0, st>>>(
        seg_scratch, prev_count, (const T*)prev_mean, (const T*)prev_var, count_out, (T*)mean_out, (T*)var_out,
        B, G, nseg);
    tsn_seg_apply_kernel<T><<<div_up(nsg, 256), 256, 0, st>>>(gu, gv, mask, seg_scratch, (const T*)prev_mean,
                                                            (const T*)prev_var, cummean, cumrstd, B, L, G, nseg,
                                                            eps);
    }
    if (vec) {
      const int grid = (int)std::min<long long>(div_up(rows * (H / 8), 256), 148LL * 16);
      tsn_apply_vec_kernel<T, W><<<grid, 256, 0, st>>>((const T*)x, cummean, cumrstd, (const W*)gamma,
                                                       gamma_offset, (const W*)beta, mask, (T*)y, rows, H, G);
    } else {
      const int grid = (int)std::min<long long>(div_up(rows * H, 256), 148LL * 16);
      tsn_apply_kernel<T, W><<<grid, 256, 0, st>>>((const T*)x, cummean, cumrstd, (const W*)gamma,
                                                   gamma_offset, (const W*)beta, mask, (T*)y, rows, H, G);
    }
  });
}

void timestep_norm_bwd(const void* dy, const void* dmean_out, const void* dvar_out, const void* x,
                       const void* prev_mean, const long long* count_final, const float* cummean,
                       const float* cumrstd, const void* gamma, float gamma_offset, const bool* mask,
                       void* dx, void* dprev_mean, void* dprev_var, float* dgamma, float* dbeta,
                       float* ux, float* ds, float* db, float* dux, float* dvx, double* seg_scratch,
                       int* cumvalid, int B, int L, int H, int G, int x_dtype, int w_dtype, cudaStream_t st,
                       float* colsum_ws) {
  const long long rows = (long long)B * L;
  const int lpg = pick_lpg(H / G);
  TSN_DISPATCH(x_dtype, w_dtype, {
    const bool vec = tsn_vec_ok(H, G, {dy, x, dx, gamma});
    if (vec) {
      VL_SWITCH(H / G / 8, {
        const long long threads = rows * G * VL;
        tsn_group_grads_vec_kernel<T, W, VL><<<div_up(threads, 256), 256, 0, st>>>(
            (const T*)dy, (const T*)x, cummean, (const W*)gamma, gamma_offset, ux, ds, db, rows * G, G);
      });
    } else {
      LPG_SWITCH(lpg, {
        const long long threads = rows * G * LPG;
        tsn_group_grads_kernel<T, W, LPG><<<div_up(threads, 256), 256, 0, st>>>(
            (const T*)dy, (const T*)x, cummean, (const W*)gamma, gamma_offset, ux, ds, db, rows, H, G);
      });
    }
    const int nseg = tsn_num_segments(L);
    const long long nsg = (long long)B * nseg * G;
    if (mask != nullptr) tsn_cumvalid_kernel<<<div_up(B, 32), 32, 0, st>>>(mask, cumvalid, B, L);
    const int* cv = mask != nullptr ? cumvalid : nullptr;
    const StepIn in{ux, ds, db, cummean, cumrstd};
    const int gt = tsn_fused_groups(nseg);
    if (gt > 0 && B <= 65535) {
      tsn_bwd_scan_fused_kernel<T><<<dim3(div_up(G, gt), B), gt * nseg, 0, st>>>(
          in, mask, cv, count_final, (const T*)prev_mean, (const T*)dmean_out, (const T*)dvar_out, (T*)dprev_mean,
          (T*)dprev_var, dux, dvx, L, G, nseg, gt);
    } else {
    tsn_bwd_seg_maps_kernel<T><<<div_up(nsg, 256), 256, 0, st>>>(in, mask, cv, count_final, (const T*)prev_mean,
                                                               seg_scratch, B, L, G, nseg);
    tsn_bwd_seg_prefix_kernel<T><<<div_up((long long)B * G, 128), 128, 0, st>>>(
        seg_scratch, (const T*)dmean_out, (const T*)dvar_out, (T*)dprev_mean, (T*)dprev_var, B, G, nseg);
    tsn_bwd_seg_apply_kernel<T><<<div_up(nsg, 256), 256, 0, st>>>(in, mask, cv, count_final, (const T*)prev_mean,
                                                                seg_scratch, dux, dvx, B, L, G, nseg);
    }
    const int grid = (int)std::min<long long>(rows, vec ? (long long)kColsumRows : 148LL * 4);
    if (vec) {
      const int hv = H / 8;
      if (hv <= kBwdThreads)
        tsn_bwd_apply_vec_kernel<T, W, 1><<<grid, kBwdThreads, 0, st>>>(
            (const T*)dy, (const T*)x, cummean, cumrstd, ux, dux, dvx, (const W*)gamma, gamma_offset, mask, (T*)dx,
            dgamma, dbeta, rows, H, G, colsum_ws);
      else if (hv <= 2 * kBwdThreads)
        tsn_bwd_apply_vec_kernel<T, W, 2><<<grid, kBwdThreads, 0, st>>>(
            (const T*)dy, (const T*)x, cummean, cumrstd, ux, dux, dvx, (const W*)gamma, gamma_offset, mask, (T*)dx,
            dgamma, dbeta, rows, H, G, colsum_ws);
      else
        tsn_bwd_apply_vec_kernel<T, W, 4><<<grid, kBwdThreads, 0, st>>>(
            (const T*)dy, (const T*)x, cummean, cumrstd, ux, dux, dvx, (const W*)gamma, gamma_offset, mask, (T*)dx,
            dgamma, dbeta, rows, H, G, colsum_ws);
      if (colsum_ws != nullptr) colsum_finish(colsum_ws, grid, H, dgamma, dbeta, st);
    } else
    tsn_bwd_apply_kernel<T, W><<<grid, kBwdThreads, 0, st>>>((const T*)dy, (const T*)x, cummean, cumrstd, ux, dux,
                                                     dvx, (const W*)gamma, gamma_offset, mask, (T*)dx,
                                                     dgamma, dbeta, rows, H, G);
  });
}

}  // namespace mb
