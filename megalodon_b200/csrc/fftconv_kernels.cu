// Causal long convolution through shared-memory FFTs, and the real FFT that goes with it.
//
//   y[b, d, t] = sum_{j <= t} k[d, j] x[b, d, t - j]          (reference: csrc/ops/fftconv_kernel.cu:23-164,
//                                                               modules/fused_ops/fftconv.py:30-110)
//
// One CTA owns one (b, d) row: the row is zero-padded to N2 = 2 * next_pow2(L) complex points in shared
// memory (8 N2 bytes, up to 128 KiB at L = 8192), transformed with an iterative radix-2 FFT, multiplied
// by the kernel spectrum (or its conjugate for the gradient w.r.t. x), transformed back, and the first
// L samples are written.  The gradient w.r.t. k needs sum_b DY_f conj(X_f): dy and x ride the real and
// imaginary part of ONE complex FFT and are separated with the Hermitian symmetry, the per-row product
// is accumulated into a [D, N2/2 + 1] spectrum with atomics, and a last pass transforms it back.
// Rows longer than 8192 samples (up to 16384, the reference's limit, csrc/fft.cuh:21) would need 256 KiB
// for N2 complex points, so they go through the packed form of the real transform: the N2 real samples
// are the real and imaginary parts of N2 / 2 complex points (even / odd samples), one half-size complex
// FFT is taken, and the real row's spectrum is recovered bin pair by bin pair (and packed again before
// the inverse transform).  The packed kernels work for every length and are also selectable for short
// rows, which is how they are tested against the plain ones.
// Megalodon's CEMA does not call this op here (it is a scan, cema_kernels.cu); it is provided because
// the reference exports it.
#include "common.cuh"
#include "kernels.h"

namespace mb {
namespace {

constexpr int kFftThreads = 512;

__device__ __forceinline__ cfloat cmulf(cfloat a, cfloat b) {
  return {fmaf(a.re, b.re, -a.im * b.im), fmaf(a.re, b.im, a.im * b.re)};
}

// In-place radix-2 decimation-in-time FFT of s[0..N) (N = 1 << logn), input in bit-reversed order,
// output in natural order.  sign = -1: forward, +1: inverse (unscaled).  All threads of the CTA call it.
__device__ void fft_inplace(cfloat* s, int logn, float sign) {
  const int N = 1 << logn;
  for (int lh = 0; lh < logn; ++lh) {           // half = 1 << lh
    const int half = 1 << lh;
    for (int i = threadIdx.x; i < N / 2; i += blockDim.x) {
      const int j = i & (half - 1);
      const int a = ((i >> lh) << (lh + 1)) + j;
      const int b = a + half;
      float sn, cs;
      sincospif(sign * (float)j / (float)half, &sn, &cs);
      const cfloat u = s[a];
      const cfloat v = cmulf(s[b], {cs, sn});
      s[a] = {u.re + v.re, u.im + v.im};
      s[b] = {u.re - v.re, u.im - v.im};
    }
    __syncthreads();
  }
}

__device__ __forceinline__ int bitrev(int i, int logn) { return (int)(__brev((unsigned)i) >> (32 - logn)); }

// natural order -> bit-reversed order, in place
__device__ void bitrev_permute(cfloat* s, int logn) {
  const int N = 1 << logn;
  for (int i = threadIdx.x; i < N; i += blockDim.x) {
    const int r = bitrev(i, logn);
    if (i < r) {
      const cfloat t = s[i];
      s[i] = s[r];
      s[r] = t;
    }
  }
  __syncthreads();
}

// s[bitrev(t)] = (re[t], im[t]) for t < L (im optional), zero elsewhere
template <typename T>
__device__ void load_rows_bitrev(cfloat* s, const T* re, const T* im, int L, int logn, bool flip) {
  const int N = 1 << logn;
  for (int t = threadIdx.x; t < N; t += blockDim.x) {
    cfloat v = {0.f, 0.f};
    if (t < L) {
      const int src = flip ? L - 1 - t : t;
      v.re = to_f(re[src]);
      if (im != nullptr) v.im = to_f(im[src]);
    }
    s[bitrev(t, logn)] = v;
  }
  __syncthreads();
}

// spectrum (half, N2/2 + 1 bins) of one real row
template <typename T>
__global__ void rfft_rows_kernel(const T* __restrict__ x, cfloat* __restrict__ out, int L, int logn, bool flip) {
  extern __shared__ __align__(16) unsigned char fft_smem[];
  cfloat* s = reinterpret_cast<cfloat*>(fft_smem);
  const long long row = blockIdx.x;
  const int N = 1 << logn;
  load_rows_bitrev<T>(s, x + row * L, nullptr, L, logn, flip);
  fft_inplace(s, logn, -1.f);
  for (int i = threadIdx.x; i <= N / 2; i += blockDim.x) out[row * (N / 2 + 1) + i] = s[i];
}

// y = irfft(rfft(x) * kf or conj(kf))[:L]; kf [D, N2/2 + 1], row = b * D + d
template <typename T>
__global__ void fftconv_rows_kernel(const T* __restrict__ x, const cfloat* __restrict__ kf, T* __restrict__ y,
                                    int L, int D, int logn, bool conj_k) {
  extern __shared__ __align__(16) unsigned char fft_smem[];
  cfloat* s = reinterpret_cast<cfloat*>(fft_smem);
  const long long row = blockIdx.x;
  const int d = (int)(row % D);
  const int N = 1 << logn;
  const cfloat* kr = kf + (long long)d * (N / 2 + 1);
  load_rows_bitrev<T>(s, x + row * L, nullptr, L, logn, false);
  fft_inplace(s, logn, -1.f);
  for (int i = threadIdx.x; i < N; i += blockDim.x) {
    cfloat k = i <= N / 2 ? kr[i] : cconj(kr[N - i]);      // Hermitian extension of the half spectrum
    if (conj_k) k = cconj(k);
    s[i] = cmulf(s[i], k);
  }
  __syncthreads();
  bitrev_permute(s, logn);
  fft_inplace(s, logn, 1.f);
  const float inv = 1.f / (float)N;
  for (int t = threadIdx.x; t < L; t += blockDim.x) y[row * L + t] = from_f<T>(s[t].re * inv);
}

// acc[d, i] += DY_f[i] conj(X_f[i]) for i <= N2/2, both spectra from one FFT of dy + i x
template <typename T>
__global__ void fftconv_dk_spectrum_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                           float* __restrict__ acc, int L, int D, int logn) {
  extern __shared__ __align__(16) unsigned char fft_smem[];
  cfloat* s = reinterpret_cast<cfloat*>(fft_smem);
  const long long row = blockIdx.x;
  const int d = (int)(row % D);
  const int N = 1 << logn;
  load_rows_bitrev<T>(s, dy + row * L, x + row * L, L, logn, false);
  fft_inplace(s, logn, -1.f);
  float* ar = acc + (long long)d * (N / 2 + 1) * 2;
  for (int i = threadIdx.x; i <= N / 2; i += blockDim.x) {
    const cfloat z = s[i];
    const cfloat zc = cconj(s[(N - i) & (N - 1)]);
    const cfloat gy = {0.5f * (z.re + zc.re), 0.5f * (z.im + zc.im)};          // DY_f
    const cfloat xs = {0.5f * (z.im - zc.im), -0.5f * (z.re - zc.re)};         // X_f = (z - zc) / (2i)
    const cfloat p = cmulf(gy, cconj(xs));
    atomicAdd(ar + 2 * i, p.re);
    atomicAdd(ar + 2 * i + 1, p.im);
  }
}

// out[row, :L] = irfft(spec[row])[:L]; spec [rows, N2/2 + 1]
__global__ void irfft_rows_kernel(const cfloat* __restrict__ spec, float* __restrict__ out, int L, int logn) {
  extern __shared__ __align__(16) unsigned char fft_smem[];
  cfloat* s = reinterpret_cast<cfloat*>(fft_smem);
  const long long row = blockIdx.x;
  const int N = 1 << logn;
  const cfloat* sr = spec + row * (N / 2 + 1);
  for (int i = threadIdx.x; i < N; i += blockDim.x) {
    const cfloat v = i <= N / 2 ? sr[i] : cconj(sr[N - i]);
    s[bitrev(i, logn)] = v;
  }
  __syncthreads();
  fft_inplace(s, logn, 1.f);
  const float inv = 1.f / (float)N;
  for (int t = threadIdx.x; t < L; t += blockDim.x) out[row * L + t] = s[t].re * inv;
}

// ---------------------------------------------------------------- packed real transforms (half-size FFT)
// s[bitrev(n)] = x[2n] + i x[2n + 1] over the zero-padded (optionally time-flipped) row; M = 1 << logm points
template <typename T>
__device__ void load_packed_bitrev(cfloat* s, const T* x, int L, int logm, bool flip) {
  const int M = 1 << logm;
  for (int n = threadIdx.x; n < M; n += blockDim.x) {
    cfloat v = {0.f, 0.f};
    const int t0 = 2 * n, t1 = 2 * n + 1;
    if (t0 < L) v.re = to_f(x[flip ? L - 1 - t0 : t0]);
    if (t1 < L) v.im = to_f(x[flip ? L - 1 - t1 : t1]);
    s[bitrev(n, logm)] = v;
  }
  __syncthreads();
}

// Bins k and M - k of the real row's spectrum from bins k and M - k of the packed transform Z:
//   E = (Z[k] + conj Z[M-k]) / 2 (even samples), O = (Z[k] - conj Z[M-k]) / 2i (odd samples),
//   X[k] = E + W O, X[M-k] = conj(E - W O), W = exp(-i pi k / M).  For k = 0 pass Z[0] twice: X[M-k] is bin M.
__device__ __forceinline__ void unpack_pair(cfloat zk, cfloat zmk, int k, int M, cfloat& xk, cfloat& xmk) {
  const cfloat e = {0.5f * (zk.re + zmk.re), 0.5f * (zk.im - zmk.im)};
  const cfloat d = {0.5f * (zk.re - zmk.re), 0.5f * (zk.im + zmk.im)};
  const cfloat o = {d.im, -d.re};
  float sn, cs;
  sincospif(-(float)k / (float)M, &sn, &cs);
  const cfloat wo = cmulf(o, {cs, sn});
  xk = {e.re + wo.re, e.im + wo.im};
  xmk = {e.re - wo.re, -(e.im - wo.im)};
}

// The inverse: packed bins Z'[k], Z'[M-k] (whose half-size inverse FFT carries the even samples in its real
// and the odd samples in its imaginary part) from the spectrum bins Y[k], Y[M-k] of a real row.
__device__ __forceinline__ void pack_pair(cfloat yk, cfloat ymk, int k, int M, cfloat& zk, cfloat& zmk) {
  const cfloat e = {0.5f * (yk.re + ymk.re), 0.5f * (yk.im - ymk.im)};
  const cfloat d = {0.5f * (yk.re - ymk.re), 0.5f * (yk.im + ymk.im)};
  float sn, cs;
  sincospif((float)k / (float)M, &sn, &cs);
  const cfloat o = cmulf(d, {cs, sn});
  zk = {e.re - o.im, e.im + o.re};
  zmk = {e.re + o.im, o.re - e.im};
}

template <typename T>
__global__ void rfft_rows_packed_kernel(const T* __restrict__ x, cfloat* __restrict__ out, int L, int logn, bool flip) {
  extern __shared__ __align__(16) unsigned char fft_smem[];
  cfloat* s = reinterpret_cast<cfloat*>(fft_smem);
  const long long row = blockIdx.x;
  const int logm = logn - 1, M = 1 << logm;
  load_packed_bitrev<T>(s, x + row * L, L, logm, flip);
  fft_inplace(s, logm, -1.f);
  cfloat* o = out + row * (M + 1);
  for (int k = threadIdx.x; k <= M / 2; k += blockDim.x) {
    cfloat xk, xmk;
    unpack_pair(s[k], s[k == 0 ? 0 : M - k], k, M, xk, xmk);
    o[k] = xk;
    if (k != M - k) o[M - k] = xmk;
  }
}

template <typename T>
__global__ void fftconv_rows_packed_kernel(const T* __restrict__ x, const cfloat* __restrict__ kf, T* __restrict__ y,
                                           int L, int D, int logn, bool conj_k) {
  extern __shared__ __align__(16) unsigned char fft_smem[];
  cfloat* s = reinterpret_cast<cfloat*>(fft_smem);
  const long long row = blockIdx.x;
  const int d = (int)(row % D);
  const int logm = logn - 1, M = 1 << logm;
  const cfloat* kr = kf + (long long)d * (M + 1);
  load_packed_bitrev<T>(s, x + row * L, L, logm, false);
  fft_inplace(s, logm, -1.f);
  // spectrum of the row, times the kernel's, packed again - pair by pair, in place
  for (int k = threadIdx.x; k <= M / 2; k += blockDim.x) {
    cfloat xk, xmk, zk, zmk;
    unpack_pair(s[k], s[k == 0 ? 0 : M - k], k, M, xk, xmk);
    cfloat ka = kr[k], kb = kr[M - k];
    if (conj_k) { ka = cconj(ka); kb = cconj(kb); }
    pack_pair(cmulf(xk, ka), cmulf(xmk, kb), k, M, zk, zmk);
    s[k] = zk;
    if (k != 0 && k != M - k) s[M - k] = zmk;
  }
  __syncthreads();
  bitrev_permute(s, logm);
  fft_inplace(s, logm, 1.f);
  const float inv = 1.f / (float)M;
  for (int t = threadIdx.x; t < L; t += blockDim.x) {
    const cfloat v = s[t >> 1];
    y[row * L + t] = from_f<T>(((t & 1) ? v.im : v.re) * inv);
  }
}

__global__ void irfft_rows_packed_kernel(const cfloat* __restrict__ spec, float* __restrict__ out, int L, int logn) {
  extern __shared__ __align__(16) unsigned char fft_smem[];
  cfloat* s = reinterpret_cast<cfloat*>(fft_smem);
  const long long row = blockIdx.x;
  const int logm = logn - 1, M = 1 << logm;
  const cfloat* sr = spec + row * (M + 1);
  for (int k = threadIdx.x; k <= M / 2; k += blockDim.x) {
    cfloat zk, zmk;
    pack_pair(sr[k], sr[M - k], k, M, zk, zmk);
    s[bitrev(k, logm)] = zk;
    if (k != 0 && k != M - k) s[bitrev(M - k, logm)] = zmk;
  }
  __syncthreads();
  fft_inplace(s, logm, 1.f);
  const float inv = 1.f / (float)M;
  for (int t = threadIdx.x; t < L; t += blockDim.x) {
    const cfloat v = s[t >> 1];
    out[row * L + t] = ((t & 1) ? v.im : v.re) * inv;
  }
}

template <typename K>
bool prepare(K kernel, size_t smem) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess;
}

}  // namespace

// FFT length (log2) used for a sequence of L samples: 2 * next_pow2(L), at least 64 points.
int fftconv_logn(int L) {
  int logn = 6;
  while ((1 << (logn - 1)) < L) ++logn;
  return logn;
}
bool fftconv_supported(int L) { return L >= 1 && fftconv_logn(L) <= 15; }
// rows of more than 8192 samples only fit shared memory in the packed form
static bool use_packed(int logn, int packed) { return packed > 0 || (packed < 0 && logn > 14); }

void rfft_rows(const void* x, float* out_spec, long long rows, int L, bool flip, int dtype, cudaStream_t st,
               int packed) {
  if (rows == 0) return;
  const int logn = fftconv_logn(L);
  if (use_packed(logn, packed)) {
    const size_t smem = sizeof(cfloat) << (logn - 1);
    MB_DISPATCH_DTYPE(dtype, {
      if (!prepare(rfft_rows_packed_kernel<scalar_t>, smem)) return;
      rfft_rows_packed_kernel<scalar_t><<<(unsigned)rows, kFftThreads, smem, st>>>((const scalar_t*)x, (cfloat*)out_spec,
                                                                                  L, logn, flip);
    });
    return;
  }
  const size_t smem = sizeof(cfloat) << logn;
  MB_DISPATCH_DTYPE(dtype, {
    if (!prepare(rfft_rows_kernel<scalar_t>, smem)) return;
    rfft_rows_kernel<scalar_t><<<(unsigned)rows, kFftThreads, smem, st>>>((const scalar_t*)x, (cfloat*)out_spec, L,
                                                                         logn, flip);
  });
}

void irfft_rows(const float* spec, float* out, long long rows, int L, cudaStream_t st, int packed) {
  if (rows == 0) return;
  const int logn = fftconv_logn(L);
  if (use_packed(logn, packed)) {
    const size_t smem = sizeof(cfloat) << (logn - 1);
    if (!prepare(irfft_rows_packed_kernel, smem)) return;
    irfft_rows_packed_kernel<<<(unsigned)rows, kFftThreads, smem, st>>>((const cfloat*)spec, out, L, logn);
    return;
  }
  const size_t smem = sizeof(cfloat) << logn;
  if (!prepare(irfft_rows_kernel, smem)) return;
  irfft_rows_kernel<<<(unsigned)rows, kFftThreads, smem, st>>>((const cfloat*)spec, out, L, logn);
}

void fftconv_rows(const void* x, const float* kf, void* y, long long rows, int L, int D, bool conj_k, int dtype,
                  cudaStream_t st, int packed) {
  if (rows == 0) return;
  const int logn = fftconv_logn(L);
  if (use_packed(logn, packed)) {
    const size_t smem = sizeof(cfloat) << (logn - 1);
    MB_DISPATCH_DTYPE(dtype, {
      if (!prepare(fftconv_rows_packed_kernel<scalar_t>, smem)) return;
      fftconv_rows_packed_kernel<scalar_t><<<(unsigned)rows, kFftThreads, smem, st>>>(
          (const scalar_t*)x, (const cfloat*)kf, (scalar_t*)y, L, D, logn, conj_k);
    });
    return;
  }
  const size_t smem = sizeof(cfloat) << logn;
  MB_DISPATCH_DTYPE(dtype, {
    if (!prepare(fftconv_rows_kernel<scalar_t>, smem)) return;
    fftconv_rows_kernel<scalar_t><<<(unsigned)rows, kFftThreads, smem, st>>>((const scalar_t*)x, (const cfloat*)kf,
                                                                            (scalar_t*)y, L, D, logn, conj_k);
  });
}

// acc_spec [D, N2/2 + 1, 2] must be zero-initialised; dk [D, L] fp32
void fftconv_dk(const void* dy, const void* x, float* acc_spec, float* dk, long long rows, int L, int D, int dtype,
                cudaStream_t st) {
  if (rows == 0) return;
  const int logn = fftconv_logn(L);
  const size_t smem = sizeof(cfloat) << logn;
  MB_DISPATCH_DTYPE(dtype, {
    if (!prepare(fftconv_dk_spectrum_kernel<scalar_t>, smem)) return;
    fftconv_dk_spectrum_kernel<scalar_t><<<(unsigned)rows, kFftThreads, smem, st>>>(
        (const scalar_t*)dy, (const scalar_t*)x, acc_spec, L, D, logn);
  });
  if (!prepare(irfft_rows_kernel, smem)) return;
  irfft_rows_kernel<<<(unsigned)D, kFftThreads, smem, st>>>((const cfloat*)acc_spec, dk, L, logn);
}

}  // namespace mb
