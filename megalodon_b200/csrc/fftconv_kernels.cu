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
bool fftconv_supported(int L) { return L >= 1 && fftconv_logn(L) <= 14; }

void rfft_rows(const void* x, float* out_spec, long long rows, int L, bool flip, int dtype, cudaStream_t st) {
  if (rows == 0) return;
  const int logn = fftconv_logn(L);
  const size_t smem = sizeof(cfloat) << logn;
  MB_DISPATCH_DTYPE(dtype, {
    if (!prepare(rfft_rows_kernel<scalar_t>, smem)) return;
    rfft_rows_kernel<scalar_t><<<(unsigned)rows, kFftThreads, smem, st>>>((const scalar_t*)x, (cfloat*)out_spec, L,
                                                                         logn, flip);
  });
}

void fftconv_rows(const void* x, const float* kf, void* y, long long rows, int L, int D, bool conj_k, int dtype,
                  cudaStream_t st) {
  if (rows == 0) return;
  const int logn = fftconv_logn(L);
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
