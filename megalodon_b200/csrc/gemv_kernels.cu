// Linear layer for a handful of rows (token-by-token decoding):
//
//   y[m, n] = act(alpha * sum_k x[m, k] w[n, k] + bias[n])        m < M <= 16
//
// With so few rows the work is one pass over the weight matrix, so the kernel is organised around
// that stream: a warp owns NR consecutive weight rows and walks K in chunks of 256 elements, every
// lane holding one 16-byte piece of each row (NR * 2 loads in flight per lane); the matching pieces
// of x come from L1/L2 (x is at most 16 x K).  Partial sums are reduced over the warp with shuffles
// and lane 0 writes the NR x M results.  The tensor-core GEMM is the wrong tool here: with one
// 128-row tile per 256 columns it would use N / 256 CTAs and leave most of the machine idle.
#include "common.cuh"
#include "kernels.h"

namespace mb {
namespace {

constexpr int kGemvThreads = 128;   // 4 warps
constexpr int kGemvNR = 4;          // weight rows per warp
constexpr int kGemvKU = 4;          // 256-element chunks of K per loop trip

template <typename T, typename OutT, int MB>
__global__ void __launch_bounds__(kGemvThreads)
gemv_small_m_kernel(const T* __restrict__ x, const T* __restrict__ w, const void* __restrict__ bias, int bias_dtype,
                    OutT* __restrict__ y, int M, int N, int K, long long ldx, long long ldw, long long ldy,
                    float alpha, int act) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int n0 = (blockIdx.x * (kGemvThreads / 32) + warp) * kGemvNR;
  if (n0 >= N) return;
  float acc[MB][kGemvNR];
#pragma unroll
  for (int m = 0; m < MB; ++m)
#pragma unroll
    for (int r = 0; r < kGemvNR; ++r) acc[m][r] = 0.f;

  // kGemvKU chunks of 256 elements per trip: NR * KU 16-byte weight loads in flight per lane, kept raw
  // (4 registers each) until they are used
  for (int k0 = lane * 8; k0 < K; k0 += 256 * kGemvKU) {
    uint4 raw[kGemvKU][kGemvNR];
#pragma unroll
    for (int u = 0; u < kGemvKU; ++u) {
      const int k = k0 + u * 256;
#pragma unroll
      for (int r = 0; r < kGemvNR; ++r) {
        if (k < K && n0 + r < N) raw[u][r] = __ldg(reinterpret_cast<const uint4*>(w + (long long)(n0 + r) * ldw + k));
        else raw[u][r] = make_uint4(0u, 0u, 0u, 0u);
      }
    }
#pragma unroll
    for (int u = 0; u < kGemvKU; ++u) {
      const int k = k0 + u * 256;
      if (k >= K) break;
      float wv[kGemvNR][8];
#pragma unroll
      for (int r = 0; r < kGemvNR; ++r) load8(reinterpret_cast<const T*>(&raw[u][r]), wv[r]);
#pragma unroll
      for (int m = 0; m < MB; ++m) {
        if (m < M) {
          float xv[8];
          load8(x + (long long)m * ldx + k, xv);
#pragma unroll
          for (int r = 0; r < kGemvNR; ++r)
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[m][r] = fmaf(xv[j], wv[r][j], acc[m][r]);
        }
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MB; ++m)
#pragma unroll
    for (int r = 0; r < kGemvNR; ++r) acc[m][r] = warp_sum(acc[m][r]);
  if (lane == 0) {
#pragma unroll
    for (int r = 0; r < kGemvNR; ++r) {
      const int n = n0 + r;
      if (n >= N) break;
      float b = 0.f;
      if (bias != nullptr) {
        if (bias_dtype == kF32) b = reinterpret_cast<const float*>(bias)[n];
        else if (bias_dtype == kBF16) b = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(bias)[n]);
        else b = __half2float(reinterpret_cast<const __half*>(bias)[n]);
      }
#pragma unroll
      for (int m = 0; m < MB; ++m) {
        if (m < M) {
          float v = alpha * acc[m][r] + b;
          if (act == 1) v = silu_f(v);
          y[(long long)m * ldy + n] = from_f<OutT>(v);
        }
      }
    }
  }
}

template <typename T, typename OutT>
void launch_gemv(const void* x, const void* w, const void* bias, int bias_dtype, void* y, int M, int N, int K,
                 long long ldx, long long ldw, long long ldy, float alpha, int act, cudaStream_t st) {
  const int rows_per_cta = (kGemvThreads / 32) * kGemvNR;
  const int grid = div_up(N, rows_per_cta);
#define GEMV_CASE(MBV)                                                                                   \
  gemv_small_m_kernel<T, OutT, MBV><<<grid, kGemvThreads, 0, st>>>((const T*)x, (const T*)w, bias, bias_dtype, \
                                                                   (OutT*)y, M, N, K, ldx, ldw, ldy, alpha, act)
  if (M <= 1) GEMV_CASE(1);
  else if (M <= 2) GEMV_CASE(2);
  else if (M <= 4) GEMV_CASE(4);
  else if (M <= 8) GEMV_CASE(8);
  else GEMV_CASE(16);
#undef GEMV_CASE
}

}  // namespace

// Returns false when the shapes / alignment are outside what the kernel handles.
bool gemv_small_m(const void* x, const void* w, const void* bias, int bias_dtype, void* y, int M, int N, int K,
                  long long ldx, long long ldw, long long ldy, float alpha, int act, int in_dtype, int out_dtype,
                  cudaStream_t st) {
  if (M < 1 || M > 16 || K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0 || in_dtype == kF32) return false;
  if (!aligned16(x) || !aligned16(w)) return false;
  if (in_dtype == kBF16) {
    if (out_dtype == kBF16) launch_gemv<__nv_bfloat16, __nv_bfloat16>(x, w, bias, bias_dtype, y, M, N, K, ldx, ldw, ldy, alpha, act, st);
    else if (out_dtype == kF32) launch_gemv<__nv_bfloat16, float>(x, w, bias, bias_dtype, y, M, N, K, ldx, ldw, ldy, alpha, act, st);
    else return false;
  } else {
    if (out_dtype == kF16) launch_gemv<__half, __half>(x, w, bias, bias_dtype, y, M, N, K, ldx, ldw, ldy, alpha, act, st);
    else if (out_dtype == kF32) launch_gemv<__half, float>(x, w, bias, bias_dtype, y, M, N, K, ldx, ldw, ldy, alpha, act, st);
    else return false;
  }
  return true;
}

}  // namespace mb
