// Shared device helpers for the sm_100a kernels: type conversion, warp/block
// reductions, vector loads.  Everything here is header-only and torch-free so
// the kernel translation units compile in seconds.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mb {

constexpr int kWarp = 32;

enum DType : int { kF32 = 0, kBF16 = 1, kF16 = 2 };

template <typename T> struct TypeTag;
template <> struct TypeTag<float> { static constexpr int value = kF32; };
template <> struct TypeTag<__nv_bfloat16> { static constexpr int value = kBF16; };
template <> struct TypeTag<__half> { static constexpr int value = kF16; };

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_f(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over the first `width` lanes groups (width a power of two <= 32).
template <int WIDTH>
__device__ __forceinline__ float subwarp_sum(float v) {
#pragma unroll
  for (int o = WIDTH / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Block-wide sum; every thread gets the result.  `scratch` holds >= 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < nwarp) ? scratch[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarp = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < nwarp) ? scratch[lane] : -INFINITY;
  t = warp_max(t);
  return t;
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float silu_grad_f(float x) {
  const float s = 1.f / (1.f + __expf(-x));
  return s * (1.f + x * (1.f - s));
}

struct cfloat {
  float re, im;
};
__device__ __forceinline__ cfloat cmul(cfloat a, cfloat b) {
  return {a.re * b.re - a.im * b.im, a.re * b.im + a.im * b.re};
}
__device__ __forceinline__ cfloat cconj(cfloat a) { return {a.re, -a.im}; }
__device__ __forceinline__ cfloat cadd(cfloat a, cfloat b) { return {a.re + b.re, a.im + b.im}; }

#define MB_DISPATCH_DTYPE(dtype, ...)                         \
  do {                                                        \
    if ((dtype) == mb::kF32) {                                \
      using scalar_t = float;                                 \
      __VA_ARGS__;                                            \
    } else if ((dtype) == mb::kBF16) {                        \
      using scalar_t = __nv_bfloat16;                         \
      __VA_ARGS__;                                            \
    } else {                                                  \
      using scalar_t = __half;                                \
      __VA_ARGS__;                                            \
    }                                                         \
  } while (0)

inline int div_up(long long a, long long b) { return (int)((a + b - 1) / b); }

}  // namespace mb
