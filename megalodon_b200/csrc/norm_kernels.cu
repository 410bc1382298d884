// Row-wise normalisations over the last dimension: RMSNorm and LayerNorm,
// forward and backward.  They replace the apex `fused_layer_norm_cuda`
// extension the reference depends on (megalodon/modules/layer_norm.py:8-11).
//
// Layout: x [M, D] contiguous.  The scale actually applied is
// `weight[j] + weight_offset` evaluated in fp32 (the modules store zero-centred
// weights and pass offset 1), which keeps small weights exact under bf16
// parameters.  Statistics are fp32; `rstd` (and `mean`) are saved for backward.
#include "common.cuh"
#include "kernels.h"

namespace mb {

namespace {

constexpr int kMaxColsPerThread = 32;

template <int ROW_THREADS>
__device__ __forceinline__ float row_sum(float v, float* scratch) {
  if constexpr (ROW_THREADS == 32) {
    return warp_sum(v);
  } else {
    return block_sum(v, scratch);
  }
}

// ROW_THREADS == 32: one warp per row, blockDim.x/32 rows per CTA iteration.
// ROW_THREADS == blockDim.x: one CTA per row.
template <typename T, typename W, bool LAYER, int ROW_THREADS>
__global__ void norm_fwd_kernel(const T* __restrict__ x, const W* __restrict__ weight,
                                const W* __restrict__ bias, float weight_offset, T* __restrict__ y,
                                float* __restrict__ mean_out, float* __restrict__ rstd_out, long long M,
                                int D, float eps) {
  __shared__ float scratch[32];
  const int rows_per_cta = blockDim.x / ROW_THREADS;
  const int sub = threadIdx.x / ROW_THREADS;
  const int t = threadIdx.x % ROW_THREADS;
  for (long long row = (long long)blockIdx.x * rows_per_cta + sub; row < M + sub;
       row += (long long)gridDim.x * rows_per_cta) {
    // with ROW_THREADS == blockDim.x every thread sees the same `row`, so the
    // block-wide reductions below are reached uniformly
    const bool live = row < M;
    const T* xr = x + (live ? row : 0) * D;
    float s = 0.f, ss = 0.f;
    if (live) {
      for (int j = t; j < D; j += ROW_THREADS) {
        const float v = to_f(xr[j]);
        s += v;
        ss += v * v;
      }
    }
    float mean = 0.f, var;
    if constexpr (LAYER) {
      s = row_sum<ROW_THREADS>(s, scratch);
      mean = s / D;
      float sq = 0.f;
      if (live) {
        for (int j = t; j < D; j += ROW_THREADS) {
          const float d = to_f(xr[j]) - mean;
          sq += d * d;
        }
      }
      var = row_sum<ROW_THREADS>(sq, scratch) / D;
    } else {
      var = row_sum<ROW_THREADS>(ss, scratch) / D;
    }
    if (!live) continue;
    const float rstd = rsqrtf(var + eps);
    T* yr = y + row * D;
    for (int j = t; j < D; j += ROW_THREADS) {
      float v = (to_f(xr[j]) - mean) * rstd;
      if (weight != nullptr) v *= to_f(weight[j]) + weight_offset;
      if (LAYER && bias != nullptr) v += to_f(bias[j]);
      yr[j] = from_f<T>(v);
    }
    if (t == 0) {
      rstd_out[row] = rstd;
      if (LAYER) mean_out[row] = mean;
    }
  }
}

template <typename T, typename W, bool LAYER, int ROW_THREADS>
__global__ void norm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                const W* __restrict__ weight, float weight_offset,
                                const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                                T* __restrict__ dx, float* __restrict__ dweight, float* __restrict__ dbias,
                                long long M, int D) {
  __shared__ float scratch[32];
  const int rows_per_cta = blockDim.x / ROW_THREADS;
  const int sub = threadIdx.x / ROW_THREADS;
  const int t = threadIdx.x % ROW_THREADS;
  float acc_w[kMaxColsPerThread], acc_b[kMaxColsPerThread];
#pragma unroll
  for (int i = 0; i < kMaxColsPerThread; ++i) acc_w[i] = acc_b[i] = 0.f;

  for (long long row = (long long)blockIdx.x * rows_per_cta + sub; row < M + sub;
       row += (long long)gridDim.x * rows_per_cta) {
    const bool live = row < M;
    const long long r = live ? row : 0;
    const T* xr = x + r * D;
    const T* gr = dy + r * D;
    const float rstd = rstd_in[r];
    const float mean = LAYER ? mean_in[r] : 0.f;
    float c1 = 0.f, c2 = 0.f;
    if (live) {
      for (int j = t; j < D; j += ROW_THREADS) {
        const float w = weight != nullptr ? to_f(weight[j]) + weight_offset : 1.f;
        const float gw = to_f(gr[j]) * w;
        const float xh = (to_f(xr[j]) - mean) * rstd;
        c1 += gw * xh;
        c2 += gw;
      }
    }
    c1 = row_sum<ROW_THREADS>(c1, scratch) / D;
    if constexpr (LAYER) c2 = row_sum<ROW_THREADS>(c2, scratch) / D; else c2 = 0.f;
    if (!live) continue;
    T* dr = dx + row * D;
#pragma unroll
    for (int i = 0; i < kMaxColsPerThread; ++i) {   // fixed trip count keeps the accumulators in registers
      const int j = t + i * ROW_THREADS;
      if (j < D) {
        const float w = weight != nullptr ? to_f(weight[j]) + weight_offset : 1.f;
        const float g = to_f(gr[j]);
        const float xh = (to_f(xr[j]) - mean) * rstd;
        dr[j] = from_f<T>(rstd * (g * w - xh * c1 - c2));
        acc_w[i] += g * xh;
        acc_b[i] += g;
      }
    }
  }
  if (dweight != nullptr) {
#pragma unroll
    for (int i = 0; i < kMaxColsPerThread; ++i) {
      const int j = t + i * ROW_THREADS;
      if (j < D) {
        atomicAdd(dweight + j, acc_w[i]);
        if (LAYER && dbias != nullptr) atomicAdd(dbias + j, acc_b[i]);
      }
    }
  }
}

template <typename T, typename W, bool LAYER>
void launch_fwd(const void* x, const void* w, const void* b, float off, void* y, float* mean, float* rstd,
                long long M, int D, float eps, cudaStream_t st) {
  if (D <= 1024) {
    const int threads = 128, rows = threads / 32;
    const int grid = (int)std::min<long long>((M + rows - 1) / rows, 148LL * 16);
    norm_fwd_kernel<T, W, LAYER, 32><<<grid, threads, 0, st>>>((const T*)x, (const W*)w, (const W*)b, off,
                                                               (T*)y, mean, rstd, M, D, eps);
  } else {
    const int threads = 256;
    const int grid = (int)std::min<long long>(M, 148LL * 8);
    norm_fwd_kernel<T, W, LAYER, 256><<<grid, threads, 0, st>>>((const T*)x, (const W*)w, (const W*)b, off,
                                                                (T*)y, mean, rstd, M, D, eps);
  }
}

template <typename T, typename W, bool LAYER>
void launch_bwd(const void* dy, const void* x, const void* w, float off, const float* mean,
                const float* rstd, void* dx, float* dw, float* db, long long M, int D, cudaStream_t st) {
  if (D <= 1024) {
    const int threads = 128, rows = threads / 32;
    const int grid = (int)std::min<long long>((M + rows - 1) / rows, 148LL * 4);
    norm_bwd_kernel<T, W, LAYER, 32><<<grid, threads, 0, st>>>((const T*)dy, (const T*)x, (const W*)w, off,
                                                               mean, rstd, (T*)dx, dw, db, M, D);
  } else {
    const int threads = 256;
    const int grid = (int)std::min<long long>(M, 148LL * 4);
    norm_bwd_kernel<T, W, LAYER, 256><<<grid, threads, 0, st>>>((const T*)dy, (const T*)x, (const W*)w, off,
                                                                mean, rstd, (T*)dx, dw, db, M, D);
  }
}

}  // namespace

#define NORM_DISPATCH(xd, wd, ...)                                   \
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

// weight dtype must be fp32 or equal to the activation dtype
void rms_norm_fwd(const void* x, const void* w, float w_off, void* y, float* rstd, long long M, int D,
                  float eps, int x_dtype, int w_dtype, cudaStream_t st) {
  NORM_DISPATCH(x_dtype, w_dtype, (launch_fwd<T, W, false>(x, w, nullptr, w_off, y, nullptr, rstd, M, D, eps, st)));
}

void rms_norm_bwd(const void* dy, const void* x, const void* w, float w_off, const float* rstd, void* dx,
                  float* dw, long long M, int D, int x_dtype, int w_dtype, cudaStream_t st) {
  NORM_DISPATCH(x_dtype, w_dtype,
                (launch_bwd<T, W, false>(dy, x, w, w_off, nullptr, rstd, dx, dw, nullptr, M, D, st)));
}

void layer_norm_fwd(const void* x, const void* w, const void* b, float w_off, void* y, float* mean,
                    float* rstd, long long M, int D, float eps, int x_dtype, int w_dtype, cudaStream_t st) {
  NORM_DISPATCH(x_dtype, w_dtype, (launch_fwd<T, W, true>(x, w, b, w_off, y, mean, rstd, M, D, eps, st)));
}

void layer_norm_bwd(const void* dy, const void* x, const void* w, float w_off, const float* mean,
                    const float* rstd, void* dx, float* dw, float* db, long long M, int D, int x_dtype,
                    int w_dtype, cudaStream_t st) {
  NORM_DISPATCH(x_dtype, w_dtype,
                (launch_bwd<T, W, true>(dy, x, w, w_off, mean, rstd, dx, dw, db, M, D, st)));
}

}  // namespace mb
