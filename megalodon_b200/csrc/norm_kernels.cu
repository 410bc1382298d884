// Row-wise normalisations over the last dimension: RMSNorm and LayerNorm,
// forward and backward.  They replace the apex `fused_layer_norm_cuda`
// extension the reference depends on (megalodon/modules/layer_norm.py:8-11).
//
// Layout: x [M, D] contiguous.  The scale actually applied is
// `weight[j] + weight_offset` evaluated in fp32 (the modules store zero-centred
// weights and pass offset 1), which keeps small weights exact under bf16
// parameters.  Statistics are fp32; `rstd` (and `mean`) are saved for backward.
#include <initializer_list>

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

// ---------------------------------------------------------------- 16-byte variants
// A row lives in registers: thread t of the ROW_THREADS that share a row owns the 8-element groups
// t, t + ROW_THREADS, ... (at most VPT of them), so x and dy are read once and every access is 16
// bytes (two for fp32).  Needs D % 8 == 0, D <= ROW_THREADS * 8 * VPT and 32-byte aligned pointers.
constexpr int kMaxVecVPT = 4;

template <typename T, typename W, bool LAYER, int ROW_THREADS, int kVecVPT>
__global__ void norm_fwd_vec_kernel(const T* __restrict__ x, const W* __restrict__ weight,
                                    const W* __restrict__ bias, float weight_offset, T* __restrict__ y,
                                    float* __restrict__ mean_out, float* __restrict__ rstd_out, long long M,
                                    int D, float eps) {
  __shared__ float scratch[32];
  const int rows_per_cta = blockDim.x / ROW_THREADS;
  const int sub = threadIdx.x / ROW_THREADS;
  const int t = threadIdx.x % ROW_THREADS;
  const int nvec = D / 8;
  for (long long row = (long long)blockIdx.x * rows_per_cta + sub; row < M + sub;
       row += (long long)gridDim.x * rows_per_cta) {
    const bool live = row < M;
    const T* xr = x + (live ? row : 0) * D;
    float v[kVecVPT][8];
    float s = 0.f, ss = 0.f;
#pragma unroll
    for (int i = 0; i < kVecVPT; ++i) {
      const int g = t + i * ROW_THREADS;
      if (live && g < nvec) {
        load8(xr + 8 * g, v[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          s += v[i][j];
          ss = fmaf(v[i][j], v[i][j], ss);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] = 0.f;
      }
    }
    float mean = 0.f, var;
    if constexpr (LAYER) {
      s = row_sum<ROW_THREADS>(s, scratch);
      mean = s / D;
      float sq = 0.f;
#pragma unroll
      for (int i = 0; i < kVecVPT; ++i) {
        if (t + i * ROW_THREADS < nvec) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float d = v[i][j] - mean;
            sq = fmaf(d, d, sq);
          }
        }
      }
      var = row_sum<ROW_THREADS>(live ? sq : 0.f, scratch) / D;
    } else {
      var = row_sum<ROW_THREADS>(ss, scratch) / D;
    }
    if (!live) continue;
    const float rstd = rsqrtf(var + eps);
    T* yr = y + row * D;
#pragma unroll
    for (int i = 0; i < kVecVPT; ++i) {
      const int g = t + i * ROW_THREADS;
      if (g < nvec) {
        float o[8], w[8], b[8];
        if (weight != nullptr) load8(weight + 8 * g, w);
        if (LAYER && bias != nullptr) load8(bias + 8 * g, b);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float r = (v[i][j] - mean) * rstd;
          if (weight != nullptr) r *= w[j] + weight_offset;
          if (LAYER && bias != nullptr) r += b[j];
          o[j] = r;
        }
        store8(yr + 8 * g, o);
      }
    }
    if (t == 0) {
      rstd_out[row] = rstd;
      if (LAYER) mean_out[row] = mean;
    }
  }
}

template <typename T, typename W, bool LAYER, int ROW_THREADS, int kVecVPT>
__global__ void norm_bwd_vec_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                    const W* __restrict__ weight, float weight_offset,
                                    const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                                    T* __restrict__ dx, float* __restrict__ dweight, float* __restrict__ dbias,
                                    long long M, int D, float* __restrict__ colsum_ws) {
  __shared__ float scratch[32];
  const int rows_per_cta = blockDim.x / ROW_THREADS;
  const int sub = threadIdx.x / ROW_THREADS;
  const int t = threadIdx.x % ROW_THREADS;
  const int nvec = D / 8;
  float acc_w[kVecVPT][8], acc_b[kVecVPT][8], w[kVecVPT][8];
#pragma unroll
  for (int i = 0; i < kVecVPT; ++i) {
    const int g = t + i * ROW_THREADS;
    if (weight != nullptr && g < nvec) {
      load8(weight + 8 * g, w[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) w[i][j] += weight_offset;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) w[i][j] = 1.f;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) acc_w[i][j] = acc_b[i][j] = 0.f;
  }
  for (long long row = (long long)blockIdx.x * rows_per_cta + sub; row < M + sub;
       row += (long long)gridDim.x * rows_per_cta) {
    const bool live = row < M;
    const long long r = live ? row : 0;
    const float rstd = rstd_in[r];
    const float mean = LAYER ? mean_in[r] : 0.f;
    float g8[kVecVPT][8], xh[kVecVPT][8];
    float c1 = 0.f, c2 = 0.f;
#pragma unroll
    for (int i = 0; i < kVecVPT; ++i) {
      const int g = t + i * ROW_THREADS;
      if (live && g < nvec) {
        load8(dy + r * D + 8 * g, g8[i]);
        load8(x + r * D + 8 * g, xh[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = (xh[i][j] - mean) * rstd;
          const float gw = g8[i][j] * w[i][j];
          c1 = fmaf(gw, xh[i][j], c1);
          c2 += gw;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) g8[i][j] = xh[i][j] = 0.f;
      }
    }
    c1 = row_sum<ROW_THREADS>(c1, scratch) / D;
    if constexpr (LAYER) c2 = row_sum<ROW_THREADS>(c2, scratch) / D; else c2 = 0.f;
    if (!live) continue;
#pragma unroll
    for (int i = 0; i < kVecVPT; ++i) {
      const int g = t + i * ROW_THREADS;
      if (g < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          o[j] = rstd * (g8[i][j] * w[i][j] - xh[i][j] * c1 - c2);
          acc_w[i][j] = fmaf(g8[i][j], xh[i][j], acc_w[i][j]);
          acc_b[i][j] += g8[i][j];
        }
        store8(dx + row * D + 8 * g, o);
      }
    }
  }
  if (dweight != nullptr && colsum_ws != nullptr) {
    // one row of partial sums per CTA (one row per CTA iteration on this path: ROW_THREADS == blockDim.x)
    constexpr int kSets = LAYER ? 2 : 1;
    float* mine = colsum_ws + (long long)blockIdx.x * kSets * D;
#pragma unroll
    for (int i = 0; i < kVecVPT; ++i) {
      const int g = t + i * ROW_THREADS;
      if (g < nvec) {
        store8(mine + 8 * g, acc_w[i]);
        if (LAYER) store8(mine + D + 8 * g, acc_b[i]);
      }
    }
  } else if (dweight != nullptr) {
#pragma unroll
    for (int i = 0; i < kVecVPT; ++i) {
      const int g = t + i * ROW_THREADS;
      if (g < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          atomicAdd(dweight + 8 * g + j, acc_w[i][j]);
          if (LAYER && dbias != nullptr) atomicAdd(dbias + 8 * g + j, acc_b[i][j]);
        }
      }
    }
  }
}

// out0[j] += sum over rows of ws[row][0][j] (and out1 from ws[row][1][j] when given): a warp owns 32
// adjacent columns (128-byte reads), the 8 warps of a CTA take every 8th row and meet in shared memory.
__global__ void colsum_finish_kernel(const float* __restrict__ ws, int rows, int D, float* __restrict__ out0,
                                     float* __restrict__ out1) {
  __shared__ float part[2][8][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int j = blockIdx.x * 32 + lane;
  const int sets = out1 != nullptr ? 2 : 1;
  float s0 = 0.f, s1 = 0.f;
  if (j < D) {
#pragma unroll 4
    for (int r = warp; r < rows; r += 8) {
      s0 += ws[((long long)r * sets) * D + j];
      if (out1 != nullptr) s1 += ws[((long long)r * sets + 1) * D + j];
    }
  }
  part[0][warp][lane] = s0;
  part[1][warp][lane] = s1;
  __syncthreads();
  if (warp == 0 && j < D) {
#pragma unroll
    for (int w = 1; w < 8; ++w) {
      s0 += part[0][w][lane];
      s1 += part[1][w][lane];
    }
    out0[j] += s0;
    if (out1 != nullptr) out1[j] += s1;
  }
}

// smallest number of 8-element groups per thread that covers a row of D elements
#define VPT_SWITCH(D, ROW_THREADS, ...)                                       \
  do {                                                                        \
    if ((D) <= (ROW_THREADS) * 8) { constexpr int VPT = 1; __VA_ARGS__; }     \
    else if ((D) <= (ROW_THREADS) * 16) { constexpr int VPT = 2; __VA_ARGS__; } \
    else { constexpr int VPT = 4; __VA_ARGS__; }                              \
  } while (0)

inline bool vec_ok(int D, int row_threads, std::initializer_list<const void*> ptrs) {
  if (D % 8 != 0 || D > row_threads * 8 * kMaxVecVPT) return false;
  for (const void* q : ptrs)
    if (q != nullptr && !aligned32(q)) return false;
  return true;
}

template <typename T, typename W, bool LAYER>
void launch_fwd(const void* x, const void* w, const void* b, float off, void* y, float* mean, float* rstd,
                long long M, int D, float eps, cudaStream_t st) {
  if (D <= 1024 && vec_ok(D, 32, {x, w, b, y})) {
    const int threads = 128, rows = threads / 32;
    const int grid = (int)std::min<long long>((M + rows - 1) / rows, 148LL * 16);
    VPT_SWITCH(D, 32, (norm_fwd_vec_kernel<T, W, LAYER, 32, VPT><<<grid, threads, 0, st>>>(
                           (const T*)x, (const W*)w, (const W*)b, off, (T*)y, mean, rstd, M, D, eps)));
    return;
  }
  if (D > 1024 && vec_ok(D, 256, {x, w, b, y})) {
    const int grid = (int)std::min<long long>(M, 148LL * 8);
    VPT_SWITCH(D, 256, (norm_fwd_vec_kernel<T, W, LAYER, 256, VPT><<<grid, 256, 0, st>>>(
                            (const T*)x, (const W*)w, (const W*)b, off, (T*)y, mean, rstd, M, D, eps)));
    return;
  }
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
                const float* rstd, void* dx, float* dw, float* db, long long M, int D, cudaStream_t st,
                float* ws) {
  if (D <= 1024 && vec_ok(D, 32, {dy, x, w, dx})) {
    const int threads = 128, rows = threads / 32;
    const int grid = (int)std::min<long long>((M + rows - 1) / rows, 148LL * 4);
    VPT_SWITCH(D, 32, (norm_bwd_vec_kernel<T, W, LAYER, 32, VPT><<<grid, threads, 0, st>>>(
                           (const T*)dy, (const T*)x, (const W*)w, off, mean, rstd, (T*)dx, dw, db, M, D, nullptr)));
    return;
  }
  if (D > 1024 && vec_ok(D, 256, {dy, x, w, dx})) {
    // one resident wave (the accumulators of the column sums cap the kernel at two CTAs per SM)
    const int grid = (int)std::min<long long>(M, (long long)kColsumRows);
    float* use_ws = (dw != nullptr && (!LAYER || db != nullptr)) ? ws : nullptr;
    VPT_SWITCH(D, 256, (norm_bwd_vec_kernel<T, W, LAYER, 256, VPT><<<grid, 256, 0, st>>>(
                            (const T*)dy, (const T*)x, (const W*)w, off, mean, rstd, (T*)dx, dw, db, M, D, use_ws)));
    if (use_ws != nullptr) colsum_finish(use_ws, grid, D, dw, LAYER ? db : nullptr, st);
    return;
  }
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

// Column sums of a row-major 16-bit matrix (the bias gradient of a linear layer): every CTA walks a strip
// of rows with 8-column vectors per thread and leaves one row of partial sums; `colsum_finish` adds them.
template <typename T, int VPT>
__global__ void colsum_partial_kernel(const T* __restrict__ g, long long M, int N, float* __restrict__ ws) {
  const int nvec = N / 8;
  float acc[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
  for (long long row = blockIdx.x; row < M; row += gridDim.x) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * 256;
      if (c < nvec) {
        float v[8];
        load8(g + row * N + c * 8, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] += v[j];
      }
    }
  }
  float* mine = ws + (long long)blockIdx.x * N;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * 256;
    if (c < nvec) store8(mine + c * 8, acc[i]);
  }
}

// out[j] += sum_m g[m, j]; needs N % 8 == 0, N <= 8192, g 16-byte aligned; ws: kColsumRows * N floats.
// Returns false (nothing launched) when the shape is not covered.
bool colsum_16bit(const void* g, long long M, int N, float* ws, float* out, int dtype, cudaStream_t st) {
  if (N % 8 != 0 || N > 8192 || (reinterpret_cast<uintptr_t>(g) & 15) != 0 || (dtype != kBF16 && dtype != kF16))
    return false;
  const int grid = (int)std::min<long long>(M, (long long)kColsumRows);
  const int vpt = (N / 8 + 255) / 256;
#define MB_COLSUM(TT)                                                                                   \
  do {                                                                                                  \
    if (vpt <= 1) colsum_partial_kernel<TT, 1><<<grid, 256, 0, st>>>((const TT*)g, M, N, ws);           \
    else if (vpt <= 2) colsum_partial_kernel<TT, 2><<<grid, 256, 0, st>>>((const TT*)g, M, N, ws);      \
    else colsum_partial_kernel<TT, 4><<<grid, 256, 0, st>>>((const TT*)g, M, N, ws);                    \
  } while (0)
  if (dtype == kBF16) MB_COLSUM(__nv_bfloat16);
  else MB_COLSUM(__half);
#undef MB_COLSUM
  colsum_finish_kernel<<<(N + 31) / 32, 256, 0, st>>>(ws, grid, N, out, nullptr);
  return true;
}

void colsum_finish(const float* ws, int rows, int D, float* out0, float* out1, cudaStream_t st) {
  colsum_finish_kernel<<<(D + 31) / 32, 256, 0, st>>>(ws, rows, D, out0, out1);
}

void rms_norm_bwd(const void* dy, const void* x, const void* w, float w_off, const float* rstd, void* dx,
                  float* dw, long long M, int D, int x_dtype, int w_dtype, cudaStream_t st, float* colsum_ws) {
  NORM_DISPATCH(x_dtype, w_dtype,
                (launch_bwd<T, W, false>(dy, x, w, w_off, nullptr, rstd, dx, dw, nullptr, M, D, st, colsum_ws)));
}

void layer_norm_fwd(const void* x, const void* w, const void* b, float w_off, void* y, float* mean,
                    float* rstd, long long M, int D, float eps, int x_dtype, int w_dtype, cudaStream_t st) {
  NORM_DISPATCH(x_dtype, w_dtype, (launch_fwd<T, W, true>(x, w, b, w_off, y, mean, rstd, M, D, eps, st)));
}

void layer_norm_bwd(const void* dy, const void* x, const void* w, float w_off, const float* mean,
                    const float* rstd, void* dx, float* dw, float* db, long long M, int D, int x_dtype,
                    int w_dtype, cudaStream_t st, float* colsum_ws) {
  NORM_DISPATCH(x_dtype, w_dtype,
                (launch_bwd<T, W, true>(dy, x, w, w_off, mean, rstd, dx, dw, db, M, D, st, colsum_ws)));
}

}  // namespace mb
