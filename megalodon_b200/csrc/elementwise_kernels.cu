// Bandwidth-bound helpers: SwiGLU gate, rotary embedding, cross-entropy,
// fused AdamW on flat shards (master fp32 + low-precision copy in one pass),
// sum of squares for the gradient norm.
#include "common.cuh"
#include "kernels.h"

namespace mb {
namespace {

// n8 groups of 8 elements through 16-byte accesses, then a scalar tail of n - 8 * n8 elements
template <typename T>
__global__ void swiglu_fwd_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out,
                                  long long n, long long n8) {
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = tid; i < n8; i += stride) {
    float av[8], bv[8], o[8];
    load8(a + 8 * i, av);
    load8(b + 8 * i, bv);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = silu_f(av[j]) * bv[j];
    store8(out + 8 * i, o);
  }
  for (long long i = 8 * n8 + tid; i < n; i += stride) out[i] = from_f<T>(silu_f(to_f(a[i])) * to_f(b[i]));
}

template <typename T>
__global__ void swiglu_bwd_kernel(const T* __restrict__ g, const T* __restrict__ a, const T* __restrict__ b,
                                  T* __restrict__ da, T* __restrict__ db, long long n, long long n8) {
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = tid; i < n8; i += stride) {
    float gv[8], av[8], bv[8], oa[8], ob[8];
    load8(g + 8 * i, gv);
    load8(a + 8 * i, av);
    load8(b + 8 * i, bv);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      oa[j] = gv[j] * bv[j] * silu_grad_f(av[j]);
      ob[j] = gv[j] * silu_f(av[j]);
    }
    store8(da + 8 * i, oa);
    store8(db + 8 * i, ob);
  }
  for (long long i = 8 * n8 + tid; i < n; i += stride) {
    const float gv = to_f(g[i]), av = to_f(a[i]), bv = to_f(b[i]);
    da[i] = from_f<T>(gv * bv * silu_grad_f(av));
    db[i] = from_f<T>(gv * silu_f(av));
  }
}

// x [rows, H, Dh]; position of a row is row % L; freqs [L, Dh/2] (cos, sin)
template <typename T>
__global__ void rotary_kernel(const T* __restrict__ x, const float2* __restrict__ freqs, T* __restrict__ out,
                              long long rows, int L, int H, int Dh, bool conj) {
  const int half = Dh / 2;
  const long long total = rows * H * half;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int k = (int)(i % half);
    const long long rh = i / half;
    const long long row = rh / H;
    const int pos = (int)(row % L);
    const float2 f = freqs[(long long)pos * half + k];
    const float c = f.x, s = conj ? -f.y : f.y;
    const float xr = to_f(x[2 * i]), xi = to_f(x[2 * i + 1]);
    out[2 * i] = from_f<T>(xr * c - xi * s);
    out[2 * i + 1] = from_f<T>(xr * s + xi * c);
  }
}

// one CTA per row
template <typename T>
__global__ void ce_fwd_kernel(const T* __restrict__ logits, const long long* __restrict__ target,
                              float* __restrict__ loss, float* __restrict__ lse, int V, long long ignore_index) {
  __shared__ float scratch[32];
  const long long row = blockIdx.x;
  const T* lr = logits + row * V;
  float m = -INFINITY;
  for (int j = threadIdx.x; j < V; j += blockDim.x) m = fmaxf(m, to_f(lr[j]));
  m = block_max(m, scratch);
  float s = 0.f;
  for (int j = threadIdx.x; j < V; j += blockDim.x) s += __expf(to_f(lr[j]) - m);
  s = block_sum(s, scratch);
  if (threadIdx.x == 0) {
    const float l = m + logf(s);
    lse[row] = l;
    const long long t = target[row];
    loss[row] = (t == ignore_index || t < 0 || t >= V) ? 0.f : l - to_f(lr[t]);
  }
}

template <typename T>
__global__ void ce_bwd_kernel(const T* __restrict__ logits, const long long* __restrict__ target,
                              const float* __restrict__ lse, const float* __restrict__ dloss,
                              T* __restrict__ dlogits, int V, long long ignore_index) {
  const long long row = blockIdx.x;
  const long long t = target[row];
  const bool skip = (t == ignore_index || t < 0 || t >= V);
  const float g = skip ? 0.f : dloss[row];
  const float l = lse[row];
  const T* lr = logits + row * V;
  T* dr = dlogits + row * V;
  for (int j = threadIdx.x; j < V; j += blockDim.x) {
    float p = __expf(to_f(lr[j]) - l);
    if (j == t) p -= 1.f;
    dr[j] = from_f<T>(p * g);
  }
}

__device__ __forceinline__ void load4(const float* p, float (&o)[4]) {
  const float4 t = *reinterpret_cast<const float4*>(p);
  o[0] = t.x; o[1] = t.y; o[2] = t.z; o[3] = t.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&o)[4]) {
  const uint2 t = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
  o[0] = __low2float(a); o[1] = __high2float(a); o[2] = __low2float(b); o[3] = __high2float(b);
}
__device__ __forceinline__ void load4(const __half* p, float (&o)[4]) {
  const uint2 t = *reinterpret_cast<const uint2*>(p);
  const __half2 a = *reinterpret_cast<const __half2*>(&t.x);
  const __half2 b = *reinterpret_cast<const __half2*>(&t.y);
  o[0] = __low2float(a); o[1] = __high2float(a); o[2] = __low2float(b); o[3] = __high2float(b);
}
__device__ __forceinline__ void store4(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float (&v)[4]) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 t;
  t.x = *reinterpret_cast<uint32_t*>(&a);
  t.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = t;
}
__device__ __forceinline__ void store4(__half* p, const float (&v)[4]) {
  __half2 a = __floats2half2_rn(v[0], v[1]), b = __floats2half2_rn(v[2], v[3]);
  uint2 t;
  t.x = *reinterpret_cast<uint32_t*>(&a);
  t.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = t;
}

// Four elements per thread per iteration (16-byte accesses to the fp32 state).
template <typename G, typename Lo>
__global__ void adamw_kernel(float* __restrict__ p, const G* __restrict__ g, float* __restrict__ m,
                             float* __restrict__ v, Lo* __restrict__ low, long long n, float lr, float beta1,
                             float beta2, float eps, float wd, float bc1, float bc2_sqrt, float grad_scale,
                             const float* __restrict__ scale_ptr) {
  const float gs = grad_scale * (scale_ptr ? *scale_ptr : 1.f);
  const float step = lr / bc1;
  const float decay = 1.f - lr * wd;
  const long long n4 = n / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4;
       i += (long long)gridDim.x * blockDim.x) {
    float pv[4], gv[4], mv[4], vv[4];
    load4(p + 4 * i, pv);
    load4(g + 4 * i, gv);
    load4(m + 4 * i, mv);
    load4(v + 4 * i, vv);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gj = gv[j] * gs;
      mv[j] = beta1 * mv[j] + (1.f - beta1) * gj;
      vv[j] = beta2 * vv[j] + (1.f - beta2) * gj * gj;
      pv[j] = pv[j] * decay - step * mv[j] / (sqrtf(vv[j]) / bc2_sqrt + eps);
    }
    store4(m + 4 * i, mv);
    store4(v + 4 * i, vv);
    store4(p + 4 * i, pv);
    if (low != nullptr) store4(low + 4 * i, pv);
  }
  // tail (n not a multiple of 4)
  for (long long i = n4 * 4 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float gj = to_f(g[i]) * gs;
    const float mj = beta1 * m[i] + (1.f - beta1) * gj;
    const float vj = beta2 * v[i] + (1.f - beta2) * gj * gj;
    const float pj = p[i] * decay - step * mj / (sqrtf(vj) / bc2_sqrt + eps);
    m[i] = mj;
    v[i] = vj;
    p[i] = pj;
    if (low != nullptr) low[i] = from_f<Lo>(pj);
  }
}

template <typename T>
__global__ void sumsq_kernel(const T* __restrict__ g, long long n, double* __restrict__ out) {
  __shared__ float scratch[32];
  float acc = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float v = to_f(g[i]);
    acc += v * v;
  }
  acc = block_sum(acc, scratch);
  if (threadIdx.x == 0) atomicAdd(out, (double)acc);
}

template <typename T>
__global__ void scale_by_ptr_kernel(T* __restrict__ g, long long n, const float* __restrict__ scale) {
  const float s = *scale;
  if (s == 1.f) return;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    g[i] = from_f<T>(to_f(g[i]) * s);
}

// coef = min(1, max_norm / (sqrt(sumsq) + 1e-6)); also writes the norm
__global__ void clip_coef_kernel(const double* __restrict__ sumsq, float max_norm, float* __restrict__ norm_out,
                                 float* __restrict__ coef_out) {
  const float norm = (float)sqrt(*sumsq);
  *norm_out = norm;
  const float c = max_norm / (norm + 1e-6f);
  *coef_out = c < 1.f ? c : 1.f;
}

int ew_grid(long long n) { return (int)std::min<long long>(div_up(n, 256), 148LL * 16); }

}  // namespace

void swiglu_fwd(const void* a, const void* b, void* out, long long n, int dtype, cudaStream_t st) {
  if (n == 0) return;
  const long long n8 = (aligned32(a) && aligned32(b) && aligned32(out)) ? n / 8 : 0;
  MB_DISPATCH_DTYPE(dtype, (swiglu_fwd_kernel<scalar_t><<<ew_grid(std::max(n8, n - 8 * n8)), 256, 0, st>>>(
                               (const scalar_t*)a, (const scalar_t*)b, (scalar_t*)out, n, n8)));
}

void swiglu_bwd(const void* g, const void* a, const void* b, void* da, void* db, long long n, int dtype,
                cudaStream_t st) {
  if (n == 0) return;
  const long long n8 = (aligned32(g) && aligned32(a) && aligned32(b) && aligned32(da) && aligned32(db)) ? n / 8 : 0;
  MB_DISPATCH_DTYPE(dtype, (swiglu_bwd_kernel<scalar_t><<<ew_grid(std::max(n8, n - 8 * n8)), 256, 0, st>>>(
                               (const scalar_t*)g, (const scalar_t*)a, (const scalar_t*)b, (scalar_t*)da,
                               (scalar_t*)db, n, n8)));
}

void rotary_apply(const void* x, const float* freqs, void* out, long long rows, int L, int H, int Dh,
                  bool conj, int dtype, cudaStream_t st) {
  const long long n = rows * H * (Dh / 2);
  MB_DISPATCH_DTYPE(dtype, (rotary_kernel<scalar_t><<<ew_grid(n), 256, 0, st>>>(
                               (const scalar_t*)x, (const float2*)freqs, (scalar_t*)out, rows, L, H, Dh, conj)));
}

void cross_entropy_fwd(const void* logits, const long long* target, float* loss, float* lse, long long rows,
                       int V, long long ignore_index, int dtype, cudaStream_t st) {
  if (rows == 0) return;
  MB_DISPATCH_DTYPE(dtype, (ce_fwd_kernel<scalar_t><<<(unsigned)rows, 256, 0, st>>>(
                               (const scalar_t*)logits, target, loss, lse, V, ignore_index)));
}

void cross_entropy_bwd(const void* logits, const long long* target, const float* lse, const float* dloss,
                       void* dlogits, long long rows, int V, long long ignore_index, int dtype,
                       cudaStream_t st) {
  if (rows == 0) return;
  MB_DISPATCH_DTYPE(dtype, (ce_bwd_kernel<scalar_t><<<(unsigned)rows, 256, 0, st>>>(
                               (const scalar_t*)logits, target, lse, dloss, (scalar_t*)dlogits, V, ignore_index)));
}

void adamw_step(float* p, const void* g, float* m, float* v, void* low, long long n, float lr, float beta1,
                float beta2, float eps, float wd, int step, float grad_scale, const float* scale_ptr,
                int g_dtype, int low_dtype, cudaStream_t st) {
  if (n == 0) return;
  const float bc1 = 1.f - powf(beta1, (float)step);
  const float bc2s = sqrtf(1.f - powf(beta2, (float)step));
  const int grid = ew_grid((n + 3) / 4);
  MB_DISPATCH_DTYPE(g_dtype, {
    using G = scalar_t;
    if (low == nullptr || low_dtype == kBF16) {
      adamw_kernel<G, __nv_bfloat16><<<grid, 256, 0, st>>>(p, (const G*)g, m, v, (__nv_bfloat16*)low, n, lr,
                                                          beta1, beta2, eps, wd, bc1, bc2s, grad_scale, scale_ptr);
    } else if (low_dtype == kF16) {
      adamw_kernel<G, __half><<<grid, 256, 0, st>>>(p, (const G*)g, m, v, (__half*)low, n, lr, beta1, beta2,
                                                   eps, wd, bc1, bc2s, grad_scale, scale_ptr);
    } else {
      adamw_kernel<G, float><<<grid, 256, 0, st>>>(p, (const G*)g, m, v, (float*)low, n, lr, beta1, beta2, eps,
                                                  wd, bc1, bc2s, grad_scale, scale_ptr);
    }
  });
}

void sum_squares(const void* g, long long n, double* out, int dtype, cudaStream_t st) {
  if (n == 0) return;
  MB_DISPATCH_DTYPE(dtype, (sumsq_kernel<scalar_t><<<ew_grid(n), 256, 0, st>>>((const scalar_t*)g, n, out)));
}

void scale_by_ptr(void* g, long long n, const float* scale, int dtype, cudaStream_t st) {
  if (n == 0) return;
  MB_DISPATCH_DTYPE(dtype, (scale_by_ptr_kernel<scalar_t><<<ew_grid(n), 256, 0, st>>>((scalar_t*)g, n, scale)));
}

void clip_coef(const double* sumsq, float max_norm, float* norm_out, float* coef_out, cudaStream_t st) {
  clip_coef_kernel<<<1, 1, 0, st>>>(sumsq, max_norm, norm_out, coef_out);
}

}  // namespace mb
