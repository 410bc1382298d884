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

// da = g * silu'(a): the backward of a SiLU fused into a GEMM epilogue (two reads, one write)
template <typename T>
__global__ void silu_bwd_kernel(const T* __restrict__ g, const T* __restrict__ a, T* __restrict__ da, long long n,
                                long long n8) {
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = tid; i < n8; i += stride) {
    float gv[8], av[8], oa[8];
    load8(g + 8 * i, gv);
    load8(a + 8 * i, av);
#pragma unroll
    for (int j = 0; j < 8; ++j) oa[j] = gv[j] * silu_grad_f(av[j]);
    store8(da + 8 * i, oa);
  }
  for (long long i = 8 * n8 + tid; i < n; i += stride) da[i] = from_f<T>(to_f(g[i]) * silu_grad_f(to_f(a[i])));
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

// Shared q / k of the MEGA attention from the normalised z, in one pass:
//   q = rot(z * (gamma_q + 1) / sqrt(Dh) + beta_q),  k = rot(z * (gamma_k + 1) / sqrt(Dh) + beta_k)
// z, q, k [rows, S] with S = H * Dh, gamma / beta [2, S] (row 0 for q, row 1 for k), rot = the rotary
// rotation of pairs (2j, 2j + 1) by freqs[row % P, j % (Dh / 2)].  One thread per 4 pairs (16-byte accesses).
template <typename T, typename W>
__global__ void qk_rotary_fwd_kernel(const T* __restrict__ z, const W* __restrict__ gamma, const W* __restrict__ beta,
                                     const float2* __restrict__ freqs, T* __restrict__ q, T* __restrict__ k,
                                     long long rows, int S, int Dh, int P, float inv_sqrt) {
  const int per_row = S / 8;
  const long long total = rows * per_row;
  const int half = Dh / 2;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / per_row;
    const int c0 = (int)(i - row * per_row) * 8;
    const int pos = (int)(row % P);
    float zv[8], qv[8], kv[8];
    load8(z + row * S + c0, zv);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = c0 + 2 * j;
      const float2 f = freqs[(long long)pos * half + ((c % Dh) >> 1)];
      const float a0 = zv[2 * j] * (to_f(gamma[c]) + 1.f) * inv_sqrt + to_f(beta[c]);
      const float a1 = zv[2 * j + 1] * (to_f(gamma[c + 1]) + 1.f) * inv_sqrt + to_f(beta[c + 1]);
      const float b0 = zv[2 * j] * (to_f(gamma[S + c]) + 1.f) * inv_sqrt + to_f(beta[S + c]);
      const float b1 = zv[2 * j + 1] * (to_f(gamma[S + c + 1]) + 1.f) * inv_sqrt + to_f(beta[S + c + 1]);
      qv[2 * j] = a0 * f.x - a1 * f.y; qv[2 * j + 1] = a0 * f.y + a1 * f.x;
      kv[2 * j] = b0 * f.x - b1 * f.y; kv[2 * j + 1] = b0 * f.y + b1 * f.x;
    }
    store8(q + row * S + c0, qv);
    store8(k + row * S + c0, kv);
  }
}

// Backward of the above.  CTA = S / 8 threads (thread t owns columns [8t, 8t + 8)) walking a slab of rows:
// dz per element, and per CTA one partial row of d gamma_q, d gamma_k, d beta_q, d beta_k
// (partial [gridDim.x, 4, S] fp32, summed over CTAs afterwards).
template <typename T, typename W>
__global__ void qk_rotary_bwd_kernel(const T* __restrict__ dq, const T* __restrict__ dk, const T* __restrict__ z,
                                     const W* __restrict__ gamma, const float2* __restrict__ freqs,
                                     T* __restrict__ dz, float* __restrict__ partial, long long rows, int S, int Dh,
                                     int P, float inv_sqrt) {
  const int c0 = threadIdx.x * 8;
  if (c0 >= S) return;
  const int half = Dh / 2;
  const long long slab = (rows + gridDim.x - 1) / gridDim.x;
  const long long r0 = (long long)blockIdx.x * slab, r1 = min(rows, r0 + slab);
  float sq[8], sk[8], gq[8], gk[8], bq[8], bk[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    sq[j] = (to_f(gamma[c0 + j]) + 1.f) * inv_sqrt;
    sk[j] = (to_f(gamma[S + c0 + j]) + 1.f) * inv_sqrt;
    gq[j] = gk[j] = bq[j] = bk[j] = 0.f;
  }
  for (long long row = r0; row < r1; ++row) {
    const int pos = (int)(row % P);
    float a[8], b[8], zv[8], o[8];
    load8(dq + row * S + c0, a);
    load8(dk + row * S + c0, b);
    load8(z + row * S + c0, zv);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = freqs[(long long)pos * half + (((c0 + 2 * j) % Dh) >> 1)];
      // inverse rotation of the incoming gradients
      const float a0 = a[2 * j] * f.x + a[2 * j + 1] * f.y, a1 = -a[2 * j] * f.y + a[2 * j + 1] * f.x;
      const float b0 = b[2 * j] * f.x + b[2 * j + 1] * f.y, b1 = -b[2 * j] * f.y + b[2 * j + 1] * f.x;
      o[2 * j] = a0 * sq[2 * j] + b0 * sk[2 * j];
      o[2 * j + 1] = a1 * sq[2 * j + 1] + b1 * sk[2 * j + 1];
      gq[2 * j] = fmaf(a0, zv[2 * j], gq[2 * j]);         gq[2 * j + 1] = fmaf(a1, zv[2 * j + 1], gq[2 * j + 1]);
      gk[2 * j] = fmaf(b0, zv[2 * j], gk[2 * j]);         gk[2 * j + 1] = fmaf(b1, zv[2 * j + 1], gk[2 * j + 1]);
      bq[2 * j] += a0; bq[2 * j + 1] += a1;
      bk[2 * j] += b0; bk[2 * j + 1] += b1;
    }
    store8(dz + row * S + c0, o);
  }
  float* pr = partial + (long long)blockIdx.x * 4 * S;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    pr[c0 + j] = gq[j] * inv_sqrt;
    pr[S + c0 + j] = gk[j] * inv_sqrt;
    pr[2 * S + c0 + j] = bq[j];
    pr[3 * S + c0 + j] = bk[j];
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

void silu_bwd(const void* g, const void* a, void* da, long long n, int dtype, cudaStream_t st) {
  if (n == 0) return;
  const long long n8 = (aligned32(g) && aligned32(a) && aligned32(da)) ? n / 8 : 0;
  MB_DISPATCH_DTYPE(dtype, (silu_bwd_kernel<scalar_t><<<ew_grid(std::max(n8, n - 8 * n8)), 256, 0, st>>>(
                               (const scalar_t*)g, (const scalar_t*)a, (scalar_t*)da, n, n8)));
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

// gamma / beta are fp32 or of the activation dtype (w_dtype)
void qk_rotary_fwd(const void* z, const void* gamma, const void* beta, const float* freqs, void* q, void* k,
                   long long rows, int S, int Dh, int P, int dtype, int w_dtype, cudaStream_t st) {
  if (rows == 0) return;
  const long long n = rows * (S / 8);
  const float inv = 1.f / sqrtf((float)Dh);
  MB_DISPATCH_16BIT(dtype, {
    if (w_dtype == kF32)
      qk_rotary_fwd_kernel<scalar_t, float><<<ew_grid(n), 256, 0, st>>>((const scalar_t*)z, (const float*)gamma,
          (const float*)beta, (const float2*)freqs, (scalar_t*)q, (scalar_t*)k, rows, S, Dh, P, inv);
    else
      qk_rotary_fwd_kernel<scalar_t, scalar_t><<<ew_grid(n), 256, 0, st>>>((const scalar_t*)z, (const scalar_t*)gamma,
          (const scalar_t*)beta, (const float2*)freqs, (scalar_t*)q, (scalar_t*)k, rows, S, Dh, P, inv);
  });
}

int qk_rotary_bwd_ctas(long long rows) { return (int)std::max<long long>(1, std::min<long long>(rows / 8, 148LL * 4)); }

// partial: [qk_rotary_bwd_ctas(rows), 4, S] fp32 (rows of d gamma_q, d gamma_k, d beta_q, d beta_k per CTA)
void qk_rotary_bwd(const void* dq, const void* dk, const void* z, const void* gamma, const float* freqs, void* dz,
                   float* partial, long long rows, int S, int Dh, int P, int dtype, int w_dtype, cudaStream_t st) {
  if (rows == 0) return;
  const float inv = 1.f / sqrtf((float)Dh);
  const int grid = qk_rotary_bwd_ctas(rows);
  const int threads = ((S / 8 + 31) / 32) * 32;
  MB_DISPATCH_16BIT(dtype, {
    if (w_dtype == kF32)
      qk_rotary_bwd_kernel<scalar_t, float><<<grid, threads, 0, st>>>((const scalar_t*)dq, (const scalar_t*)dk,
          (const scalar_t*)z, (const float*)gamma, (const float2*)freqs, (scalar_t*)dz, partial, rows, S, Dh, P, inv);
    else
      qk_rotary_bwd_kernel<scalar_t, scalar_t><<<grid, threads, 0, st>>>((const scalar_t*)dq, (const scalar_t*)dk,
          (const scalar_t*)z, (const scalar_t*)gamma, (const float2*)freqs, (scalar_t*)dz, partial, rows, S, Dh, P, inv);
  });
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
