// SequenceNorm building blocks and the memory-efficient dropout kernel.
//
// SequenceNorm normalises over the whole (non-padded) time axis per (batch,
// feature) or per (batch, group), for both the [B, L, H] and the [B, H, L]
// layout (reference: csrc/ops/sequence_norm.cc:259-529 and the 20 kernels of
// sequence_norm_kernel.cu).  Forward and backward both reduce to two bandwidth
// bound passes, so the native part is two kernels shared by all variants:
//
//   time_sums     per (b, h): sum over valid t of (u, u * v or u^2)
//                 forward:  u = x           -> sum x, sum x^2
//                 backward: u = dy, v = x   -> sum dy, sum dy * x
//   affine_apply  out[b, t, h] = a[b, h] * p + c[b, h] * q + d[b, h]  (0 on padded steps)
//                 forward:  y  = (r gamma) x + (beta - u r gamma)
//                 backward: dx = (r gamma) dy + (2 c dv) x + (c du - 2 c dv u)
//
// The [B, H]-sized statistics in between are combined on the caller's side.
//
// Dropout: counter-based Philox mask generated in the kernel from (seed, offset,
// element index), so the backward pass regenerates the mask instead of storing
// it (same idea as the reference's RNG-state replay, fused_ops/memory_efficient_dropout.py).
#include "common.cuh"
#include "kernels.h"

namespace mb {
namespace {

// x indexed [b, t, h]; `length_last` means memory layout [B, H, L]
__device__ __forceinline__ long long at(int b, int t, int h, int L, int H, bool length_last) {
  return length_last ? ((long long)b * H + h) * L + t : ((long long)b * L + t) * H + h;
}

// block (32, 8): threadIdx.x walks features (coalesced for [B, L, H]), threadIdx.y strides over time
template <typename T, bool PRODUCT>
__global__ void time_sums_blh_kernel(const T* __restrict__ u, const T* __restrict__ v, const bool* __restrict__ mask,
                                     float* __restrict__ s1, float* __restrict__ s2, int L, int H) {
  __shared__ float sh1[8][33], sh2[8][33];
  const int b = blockIdx.y;
  const int h = blockIdx.x * 32 + threadIdx.x;
  float a = 0.f, c = 0.f;
  if (h < H) {
    for (int t = threadIdx.y; t < L; t += 8) {
      if (mask && mask[(long long)b * L + t]) continue;
      const long long i = ((long long)b * L + t) * H + h;
      const float uu = to_f(u[i]);
      a += uu;
      c += PRODUCT ? uu * to_f(v[i]) : uu * uu;
    }
  }
  sh1[threadIdx.y][threadIdx.x] = a;
  sh2[threadIdx.y][threadIdx.x] = c;
  __syncthreads();
  if (threadIdx.y == 0 && h < H) {
    for (int k = 1; k < 8; ++k) {
      a += sh1[k][threadIdx.x];
      c += sh2[k][threadIdx.x];
    }
    s1[(long long)b * H + h] = a;
    s2[(long long)b * H + h] = c;
  }
}

// [B, H, L]: one CTA per (b, h) row
template <typename T, bool PRODUCT>
__global__ void time_sums_bhl_kernel(const T* __restrict__ u, const T* __restrict__ v, const bool* __restrict__ mask,
                                     float* __restrict__ s1, float* __restrict__ s2, int L, int H) {
  __shared__ float scratch[32];
  const long long row = blockIdx.x;            // b * H + h
  const int b = (int)(row / H);
  float a = 0.f, c = 0.f;
  for (int t = threadIdx.x; t < L; t += blockDim.x) {
    if (mask && mask[(long long)b * L + t]) continue;
    const float uu = to_f(u[row * L + t]);
    a += uu;
    c += PRODUCT ? uu * to_f(v[row * L + t]) : uu * uu;
  }
  a = block_sum(a, scratch);
  c = block_sum(c, scratch);
  if (threadIdx.x == 0) {
    s1[row] = a;
    s2[row] = c;
  }
}

template <typename T>
__global__ void affine_apply_kernel(const T* __restrict__ p, const T* __restrict__ q, const float* __restrict__ a,
                                    const float* __restrict__ c, const float* __restrict__ d,
                                    const bool* __restrict__ mask, T* __restrict__ out, int B, int L, int H,
                                    bool length_last) {
  const long long total = (long long)B * L * H;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    int b, t, h;
    if (length_last) {
      t = (int)(i % L);
      h = (int)((i / L) % H);
      b = (int)(i / ((long long)L * H));
    } else {
      h = (int)(i % H);
      t = (int)((i / H) % L);
      b = (int)(i / ((long long)L * H));
    }
    float o = 0.f;
    if (!(mask && mask[(long long)b * L + t])) {
      const long long bh = (long long)b * H + h;
      o = a[bh] * to_f(p[i]) + d[bh];
      if (q != nullptr) o += c[bh] * to_f(q[i]);
    }
    out[i] = from_f<T>(o);
  }
}

// Philox4x32-10
__device__ __forceinline__ uint4 philox(uint4 ctr, uint2 key) {
  const unsigned int M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    const unsigned int hi0 = __umulhi(M0, ctr.x), lo0 = M0 * ctr.x;
    const unsigned int hi1 = __umulhi(M1, ctr.z), lo1 = M1 * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += W0;
    key.y += W1;
  }
  return ctr;
}

// out = x * keep / (1 - p), keep ~ Bernoulli(1 - p) from (seed, offset, index); 4 elements per counter
template <typename T>
__global__ void dropout_kernel(const T* __restrict__ x, T* __restrict__ out, long long n, float p,
                               unsigned long long seed, unsigned long long offset) {
  const float scale = 1.f / (1.f - p);
  const long long n4 = (n + 3) / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4;
       i += (long long)gridDim.x * blockDim.x) {
    const uint4 r = philox(make_uint4((unsigned int)i, (unsigned int)(i >> 32), (unsigned int)offset,
                                      (unsigned int)(offset >> 32)),
                           make_uint2((unsigned int)seed, (unsigned int)(seed >> 32)));
    const unsigned int w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long e = 4 * i + j;
      if (e < n) {
        const float uni = (w[j] >> 8) * (1.0f / 16777216.0f);
        out[e] = from_f<T>(uni < p ? 0.f : to_f(x[e]) * scale);
      }
    }
  }
}

}  // namespace

void time_sums(const void* u, const void* v, const bool* mask, float* s1, float* s2, int B, int L, int H,
               bool length_last, int dtype, cudaStream_t st) {
  MB_DISPATCH_DTYPE(dtype, {
    using T = scalar_t;
    if (length_last) {
      if (v != nullptr)
        time_sums_bhl_kernel<T, true><<<B * H, 256, 0, st>>>((const T*)u, (const T*)v, mask, s1, s2, L, H);
      else
        time_sums_bhl_kernel<T, false><<<B * H, 256, 0, st>>>((const T*)u, nullptr, mask, s1, s2, L, H);
    } else {
      dim3 grid(div_up(H, 32), B), block(32, 8);
      if (v != nullptr)
        time_sums_blh_kernel<T, true><<<grid, block, 0, st>>>((const T*)u, (const T*)v, mask, s1, s2, L, H);
      else
        time_sums_blh_kernel<T, false><<<grid, block, 0, st>>>((const T*)u, nullptr, mask, s1, s2, L, H);
    }
  });
}

void affine_apply(const void* p, const void* q, const float* a, const float* c, const float* d, const bool* mask,
                  void* out, int B, int L, int H, bool length_last, int dtype, cudaStream_t st) {
  const long long total = (long long)B * L * H;
  if (total == 0) return;
  const int grid = (int)std::min<long long>(div_up(total, 256), 148LL * 16);
  MB_DISPATCH_DTYPE(dtype, (affine_apply_kernel<scalar_t><<<grid, 256, 0, st>>>(
                               (const scalar_t*)p, (const scalar_t*)q, a, c, d, mask, (scalar_t*)out, B, L, H,
                               length_last)));
}

void dropout_apply(const void* x, void* out, long long n, float p, unsigned long long seed,
                   unsigned long long offset, int dtype, cudaStream_t st) {
  if (n == 0) return;
  const int grid = (int)std::min<long long>(div_up((n + 3) / 4, 256), 148LL * 16);
  MB_DISPATCH_DTYPE(dtype, (dropout_kernel<scalar_t><<<grid, 256, 0, st>>>((const scalar_t*)x, (scalar_t*)out, n, p,
                                                                         seed, offset)));
}

}  // namespace mb
