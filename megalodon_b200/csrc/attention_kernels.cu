// Softmax stages of chunk-local attention, forward and backward, in place on
// the score matrix produced by the tcgen05 GEMM.
//
// Same semantics as the reference's standalone softmax op
// (csrc/softmax.cuh:86-234): with a causal mask, row r of an L1 x L2 block sees
// columns 0 .. L2 - L1 + r; a fully masked row gives zeros; DropKey removes
// keys (sets their logit to -inf with probability p) *before* the softmax.
// Because dropped keys get probability zero, the backward pass
// dS = P * (dP - sum(P * dP)) needs no mask.
//
// Layout: `rows` rows of length L2 with row stride `ld`; row index modulo L1 is
// the query position.  The forward pass also writes zeros to the masked columns
// up to the next multiple of 256, because the causal GEMMs that follow read
// whole diagonal tiles of up to 256 rows; columns further right are never read by them
// and are left untouched (they may hold uninitialised scores).
#include "common.cuh"
#include "kernels.h"

namespace mb {
namespace {

constexpr int kSmThreads = 256;
constexpr int kCausalTile = 256;      // row extent of the largest GEMM tile that reads the diagonal blocks
constexpr int kSmMaxPerThread = 32;   // rows up to 8192 columns

// Philox4x32-10 counter-based generator (Salmon et al. 2011): 4 x 32 random bits per counter.
__device__ __forceinline__ uint4 philox4x32(uint4 ctr, uint2 key) {
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

__device__ __forceinline__ float uniform01(unsigned long long seed, unsigned long long offset,
                                           unsigned long long idx) {
  const unsigned long long c = idx >> 2;
  const uint4 r = philox4x32(make_uint4((unsigned int)c, (unsigned int)(c >> 32), (unsigned int)offset,
                                        (unsigned int)(offset >> 32)),
                             make_uint2((unsigned int)seed, (unsigned int)(seed >> 32)));
  const unsigned int w = (idx & 3) == 0 ? r.x : (idx & 3) == 1 ? r.y : (idx & 3) == 2 ? r.z : r.w;
  return (w >> 8) * (1.0f / 16777216.0f);
}

template <typename T>
__global__ void attn_softmax_fwd_kernel(T* __restrict__ s, float* __restrict__ lse, int L1, int L2,
                                        long long ld, bool causal, float drop_p, unsigned long long seed,
                                        unsigned long long offset) {
  __shared__ float scratch[32];
  const long long row = blockIdx.x;
  const int pos = (int)(row % L1);
  const int n = causal ? max(0, min(L2, L2 - L1 + pos + 1)) : L2;      // visible columns
  const int zero_to = causal ? min(L2, ((n + kCausalTile - 1) / kCausalTile) * kCausalTile) : L2;  // masked columns that must read as 0
  T* sr = s + row * ld;
  float v[kSmMaxPerThread];
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < kSmMaxPerThread; ++i) {
    const int c = threadIdx.x + i * kSmThreads;
    float x = -INFINITY;
    if (c < n) {
      x = to_f(sr[c]);
      if (drop_p > 0.f && uniform01(seed, offset, (unsigned long long)row * L2 + c) < drop_p) x = -INFINITY;
    }
    v[i] = x;
    m = fmaxf(m, x);
  }
  m = block_max(m, scratch);
  float sum = 0.f;
  if (m > -INFINITY) {
#pragma unroll
    for (int i = 0; i < kSmMaxPerThread; ++i) {
      v[i] = __expf(v[i] - m);          // exp(-inf) = 0 for masked / dropped entries
      sum += v[i];
    }
  }
  sum = block_sum(sum, scratch);
  const float inv = sum > 0.f ? 1.f / sum : 0.f;
#pragma unroll
  for (int i = 0; i < kSmMaxPerThread; ++i) {
    const int c = threadIdx.x + i * kSmThreads;
    if (c < n) sr[c] = from_f<T>(m > -INFINITY ? v[i] * inv : 0.f);
    else if (c < zero_to) sr[c] = from_f<T>(0.f);
  }
  if (lse != nullptr && threadIdx.x == 0) lse[row] = sum > 0.f ? m + logf(sum) : -INFINITY;
}

template <typename T>
__global__ void attn_softmax_bwd_kernel(const T* __restrict__ p, T* __restrict__ dp, int L1, int L2, long long ld,
                                        bool causal) {
  __shared__ float scratch[32];
  const long long row = blockIdx.x;
  const int pos = (int)(row % L1);
  const int n = causal ? max(0, min(L2, L2 - L1 + pos + 1)) : L2;
  const int zero_to = causal ? min(L2, ((n + kCausalTile - 1) / kCausalTile) * kCausalTile) : L2;
  const T* pr = p + row * ld;
  T* dr = dp + row * ld;
  float pv[kSmMaxPerThread], gv[kSmMaxPerThread];
  float dot = 0.f;
#pragma unroll
  for (int i = 0; i < kSmMaxPerThread; ++i) {
    const int c = threadIdx.x + i * kSmThreads;
    pv[i] = gv[i] = 0.f;
    if (c < n) {
      pv[i] = to_f(pr[c]);
      gv[i] = to_f(dr[c]);
      dot += pv[i] * gv[i];
    }
  }
  dot = block_sum(dot, scratch);
#pragma unroll
  for (int i = 0; i < kSmMaxPerThread; ++i) {
    const int c = threadIdx.x + i * kSmThreads;
    if (c < n) dr[c] = from_f<T>(pv[i] * (gv[i] - dot));
    else if (c < zero_to) dr[c] = from_f<T>(0.f);
  }
}


// 16-byte variants: a thread owns up to kSmVecPerThread groups of 8 consecutive columns.  Requires
// L2 % 8 == 0, ld % 8 == 0 and a 16-byte aligned base, so every group is either entirely inside or
// entirely outside [0, zero_to) (zero_to is a multiple of 128 or L2 itself).
constexpr int kSmVecPerThread = kSmMaxPerThread / 8;

template <typename T>
__global__ void attn_softmax_fwd_vec_kernel(T* __restrict__ s, float* __restrict__ lse, int L1, int L2,
                                            long long ld, bool causal, float drop_p, unsigned long long seed,
                                            unsigned long long offset) {
  __shared__ float scratch[32];
  const long long row = blockIdx.x;
  const int pos = (int)(row % L1);
  const int n = causal ? max(0, min(L2, L2 - L1 + pos + 1)) : L2;
  const int zero_to = causal ? min(L2, ((n + kCausalTile - 1) / kCausalTile) * kCausalTile) : L2;
  T* sr = s + row * ld;
  float v[kSmVecPerThread][8];
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < kSmVecPerThread; ++i) {
    const int c0 = (threadIdx.x + i * kSmThreads) * 8;
    if (c0 < n) {
      load8(sr + c0, v[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int c = c0 + j;
        if (c >= n) v[i][j] = -INFINITY;
        else if (drop_p > 0.f && uniform01(seed, offset, (unsigned long long)row * L2 + c) < drop_p)
          v[i][j] = -INFINITY;
        m = fmaxf(m, v[i][j]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[i][j] = -INFINITY;
    }
  }
  m = block_max(m, scratch);
  float sum = 0.f;
  if (m > -INFINITY) {
    const float ml2 = m * 1.4426950408889634f;
#pragma unroll
    for (int i = 0; i < kSmVecPerThread; ++i) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        v[i][j] = exp2f(fmaf(v[i][j], 1.4426950408889634f, -ml2));      // exp2(-inf) = 0 for masked entries
        sum += v[i][j];
      }
    }
  }
  sum = block_sum(sum, scratch);
  const float inv = (m > -INFINITY && sum > 0.f) ? 1.f / sum : 0.f;
#pragma unroll
  for (int i = 0; i < kSmVecPerThread; ++i) {
    const int c0 = (threadIdx.x + i * kSmThreads) * 8;
    if (c0 < zero_to) {
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (m > -INFINITY) ? v[i][j] * inv : 0.f;
      store8(sr + c0, o);
    }
  }
  if (lse != nullptr && threadIdx.x == 0) lse[row] = sum > 0.f ? m + logf(sum) : -INFINITY;
}

template <typename T>
__global__ void attn_softmax_bwd_vec_kernel(const T* __restrict__ p, T* __restrict__ dp, int L1, int L2,
                                            long long ld, bool causal) {
  __shared__ float scratch[32];
  const long long row = blockIdx.x;
  const int pos = (int)(row % L1);
  const int n = causal ? max(0, min(L2, L2 - L1 + pos + 1)) : L2;
  const int zero_to = causal ? min(L2, ((n + kCausalTile - 1) / kCausalTile) * kCausalTile) : L2;
  const T* pr = p + row * ld;
  T* dr = dp + row * ld;
  float pv[kSmVecPerThread][8], gv[kSmVecPerThread][8];
  float dot = 0.f;
#pragma unroll
  for (int i = 0; i < kSmVecPerThread; ++i) {
    const int c0 = (threadIdx.x + i * kSmThreads) * 8;
    if (c0 < n) {
      load8(pr + c0, pv[i]);
      load8(dr + c0, gv[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (c0 + j >= n) pv[i][j] = gv[i][j] = 0.f;
        dot = fmaf(pv[i][j], gv[i][j], dot);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) pv[i][j] = gv[i][j] = 0.f;
    }
  }
  dot = block_sum(dot, scratch);
#pragma unroll
  for (int i = 0; i < kSmVecPerThread; ++i) {
    const int c0 = (threadIdx.x + i * kSmThreads) * 8;
    if (c0 < zero_to) {
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = pv[i][j] * (gv[i][j] - dot);
      store8(dr + c0, o);
    }
  }
}

inline bool softmax_vec_ok(const void* base, int L2, long long ld, int dtype) {
  return L2 % 8 == 0 && ld % 8 == 0 && (reinterpret_cast<uintptr_t>(base) & 31) == 0;
}

// Backward preparation of the fused-softmax attention: for every (batch, position, head) row of d_v values
//   delta = dO . O          (equals sum_j P_ij dP_ij, the softmax Jacobian's row term)
//   dO'   = dO / rowsum     (so that P~^T dO' = P^T dO with the un-normalised P~ that the forward kept)
// dO, O, dO' are [B, L, H, dv] contiguous; rowsum and delta are [B, H, L] fp32.  One warp per row.
template <typename T>
__global__ void attn_bwd_prep_kernel(const T* __restrict__ dout, const T* __restrict__ out,
                                     const float* __restrict__ rowsum, T* __restrict__ dos,
                                     float* __restrict__ delta, long long rows, int L, int H, int dv) {
  const int lane = threadIdx.x & 31;
  const long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const int h = (int)(r % H);
  const long long bl = r / H;
  const int l = (int)(bl % L);
  const long long b = bl / L;
  const long long vidx = (b * H + h) * L + l;
  const float s = rowsum[vidx];
  const float inv = s > 0.f ? 1.f / s : 0.f;
  const T* g = dout + r * dv;
  const T* o = out + r * dv;
  T* d = dos + r * dv;
  float acc = 0.f;
  for (int c = lane * 8; c < dv; c += 256) {
    float gv[8], ov[8];
    load8(g + c, gv);
    load8(o + c, ov);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      acc = fmaf(gv[i], ov[i], acc);
      gv[i] *= inv;
    }
    store8(d + c, gv);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) delta[vidx] = acc;
}

// One decode step of the chunk attention against fixed-size key / value buffers, reading only the filled
// slots.  q [B, H, dk], k_buf [B, H, C, dk], v_buf [B, H, C, dv], pos: device scalar, index of the newest key
// (keys 0 .. pos are valid).  out [B, H, dv] = softmax(scale q k^T) v.  Grid (B * H, dv / 256), 256 threads:
// every CTA computes the pos + 1 scores (warps stride over the keys, lanes over dk), normalises them in
// shared memory, and accumulates its 256 value columns.  Nothing depends on host-side lengths, so the
// launch can sit in a CUDA graph.
template <typename T>
__global__ void decode_attention_kernel(const T* __restrict__ q, const T* __restrict__ kb, const T* __restrict__ vb,
                                        const long long* __restrict__ pos, T* __restrict__ out, int C, int dk,
                                        int dv, float scale) {
  extern __shared__ float sc[];                 // C scores
  __shared__ float red[32];
  const int bh = blockIdx.x;
  const int n = min((int)pos[0] + 1, C);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const T* qr = q + (long long)bh * dk;
  const T* kr = kb + (long long)bh * C * dk;
  for (int j = warp; j < n; j += nwarps) {
    float acc = 0.f;
    for (int c = lane * 8; c < dk; c += 256) {
      float a[8], b[8];
      load8(qr + c, a);
      load8(kr + (long long)j * dk + c, b);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc = fmaf(a[i], b[i], acc);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0) sc[j] = acc * scale;
  }
  __syncthreads();
  float m = -INFINITY;
  for (int j = threadIdx.x; j < n; j += blockDim.x) m = fmaxf(m, sc[j]);
  m = block_max(m, red);
  float sum = 0.f;
  for (int j = threadIdx.x; j < n; j += blockDim.x) {
    const float e = __expf(sc[j] - m);
    sc[j] = e;
    sum += e;
  }
  sum = block_sum(sum, red);
  __syncthreads();
  const int col = blockIdx.y * blockDim.x + threadIdx.x;
  if (col >= dv) return;
  const T* vr = vb + (long long)bh * C * dv + col;
  float acc = 0.f;
  for (int j = 0; j < n; ++j) acc = fmaf(sc[j], to_f(vr[(long long)j * dv]), acc);
  out[(long long)bh * dv + col] = from_f<T>(acc / sum);
}

}  // namespace

void decode_attention(const void* q, const void* kb, const void* vb, const long long* pos, void* out, int BH, int C,
                      int dk, int dv, float scale, int dtype, cudaStream_t st) {
  if (BH == 0) return;
  dim3 grid(BH, div_up(dv, 256));
  const size_t smem = sizeof(float) * C;
  MB_DISPATCH_16BIT(dtype, {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(decode_attention_kernel<scalar_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    decode_attention_kernel<scalar_t><<<grid, 256, smem, st>>>((const scalar_t*)q, (const scalar_t*)kb, (const scalar_t*)vb,
                                                                pos, (scalar_t*)out, C, dk, dv, scale);
  });
}

void attn_bwd_prep(const void* dout, const void* out, const float* rowsum, void* dos, float* delta, int B, int L,
                   int H, int dv, int dtype, cudaStream_t st) {
  const long long rows = (long long)B * L * H;
  if (rows == 0) return;
  const int warps = 8;
  MB_DISPATCH_16BIT(dtype, (attn_bwd_prep_kernel<scalar_t><<<(unsigned)div_up(rows, warps), warps * 32, 0, st>>>(
                               (const scalar_t*)dout, (const scalar_t*)out, rowsum, (scalar_t*)dos, delta, rows, L, H,
                               dv)));
}

void attn_softmax_fwd(void* s_inout, float* lse, long long rows, int L1, int L2, long long ld, bool causal,
                      float dropkey_p, unsigned long long seed, unsigned long long offset, int dtype,
                      cudaStream_t st) {
  if (rows == 0) return;
  if (softmax_vec_ok(s_inout, L2, ld, dtype)) {
    MB_DISPATCH_DTYPE(dtype, (attn_softmax_fwd_vec_kernel<scalar_t><<<(unsigned)rows, kSmThreads, 0, st>>>(
                                 (scalar_t*)s_inout, lse, L1, L2, ld, causal, dropkey_p, seed, offset)));
    return;
  }
  MB_DISPATCH_DTYPE(dtype, (attn_softmax_fwd_kernel<scalar_t><<<(unsigned)rows, kSmThreads, 0, st>>>(
                               (scalar_t*)s_inout, lse, L1, L2, ld, causal, dropkey_p, seed, offset)));
}

void attn_softmax_bwd(const void* p, void* dp_inout, long long rows, int L1, int L2, long long ld, bool causal,
                      int dtype, cudaStream_t st) {
  if (rows == 0) return;
  if (softmax_vec_ok(p, L2, ld, dtype) && (reinterpret_cast<uintptr_t>(dp_inout) & 31) == 0) {
    MB_DISPATCH_DTYPE(dtype, (attn_softmax_bwd_vec_kernel<scalar_t><<<(unsigned)rows, kSmThreads, 0, st>>>(
                                 (const scalar_t*)p, (scalar_t*)dp_inout, L1, L2, ld, causal)));
    return;
  }
  MB_DISPATCH_DTYPE(dtype, (attn_softmax_bwd_kernel<scalar_t><<<(unsigned)rows, kSmThreads, 0, st>>>(
                               (const scalar_t*)p, (scalar_t*)dp_inout, L1, L2, ld, causal)));
}

}  // namespace mb
