// Persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   C[M, N] = epilogue( A * B^T )       fp32 accumulation in tensor memory
//
// A supplies M rows, B supplies N rows, both reduced over K.  Each operand is
// either K-major (stored [rows, K], K contiguous) or MN-major (stored
// [K, rows], rows contiguous), so the three GEMMs of a linear layer need no
// transposed copies:
//   forward  y  = x  w^T      A = x  [M, K]  K-major,   B = w  [N, K]  K-major
//   dgrad    dx = dy w        A = dy [M, N'] K-major,   B = w  [N', K'] MN-major
//   wgrad    dw = dy^T x      A = dy [T, N'] MN-major,  B = x  [T, K'] MN-major
//
// CTA = 6 warps: warp 0 issues TMA loads (128B-swizzled tiles, no multicast)
// into a 4-stage shared-memory ring; warp 1 issues tcgen05.mma (128 x BN x 16)
// into one of two TMEM accumulators; warps 2-5 drain the other accumulator
// with tcgen05.ld, apply bias / SiLU and store, so the epilogue of tile i
// overlaps the main loop of tile i+1.  Tiles are walked M-fastest so CTAs that
// run together share B tiles in L2.
//
// All mbarrier waits are bounded; a timeout sets `*err` and the CTA unwinds
// (releasing its TMEM) instead of hanging.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#include "common.cuh"
#include "kernels.h"
#include "sm100_ptx.cuh"

namespace mb {
namespace {

using namespace ptx;

constexpr int BM = 128;
constexpr int BK = 64;          // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int kStages = 4;
constexpr int kGemmThreads = 192;
constexpr int kEpiWarps = 4;
constexpr int kMaxPeers = 8;

template <int BN>
struct SmemLayout {
  static constexpr int a_bytes = BM * BK * 2;       // 16 KiB
  static constexpr int b_bytes = BN * BK * 2;       // 32 KiB at BN = 256
  static constexpr int stage_bytes = a_bytes + b_bytes;
  static constexpr int bar_offset = kStages * stage_bytes;
  static constexpr int total = bar_offset + 256 + 1024;  // barriers + alignment slack
};

// Triangular (causal) structure, used when the GEMM is one of the products of
// chunk-local causal attention (row index and contraction / column index count
// the same positions):
//   1  skip output tiles that lie entirely above the diagonal   (S = Q K^T, dP = dO V^T)
//   2  contract only over k <= last row of the tile             (O = P V, dQ = dS K;  A lower-triangular)
//   3  contract only over k >= first row of the tile            (dV = P^T dO, dK = dS^T Q; A^T lower-triangular)
struct GemmParams {
  int M, N, K;
  void* C;             // [M, N] with row stride ldc
  void* preact;        // optional [M, N]: value before the activation
  const void* bias;    // optional [N]
  int bias_dtype;      // DType
  int act;             // 0 none, 1 SiLU
  int* err;
  long long ldc;       // elements
  int mode;            // 0 dense, 1..3 see above
  float alpha;         // C = alpha * acc (+ bias)
  int accumulate;      // 1: C += alpha * acc (+ bias); the old C is read in the epilogue
  int batch;           // independent problems sharing shapes (tensor maps carry their strides)
  long long c_batch_stride;   // elements between consecutive C (and preact) matrices
  // all-gather -> GEMM: A is the concatenation along K of `a_parts` pieces of `a_part_k` columns, piece i
  // read through tensor map i (a peer GPU's memory); the walk over K starts at piece `a_first`
  int a_parts, a_part_k, a_first;
  // GEMM -> reduce-scatter: column block i of `c_part_cols` columns is stored to c_parts[i] (row stride
  // c_part_cols), a slot in the memory of the rank that owns those columns
  int c_nparts, c_part_cols;
  void* c_parts[kMaxPeers];
  // all-gather -> GEMM on the weight operand (B, K-major [N, K], rows sharded over `g_world` ranks in
  // blocks of N / g_world rows; pair kernel only).  g_src[r] is rank r's block (peer memory for r !=
  // g_rank), g_dst the local full matrix that tmap_b reads.  The copy warps of all CTAs move the matrix
  // in 128-row chunks (claimed 8 KiB at a time through g_flags[0], starting with this rank's own rows);
  // g_flags[1 + c] counts the finished 8 KiB units of chunk c, and a producer loads B rows of chunk c
  // only once all K / 32 of them are in.  The n-tile walk starts at this rank's own rows too.
  int g_world, g_rank;
  const void* g_src[kMaxPeers];
  void* g_dst;
  unsigned int* g_flags;
  // Softmax of chunk-local attention fused into the epilogues of its products (fp32 row vectors indexed
  // [batch, row]; column j of row i takes part iff j <= i + causal_off when mode == 1, always otherwise):
  //   1 row max     nothing is stored; row_out[i] = max(row_out[i], alpha * acc[i, j])        (S = Q K^T, pass 1)
  //   2 exp         C = exp(alpha * acc - row_in[i]) (0 where masked), row_out[i] += sum_j C  (S = Q K^T, pass 2)
  //   3 row scale   C = alpha * acc / row_in[i]  (0 for an empty row)                         (O = P V)
  //   4 dS          C = aux[i, j] / row_in[i] * (alpha * acc - row_in2[i])                    (dP = dO V^T -> dS)
  // `aux` has the layout of C and may be C itself.
  int epi;
  const float* row_in;
  const float* row_in2;
  float* row_out;
  const void* aux;
  int causal_off;
};

struct TmapArray {
  CUtensorMap m[kMaxPeers];
};

struct TileCoord {
  int m0, n0, bz;
};
template <int BN>
__device__ __forceinline__ TileCoord decode_tile(int tile, int num_m, int tiles_per_batch) {
  const int bz = tile / tiles_per_batch;
  const int t = tile - bz * tiles_per_batch;
  return {(t % num_m) * BM, (t / num_m) * BN, bz};
}

template <int BN>
__device__ __forceinline__ bool tile_skipped(const GemmParams& p, int m0, int n0) {
  return p.mode == 1 && n0 > m0 + BM - 1;
}

__device__ __forceinline__ void k_range(const GemmParams& p, int m0, int num_k, int& kb0, int& kb1) {
  kb0 = 0;
  kb1 = num_k;
  if (p.mode == 2) kb1 = min(num_k, (m0 + BM + BK - 1) / BK);
  if (p.mode == 3) kb0 = min(num_k - 1, m0 / BK);
}

__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 0xff) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > kWaitTimeoutNs) return false;
    }
  }
  return true;
}

template <typename OutT>
__device__ __forceinline__ void store_row32(OutT* dst, const float (&v)[32], int ncols_valid);

template <>
__device__ __forceinline__ void store_row32<__nv_bfloat16>(__nv_bfloat16* dst, const float (&v)[32], int nvalid) {
  if (nvalid >= 32) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 pk;
      __nv_bfloat162 t0 = __floats2bfloat162_rn(v[8 * i + 0], v[8 * i + 1]);
      __nv_bfloat162 t1 = __floats2bfloat162_rn(v[8 * i + 2], v[8 * i + 3]);
      __nv_bfloat162 t2 = __floats2bfloat162_rn(v[8 * i + 4], v[8 * i + 5]);
      __nv_bfloat162 t3 = __floats2bfloat162_rn(v[8 * i + 6], v[8 * i + 7]);
      pk.x = *reinterpret_cast<uint32_t*>(&t0);
      pk.y = *reinterpret_cast<uint32_t*>(&t1);
      pk.z = *reinterpret_cast<uint32_t*>(&t2);
      pk.w = *reinterpret_cast<uint32_t*>(&t3);
      reinterpret_cast<uint4*>(dst)[i] = pk;
    }
  } else {
    for (int i = 0; i < nvalid; ++i) dst[i] = __float2bfloat16_rn(v[i]);
  }
}

template <>
__device__ __forceinline__ void store_row32<__half>(__half* dst, const float (&v)[32], int nvalid) {
  if (nvalid >= 32) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 pk;
      __half2 t0 = __floats2half2_rn(v[8 * i + 0], v[8 * i + 1]);
      __half2 t1 = __floats2half2_rn(v[8 * i + 2], v[8 * i + 3]);
      __half2 t2 = __floats2half2_rn(v[8 * i + 4], v[8 * i + 5]);
      __half2 t3 = __floats2half2_rn(v[8 * i + 6], v[8 * i + 7]);
      pk.x = *reinterpret_cast<uint32_t*>(&t0);
      pk.y = *reinterpret_cast<uint32_t*>(&t1);
      pk.z = *reinterpret_cast<uint32_t*>(&t2);
      pk.w = *reinterpret_cast<uint32_t*>(&t3);
      reinterpret_cast<uint4*>(dst)[i] = pk;
    }
  } else {
    for (int i = 0; i < nvalid; ++i) dst[i] = __float2half_rn(v[i]);
  }
}

template <>
__device__ __forceinline__ void store_row32<float>(float* dst, const float (&v)[32], int nvalid) {
  if (nvalid >= 32) {
#pragma unroll
    for (int i = 0; i < 8; ++i)
      reinterpret_cast<float4*>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  } else {
    for (int i = 0; i < nvalid; ++i) dst[i] = v[i];
  }
}

// v[i] += dst[i] for the first nvalid of 32 consecutive elements (accumulating epilogue)
template <typename OutT>
__device__ __forceinline__ void add_row32(const OutT* src, float (&v)[32], int nvalid) {
  if (nvalid >= 32) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float t[8];
      load8(src + 8 * i, t);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[8 * i + j] += t[j];
    }
  } else {
    for (int i = 0; i < nvalid; ++i) v[i] += to_f(src[i]);
  }
}

enum EpiMode : int { kEpiStd = 0, kEpiRowMax = 1, kEpiExp = 2, kEpiRowScale = 3, kEpiDS = 4 };

__device__ __forceinline__ void atomic_max_float(float* addr, float v) {
  if (v >= 0.f) atomicMax(reinterpret_cast<int*>(addr), __float_as_int(v));
  else atomicMin(reinterpret_cast<unsigned int*>(addr), __float_as_uint(v));
}

// Per-row state of the fused-softmax epilogues: one thread owns one output row of the tile.
struct EpiRow {
  float a, b, acc;       // a, b: row scalars read once per tile; acc: running max / sum over the tile
};
__device__ __forceinline__ void epi_row_begin(const GemmParams& p, long long ridx, bool row_ok, EpiRow& r) {
  r.a = r.b = 0.f;
  r.acc = p.epi == kEpiRowMax ? -INFINITY : 0.f;
  if (!row_ok) return;
  if (p.epi == kEpiExp) r.a = p.row_in[ridx];
  else if (p.epi == kEpiRowScale || p.epi == kEpiDS) {
    const float s = p.row_in[ridx];
    r.a = s > 0.f ? 1.f / s : 0.f;
    if (p.epi == kEpiDS) r.b = p.row_in2[ridx];
  }
}
__device__ __forceinline__ void epi_row_end(const GemmParams& p, long long ridx, bool row_ok, const EpiRow& r) {
  if (!row_ok) return;
  if (p.epi == kEpiRowMax) { if (r.acc > -INFINITY) atomic_max_float(p.row_out + ridx, r.acc); }
  else if (p.epi == kEpiExp) atomicAdd(p.row_out + ridx, r.acc);
}
// One 32-column chunk of row `row` (v = alpha * acc).  Returns false when the standard epilogue should run.
template <typename OutT>
__device__ __forceinline__ bool epi_chunk(const GemmParams& p, float (&v)[32], int row, int col0, int nvalid,
                                          long long off, OutT* C, EpiRow& r) {
  if (p.epi == kEpiStd) return false;
  const int last = p.mode == 1 ? row + p.causal_off : 0x7fffffff;      // last column that takes part
  if (p.epi == kEpiRowMax) {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < nvalid && col0 + i <= last) r.acc = fmaxf(r.acc, v[i]);
    return true;
  }
  if (p.epi == kEpiExp) {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      float e = (i < nvalid && col0 + i <= last) ? __expf(v[i] - r.a) : 0.f;
      e = to_f(from_f<OutT>(e));                 // the sum is taken over the values as they are stored
      r.acc += e;
      v[i] = e;
    }
    store_row32<OutT>(C + off, v, nvalid);
    return true;
  }
  if (p.epi == kEpiRowScale) {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] *= r.a;
    store_row32<OutT>(C + off, v, nvalid);
    return true;
  }
  // kEpiDS
  float pt[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) pt[i] = 0.f;
  add_row32<OutT>(reinterpret_cast<const OutT*>(p.aux) + off, pt, nvalid);
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = (i < nvalid && col0 + i <= last) ? pt[i] * r.a * (v[i] - r.b) : 0.f;
  store_row32<OutT>(C + off, v, nvalid);
  return true;
}

template <int BN, bool A_MN, bool B_MN, typename OutT>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ TmapArray tmaps_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ GemmParams p, int in_fmt) {
  using L = SmemLayout<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::bar_offset);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full = empty_bar + kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (p.M + BM - 1) / BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int tiles_per_batch = num_m * num_n;
  const int num_tiles = tiles_per_batch * p.batch;
  const int num_k = (p.K + BK - 1) / BK;
  constexpr uint32_t kTmemCols = 2 * BN;     // two accumulators (power of two: 256 or 512)

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(full_bar + i, 1);
      mbar_init(empty_bar + i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(tmem_full + i, 1);
      mbar_init(tmem_empty + i, kEpiWarps);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, kTmemCols);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      for (int i = 0; i < p.a_parts; ++i) prefetch_tmap(&tmaps_a.m[i]);
      prefetch_tmap(&tmap_b);
      const int kb_shift = p.a_parts > 1 ? p.a_first * (p.a_part_k / BK) : 0;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const TileCoord tc = decode_tile<BN>(tile, num_m, tiles_per_batch);
        const int m0 = tc.m0, n0 = tc.n0, bz = tc.bz;
        if (tile_skipped<BN>(p, m0, n0)) continue;
        int kb0, kb1;
        k_range(p, m0, num_k, kb0, kb1);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!wait_or_abort(empty_bar + stage, phase ^ 1, abort_flag)) { ok = false; break; }
          uint8_t* sa = smem + stage * L::stage_bytes;
          uint8_t* sb = sa + L::a_bytes;
          mbar_expect_tx(full_bar + stage, L::stage_bytes);
          // with a gathered A the K walk is rotated so that every rank starts on its own piece
          const int kbr = p.a_parts > 1 ? (kb + kb_shift) % num_k : kb;
          const int k0 = kbr * BK;
          const int part = p.a_parts > 1 ? k0 / p.a_part_k : 0;
          const int ka = p.a_parts > 1 ? k0 - part * p.a_part_k : k0;     // column inside the piece
          const CUtensorMap* tmap_a = &tmaps_a.m[part];
          if constexpr (!A_MN) {
            tma_load_3d(sa, tmap_a, full_bar + stage, ka, m0, bz);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_3d(sa + j * 8192, tmap_a, full_bar + stage, m0 + 64 * j, ka, bz);
          }
          if constexpr (!B_MN) {
            tma_load_3d(sb, &tmap_b, full_bar + stage, k0, n0, bz);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_3d(sb + j * 8192, &tmap_b, full_bar + stage, n0 + 64 * j, k0, bz);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) { *abort_flag = 1; atomicExch(p.err, 1); }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc = make_idesc_f16(BM, BN, in_fmt, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const TileCoord tc = decode_tile<BN>(tile, num_m, tiles_per_batch);
        const int m0 = tc.m0, n0 = tc.n0;
        if (tile_skipped<BN>(p, m0, n0)) continue;
        int kb0, kb1;
        k_range(p, m0, num_k, kb0, kb1);
        if (!wait_or_abort(tmem_empty + acc, acc_phase ^ 1, abort_flag)) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!wait_or_abort(full_bar + stage, phase, abort_flag)) { ok = false; break; }
          tcgen05_fence_after();
          const uint32_t sa = smem_u32(smem + stage * L::stage_bytes);
          const uint32_t sb = sa + L::a_bytes;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t da = A_MN ? make_smem_desc(sa + kk * 2048, 8192, 1024)
                                     : make_smem_desc(sa + kk * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc(sb + kk * 2048, 8192, 1024)
                                     : make_smem_desc(sb + kk * 32, 16, 1024);
            umma_f16(d_tmem, da, db, idesc, (kb != kb0 || kk != 0) ? 1u : 0u);
          }
          umma_commit(empty_bar + stage);      // stage reusable once these MMAs have read it
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(tmem_full + acc);          // accumulator complete
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
      if (!ok) { *abort_flag = 1; atomicExch(p.err, 2); }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;              // TMEM lanes [32 * quarter, +32) belong to this warp
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    OutT* C = reinterpret_cast<OutT*>(p.C);
    OutT* P = reinterpret_cast<OutT*>(p.preact);
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const TileCoord tc = decode_tile<BN>(tile, num_m, tiles_per_batch);
      const int m0 = tc.m0, n0 = tc.n0;
      if (tile_skipped<BN>(p, m0, n0)) continue;
      if (!wait_or_abort(tmem_full + acc, acc_phase, abort_flag)) { ok = false; break; }
      tcgen05_fence_after();
      const int row = m0 + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + acc * BN + ((uint32_t)(quarter * 32) << 16);
      const long long ridx = (long long)tc.bz * p.M + row;
      EpiRow er;
      if (p.epi != kEpiStd) epi_row_begin(p, ridx, row < p.M, er);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) continue;            // warp-uniform
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
        const int nvalid = min(32, p.N - col0);
        if (p.epi != kEpiStd) {
          if (row < p.M)
            epi_chunk<OutT>(p, v, row, col0, nvalid, (long long)tc.bz * p.c_batch_stride + (long long)row * p.ldc + col0,
                            C, er);
          continue;
        }
        if (p.bias != nullptr) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (i < nvalid) {
              float bv;
              if (p.bias_dtype == kF32) bv = reinterpret_cast<const float*>(p.bias)[col0 + i];
              else if (p.bias_dtype == kBF16) bv = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[col0 + i]);
              else bv = __half2float(reinterpret_cast<const __half*>(p.bias)[col0 + i]);
              v[i] += bv;
            }
          }
        }
        if (row < p.M) {
          if (p.c_nparts > 1) {
            // push this 32-column chunk into the slot of the rank that owns these columns
            const int owner = col0 / p.c_part_cols;
            OutT* slot = reinterpret_cast<OutT*>(p.c_parts[owner]);
            store_row32<OutT>(slot + (long long)row * p.c_part_cols + (col0 - owner * p.c_part_cols), v, nvalid);
          } else {
            const long long off = (long long)tc.bz * p.c_batch_stride + (long long)row * p.ldc + col0;
            if (p.accumulate) add_row32<OutT>(C + off, v, nvalid);
            if (p.aux != nullptr) add_row32<OutT>(reinterpret_cast<const OutT*>(p.aux) + off, v, nvalid);   // + addend
            if (P != nullptr) store_row32<OutT>(P + off, v, nvalid);
            if (p.act == 1) {
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = silu_f(v[i]);
            }
            store_row32<OutT>(C + off, v, nvalid);
          }
        }
      }
      if (p.epi != kEpiStd) epi_row_end(p, ridx, row < p.M, er);
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty + acc);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    if (!ok && lane == 0) { *abort_flag = 1; atomicExch(p.err, 3); }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------- CTA-pair variant
// Same roles and pipeline, but two CTAs of a 2-CTA cluster share one 256 x 256 output tile through
// tcgen05.mma.cta_group::2: CTA r stages rows [m0 + 128 r, +128) of A and rows [n0 + 128 r, +128) of
// B, so each SM streams 32 KiB per k-block instead of 48 KiB and the ring is 6 stages deep.  The even
// CTA issues the MMAs; every "stage consumed" and "accumulator ready" signal is committed once to
// each CTA's barrier, and both CTAs' epilogue warps release the accumulator on the even CTA's barrier.
constexpr int kPairStages = 6;
constexpr int kPairBM = 256;      // rows of the pair's tile
constexpr int kPairBN = 256;

struct PairSmem {
  static constexpr int a_bytes = BM * BK * 2;                 // this CTA's 128 rows of A
  static constexpr int b_bytes = (kPairBN / 2) * BK * 2;      // this CTA's 128 rows of B
  static constexpr int stage_bytes = a_bytes + b_bytes;       // 32 KiB
  static constexpr int bar_offset = kPairStages * stage_bytes;
  // one staging buffer per epilogue warp: 32 rows x 128 bytes (64 columns of a 16-bit output)
  static constexpr int epi_stage_bytes = 32 * 128;
  static constexpr int epi_offset = bar_offset + 256;
  static constexpr int total = epi_offset + kEpiWarps * epi_stage_bytes + 1024;
};

__device__ __forceinline__ bool pair_tile_skipped(const GemmParams& p, int m0, int n0) {
  return p.mode == 1 && n0 > m0 + kPairBM - 1;
}

__device__ __forceinline__ void pair_k_range(const GemmParams& p, int m0, int num_k, int& kb0, int& kb1) {
  kb0 = 0;
  kb1 = num_k;
  if (p.mode == 2) kb1 = min(num_k, (m0 + kPairBM + BK - 1) / BK);
  if (p.mode == 3) kb0 = min(num_k - 1, m0 / BK);
}

constexpr int kGatherWarps = 4;                 // copy warps of the gathering variant
constexpr int kGatherUnitBytes = 8192;          // one claim: 32 lanes x 16 loads of 16 bytes

// Tiles of one batch element that the kernel computes: with mode 1 (causal scores) only those on or below
// the diagonal.
__device__ __forceinline__ int pair_tiles_per_batch(const GemmParams& p, int num_m, int num_n) {
  if (p.mode != 1) return num_m * num_n;
  int t = 0;
  for (int mt = 0; mt < num_m; ++mt) t += min(mt + 1, num_n);
  return t;
}

// Tile -> (m0, n0, batch).  With a gathered B the n-tiles are walked starting at this rank's own rows,
// whose chunks are copied first.  The causal modes hand every CTA pair tiles `pair, pair + P, ...` of an
// ORDER chosen for balance: mode 1 numbers only the tiles it computes (the plain order left a pair with up
// to 10 of them against a mean of 7.4); modes 2 and 3, whose k loop grows with the distance from the
// diagonal, order all tiles of all batch elements from the longest k loop to the shortest and deal them
// out in alternating direction (the plain order: 0.84 of the mean on the busiest pair, this one 0.97).
__device__ __forceinline__ void pair_tile_coords(const GemmParams& p, int tile, int num_m, int num_n,
                                                 int tiles_per_batch, int num_pairs, int& m0, int& n0, int& bz) {
  if (p.mode >= 1 && p.mode <= 3 && p.g_world == 0) {
    const int num_tiles = tiles_per_batch * p.batch;
    const int round = tile / num_pairs;
    int pos = tile - round * num_pairs;
    if (round & 1) pos = min(num_pairs, num_tiles - round * num_pairs) - 1 - pos;
    const int i = round * num_pairs + pos;
    int mt, nt;
    if (p.mode == 1) {
      bz = i / tiles_per_batch;
      int t = i - bz * tiles_per_batch;
      mt = 0;
      while (t >= min(mt + 1, num_n)) {
        t -= min(mt + 1, num_n);
        ++mt;
      }
      nt = t;
    } else {
      const int per_m = num_n * p.batch;
      const int q = i / per_m, rem = i - q * per_m;
      mt = p.mode == 2 ? num_m - 1 - q : q;       // longest k loop first
      bz = rem / num_n;
      nt = rem - bz * num_n;
    }
    m0 = mt * kPairBM;
    n0 = nt * kPairBN;
    return;
  }
  bz = tile / tiles_per_batch;
  const int t = tile - bz * tiles_per_batch;
  int nt = t / num_m;
  if (p.g_world > 0) {
    nt += (int)(((long long)p.g_rank * (p.N / p.g_world)) / kPairBN);
    if (nt >= num_n) nt -= num_n;
  }
  m0 = (t % num_m) * kPairBM;
  n0 = nt * kPairBN;
}

__device__ __forceinline__ unsigned int ld_acquire_gpu_u32(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Bounded wait until chunk `chunk` of the gathered matrix is complete in local memory.
__device__ __forceinline__ bool wait_chunk(const GemmParams& p, int chunk, volatile int* abort_flag) {
  const unsigned int need = (unsigned int)(p.K / 32);
  const unsigned int* flag = p.g_flags + 1 + chunk;
  if (ld_acquire_gpu_u32(flag) < need) {
    const unsigned long long t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (ld_acquire_gpu_u32(flag) < need) {
      if ((++spins & 0x3f) == 0) {
        if (*abort_flag) return false;
        if (globaltimer_ns() - t0 > kWaitTimeoutNs) return false;
      }
      __nanosleep(64);
    }
  }
  fence_proxy_async_all();        // the copy warps wrote through the generic proxy, TMA reads through the async one
  return true;
}

// Body of one copy warp: claim 8 KiB units until none is left.  Never waits for anything.
__device__ __forceinline__ void gather_copy_warp(const GemmParams& p, int lane) {
  const int nchunks = p.N / 128;
  const int upc = p.K / 32;                              // 8 KiB units per 128-row chunk (K * 256 B / 8192)
  const int total = nchunks * upc;
  const int rows_per_rank = p.N / p.g_world;
  const int first_chunk = (int)(((long long)p.g_rank * rows_per_rank) / 128);
  while (true) {
    unsigned int u = 0;
    if (lane == 0) u = atomicAdd(p.g_flags, 1u);
    u = __shfl_sync(0xffffffffu, u, 0);
    if (u >= (unsigned int)total) break;
    const int oc = (int)u / upc, sub = (int)u - oc * upc;
    int chunk = oc + first_chunk;
    if (chunk >= nchunks) chunk -= nchunks;
    const int row0 = chunk * 128;
    const int owner = row0 / rows_per_rank;
    const long long src_byte = (long long)(row0 - owner * rows_per_rank) * p.K * 2 + (long long)sub * kGatherUnitBytes;
    const long long dst_byte = (long long)row0 * p.K * 2 + (long long)sub * kGatherUnitBytes;
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(p.g_src[owner]) + src_byte);
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<char*>(p.g_dst) + dst_byte);
    uint4 v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __ldcv(src + lane + 32 * i);
#pragma unroll
    for (int i = 0; i < 16; ++i) dst[lane + 32 * i] = v[i];
    fence_proxy_async_all();
    __threadfence();
    __syncwarp();
    if (lane == 0) atomicAdd(p.g_flags + 1 + chunk, 1u);
  }
}

// ---- staged epilogue of the pair kernel (16-bit outputs).  A thread owns one row of the accumulator, so
// writing its 32 columns straight to global memory makes every warp store touch 32 different lines, 16
// bytes each: the load/store unit, not DRAM, bounds products with short k loops (attention scores: 77 %
// of the L1 data path busy, tensor pipe 12 %).  Instead the warp collects 64 columns (128 bytes per row)
// in shared memory and moves them with 8 instructions that each cover 4 whole rows; inputs of the
// epilogue (the accumulated C, an addend, the stored probabilities of the dS epilogue) come in the same
// way.  Pieces of 16 bytes are XOR-swizzled by the row, which makes both directions conflict-free.
__device__ __forceinline__ uint32_t epi_stage_addr(uint32_t base, int row, int piece) {
  return base + row * 128 + ((piece ^ (row & 7)) << 4);
}
__device__ __forceinline__ void lds128(uint32_t addr, uint4& v) {
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
}
__device__ __forceinline__ void sts128(uint32_t addr, const uint4& v) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
template <typename OutT>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 t = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}
template <>
__device__ __forceinline__ uint32_t pack2<float>(float a, float) { return __float_as_uint(a); }   // never used
template <typename OutT>
__device__ __forceinline__ void unpack2(uint32_t w, float& a, float& b);
template <>
__device__ __forceinline__ void unpack2<__nv_bfloat16>(uint32_t w, float& a, float& b) {
  a = __uint_as_float(w << 16);
  b = __uint_as_float(w & 0xffff0000u);
}
template <>
__device__ __forceinline__ void unpack2<__half>(uint32_t w, float& a, float& b) {
  const __half2 t = *reinterpret_cast<__half2*>(&w);
  a = __low2float(t);
  b = __high2float(t);
}
template <>
__device__ __forceinline__ void unpack2<float>(uint32_t w, float& a, float& b) { a = b = __uint_as_float(w); }
// global [32 rows x 64 columns] <-> the warp's staging buffer; rows >= rows_valid are skipped
template <typename OutT>
__device__ __forceinline__ void epi_stage_in(uint32_t stg, const OutT* src, long long ld, int rows_valid, int lane) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int r = 4 * j + (lane >> 3), q = lane & 7;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < rows_valid) v = *reinterpret_cast<const uint4*>(src + (long long)r * ld + q * 8);
    sts128(epi_stage_addr(stg, r, q), v);
  }
}
template <typename OutT>
__device__ __forceinline__ void epi_stage_out(uint32_t stg, OutT* dst, long long ld, int rows_valid, int lane) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int r = 4 * j + (lane >> 3), q = lane & 7;
    uint4 v;
    lds128(epi_stage_addr(stg, r, q), v);
    if (r < rows_valid) *reinterpret_cast<uint4*>(dst + (long long)r * ld + q * 8) = v;
  }
}
// the thread's own row: 32 columns (half h of the 64) as floats
template <typename OutT>
__device__ __forceinline__ void epi_stage_get(uint32_t stg, int lane, int h, float (&v)[32]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 w;
    lds128(epi_stage_addr(stg, lane, h * 4 + i), w);
    unpack2<OutT>(w.x, v[8 * i + 0], v[8 * i + 1]);
    unpack2<OutT>(w.y, v[8 * i + 2], v[8 * i + 3]);
    unpack2<OutT>(w.z, v[8 * i + 4], v[8 * i + 5]);
    unpack2<OutT>(w.w, v[8 * i + 6], v[8 * i + 7]);
  }
}
template <typename OutT>
__device__ __forceinline__ void epi_stage_put(uint32_t stg, int lane, int h, const float (&v)[32]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 w;
    w.x = pack2<OutT>(v[8 * i + 0], v[8 * i + 1]);
    w.y = pack2<OutT>(v[8 * i + 2], v[8 * i + 3]);
    w.z = pack2<OutT>(v[8 * i + 4], v[8 * i + 5]);
    w.w = pack2<OutT>(v[8 * i + 6], v[8 * i + 7]);
    sts128(epi_stage_addr(stg, lane, h * 4 + i), w);
  }
}
// Per-row constants of the fused epilogues, folded so that an element costs one FMA plus the operation
// itself: exp(alpha s - m) = 2^(s * alpha log2e - m log2e); dS = p~ (s * alpha / l - delta / l).
struct EpiFold {
  float k1, k2;
};
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 32 columns of the thread's row: raw accumulator `r` -> values to store in `v`.  MASKED: the tile touches
// the diagonal and columns beyond `last` give zero (and take no part in maxima / sums); tiles below the
// diagonal skip the comparison.  The row sum of kEpiExp adds the values before they are rounded to the
// output type.
template <typename OutT, bool MASKED>
__device__ __forceinline__ void epi_compute(const GemmParams& p, const uint32_t (&r)[32], const float (&pt)[32],
                                            float (&v)[32], int last, int col0, const EpiFold& f, EpiRow& er) {
  if (p.epi == kEpiRowMax) {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (!MASKED || col0 + i <= last) er.acc = fmaxf(er.acc, __uint_as_float(r[i]));     // raw: scaled by alpha at the end
  } else if (p.epi == kEpiExp) {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      float e = ex2_approx(fmaf(__uint_as_float(r[i]), f.k1, -f.k2));
      if (MASKED && col0 + i > last) e = 0.f;
      er.acc += e;
      v[i] = e;
    }
  } else if (p.epi == kEpiRowScale) {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * f.k1;
  } else {   // kEpiDS
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float d = pt[i] * fmaf(__uint_as_float(r[i]), f.k1, -f.k2);
      v[i] = (MASKED && col0 + i > last) ? 0.f : d;
    }
  }
}

template <bool A_MN, bool B_MN, typename OutT, bool GATHER = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads + (GATHER ? kGatherWarps * 32 : 0), 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ TmapArray tmaps_a, const __grid_constant__ CUtensorMap tmap_b,
                         const __grid_constant__ GemmParams p, int in_fmt) {
  using L = PairSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::bar_offset);     // used in the even CTA only
  uint64_t* empty_bar = full_bar + kPairStages;                               // one set per CTA
  uint64_t* tmem_full = empty_bar + kPairStages;                              // one set per CTA
  uint64_t* tmem_empty = tmem_full + 2;                                       // used in the even CTA only
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0 = even CTA (issues the MMAs), 1 = its peer
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int num_m = (p.M + kPairBM - 1) / kPairBM;
  const int num_n = (p.N + kPairBN - 1) / kPairBN;
  const int tiles_per_batch = pair_tiles_per_batch(p, num_m, num_n);
  const int num_tiles = tiles_per_batch * p.batch;
  const int num_k = (p.K + BK - 1) / BK;
  constexpr uint32_t kTmemCols = 2 * kPairBN;       // two accumulators of 256 columns

  if (threadIdx.x == 0) {
    for (int i = 0; i < kPairStages; ++i) {
      mbar_init(full_bar + i, 2);                   // one arrive.expect_tx from each CTA's producer
      mbar_init(empty_bar + i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(tmem_full + i, 1);
      mbar_init(tmem_empty + i, 2 * kEpiWarps);     // epilogue warps of both CTAs
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_holder, kTmemCols);
    tmem_relinquish_pair();
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();                               // the peer's barriers exist before anything signals them
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (elect_one()) {
      for (int i = 0; i < p.a_parts; ++i) prefetch_tmap(&tmaps_a.m[i]);
      prefetch_tmap(&tmap_b);
      const int kb_shift = p.a_parts > 1 ? p.a_first * (p.a_part_k / BK) : 0;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        int m0, n0, bz;
        pair_tile_coords(p, tile, num_m, num_n, tiles_per_batch, num_pairs, m0, n0, bz);
        if (pair_tile_skipped(p, m0, n0)) continue;
        const int my_m = m0 + (int)rank * BM;
        const int my_n = n0 + (int)rank * (kPairBN / 2);
        int kb0, kb1;
        pair_k_range(p, m0, num_k, kb0, kb1);
        if constexpr (GATHER) {
          // this CTA's 128 rows of B are exactly one chunk of the gathered matrix
          if (my_n < p.N && !wait_chunk(p, my_n / 128, abort_flag)) { ok = false; break; }
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!wait_or_abort(empty_bar + stage, phase ^ 1, abort_flag)) { ok = false; break; }
          uint8_t* sa = smem + stage * L::stage_bytes;
          uint8_t* sb = sa + L::a_bytes;
          const uint32_t full0 = map_to_cta(smem_u32(full_bar + stage), 0);
          mbar_expect_tx_cluster(full0, L::stage_bytes);
          const int kbr = p.a_parts > 1 ? (kb + kb_shift) % num_k : kb;
          const int k0 = kbr * BK;
          const int part = p.a_parts > 1 ? k0 / p.a_part_k : 0;
          const int ka = p.a_parts > 1 ? k0 - part * p.a_part_k : k0;
          const CUtensorMap* tmap_a = &tmaps_a.m[part];
          if constexpr (!A_MN) {
            tma_load_3d_pair(sa, tmap_a, full0, ka, my_m, bz);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_3d_pair(sa + j * 8192, tmap_a, full0, my_m + 64 * j, ka, bz);
          }
          if constexpr (!B_MN) {
            tma_load_3d_pair(sb, &tmap_b, full0, k0, my_n, bz);
          } else {
#pragma unroll
            for (int j = 0; j < kPairBN / 128; ++j)
              tma_load_3d_pair(sb + j * 8192, &tmap_b, full0, my_n + 64 * j, k0, bz);
          }
          if (++stage == kPairStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) { *abort_flag = 1; atomicExch(p.err, 1); }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (even CTA only)
    if (rank == 0 && elect_one()) {
      const uint32_t idesc = make_idesc_f16(kPairBM, kPairBN, in_fmt, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        int m0, n0, bz;
        pair_tile_coords(p, tile, num_m, num_n, tiles_per_batch, num_pairs, m0, n0, bz);
        if (pair_tile_skipped(p, m0, n0)) continue;
        int kb0, kb1;
        pair_k_range(p, m0, num_k, kb0, kb1);
        if (!wait_or_abort(tmem_empty + acc, acc_phase ^ 1, abort_flag)) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kPairBN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!wait_or_abort(full_bar + stage, phase, abort_flag)) { ok = false; break; }
          tcgen05_fence_after();
          const uint32_t sa = smem_u32(smem + stage * L::stage_bytes);
          const uint32_t sb = sa + L::a_bytes;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t da = A_MN ? make_smem_desc(sa + kk * 2048, 8192, 1024)
                                     : make_smem_desc(sa + kk * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc(sb + kk * 2048, 8192, 1024)
                                     : make_smem_desc(sb + kk * 32, 16, 1024);
            umma_f16_pair(d_tmem, da, db, idesc, (kb != kb0 || kk != 0) ? 1u : 0u);
          }
          // the stage is reusable in both CTAs once these MMAs have read it
          const uint32_t e = smem_u32(empty_bar + stage);
          umma_commit_pair(e);
          umma_commit_pair(map_to_cta(e, 1));
          if (++stage == kPairStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        const uint32_t f = smem_u32(tmem_full + acc);
        umma_commit_pair(f);
        umma_commit_pair(map_to_cta(f, 1));
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
      if (!ok) { *abort_flag = 1; atomicExch(p.err, 2); }
    }
  } else if (GATHER && warp >= kGemmThreads / 32) {
    // ------------------------------------------------------------ copy warps (gathering variant)
    gather_copy_warp(p, lane);
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int quarter = warp & 3;
    const uint32_t stage_buf = smem_u32(smem + L::epi_offset + quarter * L::epi_stage_bytes);
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    OutT* C = reinterpret_cast<OutT*>(p.C);
    OutT* P = reinterpret_cast<OutT*>(p.preact);
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      int m0, n0, bz;
      pair_tile_coords(p, tile, num_m, num_n, tiles_per_batch, num_pairs, m0, n0, bz);
      if (pair_tile_skipped(p, m0, n0)) continue;
      if (!wait_or_abort(tmem_full + acc, acc_phase, abort_flag)) { ok = false; break; }
      tcgen05_fence_after();
      const int row = m0 + (int)rank * BM + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + acc * kPairBN + ((uint32_t)(quarter * 32) << 16);
      const long long ridx = (long long)bz * p.M + row;
      EpiRow er;
      if (p.epi != kEpiStd) epi_row_begin(p, ridx, row < p.M, er);
      // chunk c (32 columns) written straight from the registers: partial groups, fp32 outputs, split C
      auto direct_chunk = [&](int c) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) return;              // warp-uniform
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
        const int nvalid = min(32, p.N - col0);
        if (p.epi != kEpiStd) {
          if (row < p.M)
            epi_chunk<OutT>(p, v, row, col0, nvalid, (long long)bz * p.c_batch_stride + (long long)row * p.ldc + col0,
                            C, er);
          return;
        }
        if (p.bias != nullptr) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (i < nvalid) {
              float bv;
              if (p.bias_dtype == kF32) bv = reinterpret_cast<const float*>(p.bias)[col0 + i];
              else if (p.bias_dtype == kBF16) bv = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[col0 + i]);
              else bv = __half2float(reinterpret_cast<const __half*>(p.bias)[col0 + i]);
              v[i] += bv;
            }
          }
        }
        if (row < p.M) {
          if (p.c_nparts > 1) {
            const int owner = col0 / p.c_part_cols;
            OutT* slot = reinterpret_cast<OutT*>(p.c_parts[owner]);
            store_row32<OutT>(slot + (long long)row * p.c_part_cols + (col0 - owner * p.c_part_cols), v, nvalid);
          } else {
            const long long off = (long long)bz * p.c_batch_stride + (long long)row * p.ldc + col0;
            if (p.accumulate) add_row32<OutT>(C + off, v, nvalid);
            if (p.aux != nullptr) add_row32<OutT>(reinterpret_cast<const OutT*>(p.aux) + off, v, nvalid);   // + addend
            if (P != nullptr) store_row32<OutT>(P + off, v, nvalid);
            if (p.act == 1) {
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = silu_f(v[i]);
            }
            store_row32<OutT>(C + off, v, nvalid);
          }
        }
            };
      const int row_base = m0 + (int)rank * BM + quarter * 32;
      const int rows_valid = p.M - row_base;
      const bool std_in = p.epi == kEpiStd && (p.accumulate || p.aux != nullptr);
      // groups of 64 columns: both 32-column reads of tensor memory are issued before the wait, the
      // results pass through the warp's staging buffer and leave as whole 128-byte row segments
      const bool can_group = sizeof(OutT) == 2 && P == nullptr && p.c_nparts <= 1 &&
                             !(p.epi == kEpiStd && p.accumulate && p.aux != nullptr) &&
                             ((p.ldc | p.c_batch_stride) & 7) == 0 &&
                             ((reinterpret_cast<uintptr_t>(C) | reinterpret_cast<uintptr_t>(p.aux)) & 15) == 0 &&
                             n0 + kPairBN <= p.N && !(p.epi == kEpiRowMax && p.alpha < 0.f);
      // (the gathering variant, whose 320 threads leave fewer registers each, keeps the direct form: a
      // register spilled between an asynchronous tensor-memory read and its wait would be read too early)
      if (GATHER || !can_group) {
#pragma unroll 1
        for (int c = 0; c < kPairBN / 32; ++c) direct_chunk(c);
      } else if constexpr (!GATHER) {
        const bool need_in = p.epi == kEpiDS || std_in;
        const OutT* src = (p.epi == kEpiDS || !p.accumulate) ? reinterpret_cast<const OutT*>(p.aux) : C;
        const long long off_row0 = (long long)bz * p.c_batch_stride + (long long)row_base * p.ldc + n0;
        const int last = p.mode == 1 ? row + p.causal_off : 0x7fffffff;
        // does any row of this warp end inside the tile?  (warp-uniform)
        const bool masked = p.mode == 1 && n0 + kPairBN - 1 > row_base + p.causal_off;
        EpiFold fold{p.alpha, 0.f};
        if (p.epi == kEpiExp) fold = {p.alpha * 1.4426950408889634f, er.a * 1.4426950408889634f};
        else if (p.epi == kEpiRowScale) fold = {p.alpha * er.a, 0.f};
        else if (p.epi == kEpiDS) fold = {p.alpha * er.a, er.a * er.b};
#pragma unroll 1
        for (int g = 0; g < kPairBN / 64; ++g) {
          const int colg = n0 + g * 64;
          const long long off0 = off_row0 + g * 64;
          uint32_t ra[32], rb[32];
          tmem_ld_32x32(t_row + g * 64, ra);
          tmem_ld_32x32(t_row + g * 64 + 32, rb);
          if (need_in) epi_stage_in<OutT>(stage_buf, src + off0, p.ldc, rows_valid, lane);
          tmem_ld_wait();
          if (need_in) __syncwarp();
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int col0 = colg + h * 32;
            const uint32_t (&rr)[32] = h == 0 ? ra : rb;
            float v[32], pt[32];
            if (need_in) epi_stage_get<OutT>(stage_buf, lane, h, pt);
            if (p.epi != kEpiStd) {
              if (masked) epi_compute<OutT, true>(p, rr, pt, v, last, col0, fold, er);
              else epi_compute<OutT, false>(p, rr, pt, v, last, col0, fold, er);
              if (p.epi == kEpiRowMax) continue;
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(rr[i]) * p.alpha;
              if (p.bias != nullptr) {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                  float bv;
                  if (p.bias_dtype == kF32) bv = reinterpret_cast<const float*>(p.bias)[col0 + i];
                  else if (p.bias_dtype == kBF16) bv = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[col0 + i]);
                  else bv = __half2float(reinterpret_cast<const __half*>(p.bias)[col0 + i]);
                  v[i] += bv;
                }
              }
              if (need_in) {
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] += pt[i];
              }
              if (p.act == 1) {
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = silu_f(v[i]);
              }
            }
            epi_stage_put<OutT>(stage_buf, lane, h, v);
          }
          if (p.epi != kEpiRowMax) {
            __syncwarp();
            epi_stage_out<OutT>(stage_buf, C + off0, p.ldc, rows_valid, lane);
            __syncwarp();
          }
        }
        if (p.epi == kEpiRowMax) {
          // the maximum was taken over raw accumulators: alpha >= 0 on this path, so it scales through
          er.acc = er.acc > -INFINITY ? er.acc * p.alpha : er.acc;
        }
      }
      if (p.epi != kEpiStd) epi_row_end(p, ridx, row < p.M, er);
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(tmem_empty + acc), 0));
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    if (!ok && lane == 0) { *abort_flag = 1; atomicExch(p.err, 3); }
  }

  // Neither CTA may leave (or free tensor memory) while the other can still signal its barriers,
  // read its shared memory or write its accumulator.
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

}  // namespace

// 2-D bf16/fp16 tensor map: `inner` contiguous elements per row, `outer` rows, 128-byte swizzle.
// 3-D bf16/fp16 tensor map [batch, outer, inner] (inner contiguous) with a {1, box_outer, box_inner} box
// and 128-byte swizzle.  Strides are in elements and must be multiples of 8 (16 bytes).
bool make_tmap_3d(CUtensorMap* out, const void* base, long long inner, long long outer, long long batch,
                  long long row_stride, long long batch_stride, int box_inner, int box_outer, int elem_dtype) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return false;
  // The encoder is a driver entry point and needs a current context; a thread that has made no
  // runtime call yet (the autograd engine's worker on its first backward) has none bound.
  static thread_local bool context_bound = false;
  if (!context_bound) {
    cudaFree(nullptr);
    context_bound = true;
  }
  if (batch <= 1) batch_stride = row_stride * outer;      // unused, but must be a valid stride
  const cuuint64_t dims[3] = {(cuuint64_t)inner, (cuuint64_t)outer, (cuuint64_t)(batch < 1 ? 1 : batch)};
  const cuuint64_t strides[2] = {(cuuint64_t)row_stride * 2, (cuuint64_t)batch_stride * 2};
  const cuuint32_t box[3] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapDataType dt = elem_dtype == kBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUresult res = fn(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (res != CUDA_SUCCESS)
    fprintf(stderr,
            "tensor map encode failed (CUresult %d): base %p dims {%llu, %llu, %llu} strides {%llu, %llu} B box {%u, %u}\n",
            (int)res, base, (unsigned long long)dims[0], (unsigned long long)dims[1], (unsigned long long)dims[2],
            (unsigned long long)strides[0], (unsigned long long)strides[1], box[0], box[1]);
  return res == CUDA_SUCCESS;
}

template <int BN, bool A_MN, bool B_MN, typename OutT>
static int launch_gemm(const TmapArray& ta, const CUtensorMap& tb, const GemmParams& p, int in_fmt, int sms,
                       cudaStream_t st) {
  using L = SmemLayout<BN>;
  auto kern = gemm_tcgen05_kernel<BN, A_MN, B_MN, OutT>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::total) != cudaSuccess) return -2;
    configured = true;
  }
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN) * p.batch;
  const int grid = tiles < sms ? tiles : sms;
  kern<<<grid, kGemmThreads, L::total, st>>>(ta, tb, p, in_fmt);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// Pair kernel with copy warps that gather the K-major weight operand from its owners while the tensor
// cores work (see GemmParams::g_*).  The claim counter and the chunk flags are cleared on the stream first.
template <typename OutT>
static int launch_gemm_pair_gather(const TmapArray& ta, const CUtensorMap& tb, const GemmParams& p, int in_fmt,
                                   int sms, cudaStream_t st) {
  using L = PairSmem;
  auto kern = gemm_tcgen05_pair_kernel<false, false, OutT, true>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::total) != cudaSuccess) return -2;
    configured = true;
  }
  if (cudaMemsetAsync(p.g_flags, 0, sizeof(unsigned int) * (1 + p.N / 128), st) != cudaSuccess) return -8;
  const int tiles = ((p.M + kPairBM - 1) / kPairBM) * ((p.N + kPairBN - 1) / kPairBN) * p.batch;
  const int pairs = sms / 2;
  const int grid = 2 * (tiles < pairs ? tiles : pairs);
  kern<<<grid, kGemmThreads + kGatherWarps * 32, L::total, st>>>(ta, tb, p, in_fmt);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

template <bool A_MN, bool B_MN, typename OutT>
static int launch_gemm_pair(const TmapArray& ta, const CUtensorMap& tb, const GemmParams& p, int in_fmt, int sms,
                            cudaStream_t st) {
  using L = PairSmem;
  auto kern = gemm_tcgen05_pair_kernel<A_MN, B_MN, OutT>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::total) != cudaSuccess) return -2;
    configured = true;
  }
  const int tiles = ((p.M + kPairBM - 1) / kPairBM) * ((p.N + kPairBN - 1) / kPairBN) * p.batch;
  const int pairs = sms / 2;
  const int grid = 2 * (tiles < pairs ? tiles : pairs);
  kern<<<grid, kGemmThreads, L::total, st>>>(ta, tb, p, in_fmt);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

static bool g_use_pair = true;

// Returns 0 on success, negative on a host-side failure.  `err` is a device int
// that the kernel sets non-zero if one of its bounded waits gives up.
int gemm_bf16_tcgen05(const void* A, const void* B, void* C, void* preact, const void* bias, int bias_dtype,
                      int act, int M, int N, int K, long long lda, long long ldb, long long ldc, bool a_mn,
                      bool b_mn, int mode, float alpha, int batch, long long a_bs, long long b_bs, long long c_bs,
                      int in_dtype, int out_dtype, int* err, int num_sms, cudaStream_t st,
                      const GemmPeerSpec* peers, bool accumulate, const GemmGatherSpec* gather,
                      const GemmSoftmaxSpec* softmax) {
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return 0;
  // TMA wants 16-byte strides; the vectorised epilogue wants 16-byte aligned rows of C
  if (lda % 8 != 0 || ldb % 8 != 0 || ldc % 8 != 0) return -1;
  if (batch > 1 && (a_bs % 8 != 0 || b_bs % 8 != 0 || c_bs % 8 != 0)) return -1;
  const int BN = 256;
  TmapArray ta;
  CUtensorMap tb;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.C = C; p.preact = preact; p.bias = bias; p.bias_dtype = bias_dtype; p.act = act;
  p.err = err; p.ldc = ldc; p.mode = mode; p.alpha = alpha; p.batch = batch; p.c_batch_stride = c_bs;
  p.a_parts = 1; p.a_part_k = K; p.a_first = 0; p.c_nparts = 1; p.c_part_cols = N;
  p.accumulate = accumulate ? 1 : 0;
  if (softmax != nullptr && softmax->kind == 0 && softmax->aux != nullptr) {
    if (peers != nullptr && peers->c_nparts > 1) return -10;
    p.aux = softmax->aux;              // standard epilogue with an addend of C's layout
  }
  if (softmax != nullptr && softmax->kind != 0) {
    if (softmax->kind < 1 || softmax->kind > 4 || bias != nullptr || act != 0 || preact != nullptr || accumulate ||
        peers != nullptr)
      return -10;
    p.epi = softmax->kind; p.row_in = softmax->row_in; p.row_in2 = softmax->row_in2; p.row_out = softmax->row_out;
    p.aux = softmax->aux; p.causal_off = softmax->causal_off;
  }
  bool ok = true;
  if (peers != nullptr && peers->a_parts > 1) {
    // gathered A: K-major pieces [M, K / parts] living on different GPUs
    if (a_mn || batch != 1 || peers->a_parts > kMaxPeers || K % peers->a_parts != 0) return -6;
    p.a_parts = peers->a_parts;
    p.a_part_k = K / peers->a_parts;
    p.a_first = peers->a_first;
    if (p.a_part_k % BK != 0) return -6;
    for (int i = 0; i < p.a_parts; ++i)
      ok = ok && make_tmap_3d(&ta.m[i], peers->a_ptrs[i], p.a_part_k, M, 1, lda, 0, BK, BM, in_dtype);
  } else {
    ok = a_mn ? make_tmap_3d(&ta.m[0], A, M, K, batch, lda, a_bs, 64, 64, in_dtype)
              : make_tmap_3d(&ta.m[0], A, K, M, batch, lda, a_bs, BK, BM, in_dtype);
  }
  if (peers != nullptr && peers->c_nparts > 1) {
    if (batch != 1 || peers->c_nparts > kMaxPeers || N % peers->c_nparts != 0) return -7;
    p.c_nparts = peers->c_nparts;
    p.c_part_cols = N / peers->c_nparts;
    if (p.c_part_cols % 32 != 0) return -7;
    for (int i = 0; i < p.c_nparts; ++i) p.c_parts[i] = peers->c_ptrs[i];
  }
  const bool pair = g_use_pair && M > BM && num_sms >= 2;
  if (!ok) return -41;
  if (gather != nullptr && gather->world > 0) {
    // B must be the whole K-major weight, contiguous, its row blocks whole 128-row chunks
    if (!gemm_gather_supported(M, N, K, gather->world) || !pair || a_mn || b_mn || batch != 1 || mode != 0 ||
        p.a_parts != 1 || ldb != K || gather->world > kMaxPeers || gather->flags == nullptr || B != gather->dst)
      return -9;
    p.g_world = gather->world; p.g_rank = gather->rank; p.g_dst = gather->dst; p.g_flags = gather->flags;
    for (int i = 0; i < gather->world; ++i) p.g_src[i] = gather->src[i];
  }
  ok = ok && (b_mn ? make_tmap_3d(&tb, B, N, K, batch, ldb, b_bs, 64, 64, in_dtype)
                   : make_tmap_3d(&tb, B, K, N, batch, ldb, b_bs, BK, pair ? kPairBN / 2 : BN, in_dtype));
  if (!ok) return -4;
  const int fmt = in_dtype == kBF16 ? 1 : 0;
  if (p.g_world > 0) {
    if (out_dtype == kBF16) return launch_gemm_pair_gather<__nv_bfloat16>(ta, tb, p, fmt, num_sms, st);
    if (out_dtype == kF16) return launch_gemm_pair_gather<__half>(ta, tb, p, fmt, num_sms, st);
    return launch_gemm_pair_gather<float>(ta, tb, p, fmt, num_sms, st);
  }
  if (pair) {
#define GEMM_PAIR_CASE(AMN, BMN)                                                                        \
  if (a_mn == AMN && b_mn == BMN) {                                                                     \
    if (out_dtype == kBF16) return launch_gemm_pair<AMN, BMN, __nv_bfloat16>(ta, tb, p, fmt, num_sms, st); \
    if (out_dtype == kF16) return launch_gemm_pair<AMN, BMN, __half>(ta, tb, p, fmt, num_sms, st);      \
    return launch_gemm_pair<AMN, BMN, float>(ta, tb, p, fmt, num_sms, st);                              \
  }
    GEMM_PAIR_CASE(false, false)
    GEMM_PAIR_CASE(false, true)
    GEMM_PAIR_CASE(true, true)
    GEMM_PAIR_CASE(true, false)
#undef GEMM_PAIR_CASE
    return -5;
  }
#define GEMM_CASE(AMN, BMN)                                                                              \
  if (a_mn == AMN && b_mn == BMN) {                                                                      \
    if (out_dtype == kBF16) return launch_gemm<256, AMN, BMN, __nv_bfloat16>(ta, tb, p, fmt, num_sms, st); \
    if (out_dtype == kF16) return launch_gemm<256, AMN, BMN, __half>(ta, tb, p, fmt, num_sms, st);       \
    return launch_gemm<256, AMN, BMN, float>(ta, tb, p, fmt, num_sms, st);                               \
  }
  GEMM_CASE(false, false)
  GEMM_CASE(false, true)
  GEMM_CASE(true, true)
  GEMM_CASE(true, false)
#undef GEMM_CASE
  return -5;
}

void gemm_set_cta_pairs(bool on) { g_use_pair = on; }

bool gemm_gather_supported(int M, int N, int K, int world) {
  return g_use_pair && M > BM && world > 1 && world <= kMaxPeers && N % (world * 128) == 0 && K % 64 == 0;
}
int gemm_gather_flag_words(int N) { return 1 + N / 128; }

// How many CTA pairs of the pair kernel the device can hold at once (diagnostic).
int gemm_pair_max_active_clusters() {
  auto kern = gemm_tcgen05_pair_kernel<false, false, __nv_bfloat16>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PairSmem::total) != cudaSuccess) return -1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(148, 1, 1);
  cfg.blockDim = dim3(kGemmThreads, 1, 1);
  cfg.dynamicSmemBytes = PairSmem::total;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = -1;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) return -2;
  return n;
}

}  // namespace mb
