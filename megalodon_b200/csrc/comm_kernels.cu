// Communication kernels over peer-mapped ("symmetric") memory on an NVSwitch
// box: every rank holds a buffer of the same size and knows the device address
// of every peer's copy, so a kernel moves data with plain loads / stores over
// NVLink and synchronises with flags it reads and writes itself.
//
//   p2p_send / p2p_recv   chunk-parallel state handoff: the sender stores the
//                         payload straight into the receiver's mailbox slot and
//                         raises a sequence-numbered flag there; the receiver
//                         polls its own flag, copies the payload out and
//                         acknowledges into the sender's memory (flow control).
//                         Replaces the blocking NCCL send/recv pair of the
//                         reference (modules/chunk_parallel/mappings.py:25-89).
//   peer_barrier          all ranks exchange an epoch number through signal pads.
//   allreduce_sumsq       sum over ranks of a buffer held in symmetric memory;
//                         each rank reduces one slice by pulling it from every
//                         peer, accumulates the squared norm of the reduced
//                         slice on the way (the gradient-norm partial sum that
//                         clipping needs) and pushes the result to every peer.
//                         Replaces the bucketed all_reduce of grad_all_reduce
//                         plus the separate norm pass (fairscale_fsdp.py:89-219).
//
// Failure handling.  Every wait is bounded by a caller-supplied timeout, and all
// communication objects of a device share one "abort record" (kAbortWords ints,
// see `record_abort`).  The first wait that runs out writes its identity there
// (which rank, which kind of wait, direction, sequence number wanted and seen).
// From then on the failure spreads without further timeouts:
//   * every later wait on this GPU polls word 0 of the record and returns at
//     once when it is set;
//   * a kernel that gives up still signals its peer, but with the poison value
//     kPoison instead of a sequence number / epoch, so the peer's wait returns
//     immediately, records "peer gave up" and poisons its own neighbours in
//     turn.
// One lost signal therefore costs ONE timeout for the whole job, and the host
// reads who waited for what.  The record is also copied to a pinned host word
// (if one is registered) so the host can notice a failure without synchronising
// the device.  Only plain (non-multimem) peer accesses are used here.
#include <cmath>

#include "common.cuh"
#include "kernels.h"

namespace mb {
namespace {

__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

constexpr unsigned int kPoison = 0xffffffffu;     // flag value meaning "the writer gave up"

// Abort record: [0] code (0 = healthy), [1] kind of wait, [2] direction / peer index, [3] value wanted,
// [4] value seen, [5] rank of the waiting GPU in its group, [6] tag (caller's choice, e.g. unit number),
// [7] 1 when the cause was a peer's poison rather than a timeout, [8..9] address of the pinned host mirror.
constexpr int kAbortWords = 16;
enum WaitKind : int { kWaitSendAck = 1, kWaitRecv = 2, kWaitBarrier = 3, kWaitStaged = 4 };
constexpr int kCodeBadIndex = 30;     // a table-driven kernel computed an index outside its buffer
enum WaitResult : int { kWaitOk = 0, kWaitTimedOut = 1, kWaitAborted = 2, kWaitPoisoned = 3 };

__device__ __forceinline__ int ld_volatile(const int* p) { return *reinterpret_cast<const volatile int*>(p); }

// Wait until *flag >= want (unsigned, sequence numbers and epochs only grow and never reach kPoison).
__device__ __forceinline__ WaitResult wait_flag_ge(const unsigned int* flag, unsigned int want,
                                                   unsigned long long timeout_ns, const int* abort,
                                                   unsigned int* seen) {
  unsigned int v = ld_acquire_sys(flag);
  const unsigned long long t0 = now_ns();
  // Exponential back-off up to 2 us per poll: a waiting warp shares its SM with whatever compute
  // kernel runs on the other streams, and a tight poll loop steals issue slots from it.
  unsigned int spins = 0, pause_ns = 32;
  while (true) {
    *seen = v;
    if (v == kPoison) return kWaitPoisoned;
    if (v >= want) return kWaitOk;
    if ((++spins & 0x7) == 0) {
      if (ld_volatile(abort) != 0) return kWaitAborted;
      if (now_ns() - t0 > timeout_ns) return kWaitTimedOut;
    }
    __nanosleep(pause_ns);
    if (pause_ns < 2048) pause_ns <<= 1;
    v = ld_acquire_sys(flag);
  }
}

// First failure wins.  `res` is what wait_flag_ge returned (a wait that ended because the record was
// already set has nothing to add).
__device__ __forceinline__ void record_abort(int* abort, WaitResult res, int kind, int dir_or_peer,
                                             unsigned int want, unsigned int seen, int rank, int tag) {
  if (res != kWaitTimedOut && res != kWaitPoisoned) return;
  if (atomicCAS(abort, 0, 10 + kind) != 0) return;
  abort[1] = kind; abort[2] = dir_or_peer; abort[3] = (int)want; abort[4] = (int)seen; abort[5] = rank;
  abort[6] = tag; abort[7] = res == kWaitPoisoned ? 1 : 0;
  __threadfence();
  const unsigned long long host = ((unsigned long long)(unsigned int)abort[9] << 32) | (unsigned int)abort[8];
  if (host != 0) {
    volatile int* h = reinterpret_cast<volatile int*>(host);
    for (int i = 1; i < 8; ++i) h[i] = abort[i];
    __threadfence_system();
    h[0] = 10 + kind;
  }
}

// Index check of the table-driven kernels (a wrong piece table must not become a fault on a peer GPU):
// returns true if [idx, idx + n) lies inside [0, limit); otherwise records the index once and the caller
// skips the access.  `limit` <= 0 disables the check.
__device__ __forceinline__ bool index_ok(long long idx, long long n, long long limit, int* abort, int where) {
  if (limit <= 0 || (idx >= 0 && idx + n <= limit)) return true;
  if (abort != nullptr && atomicCAS(abort, 0, kCodeBadIndex) == 0) {
    abort[1] = where; abort[2] = (int)(idx >> 32); abort[3] = (int)(limit & 0x7fffffff); abort[4] = (int)(idx & 0xffffffff);
    abort[5] = -1; abort[6] = 0; abort[7] = 0;
  }
  return false;
}

// True (for every thread of the CTA alike) when the device's abort record is set: data kernels then
// return without touching peer memory, so a failed step drains quickly.
__device__ __forceinline__ bool block_sees_abort(const int* abort) {
  __shared__ int dead;
  if (threadIdx.x == 0) dead = abort != nullptr && ld_volatile(abort) != 0;
  __syncthreads();
  return dead != 0;
}

// Counts CTAs that have finished; returns true in exactly one thread of the last CTA to arrive.
// `failed` CTAs leave a mark, and `*any_failed` tells the last CTA whether any did.
__device__ __forceinline__ bool last_block_done(unsigned int* counter, bool failed, bool* any_failed) {
  __shared__ bool is_last;
  __shared__ bool some_failed;
  __threadfence_system();           // this CTA's (possibly remote) stores are ordered before the count
  __syncthreads();
  if (threadIdx.x == 0) {
    if (failed) atomicOr(counter, 0x40000000u);
    const unsigned int prev = atomicAdd(counter, 1u);
    is_last = (prev & 0xffffu) == gridDim.x - 1;
    some_failed = (prev & 0x40000000u) != 0;
    if (is_last) *counter = 0;      // ready for the next launch
  }
  __syncthreads();
  *any_failed = some_failed;
  return is_last && threadIdx.x == 0;
}

// payload: n16 16-byte words.  remote_* live in the receiver's memory, local_ack in ours.
__global__ void p2p_send_kernel(const uint4* __restrict__ src, uint4* __restrict__ remote_dst, long long n16,
                                unsigned int* remote_flag, unsigned int seq, const unsigned int* local_ack,
                                unsigned int need_ack, unsigned int* counter, unsigned long long timeout_ns,
                                int* abort, int rank, int dir) {
  __shared__ int ok;
  if (threadIdx.x == 0) {
    WaitResult res = ld_volatile(abort) != 0 ? kWaitAborted : kWaitOk;
    unsigned int seen = 0;
    if (res == kWaitOk && need_ack != 0) res = wait_flag_ge(local_ack, need_ack, timeout_ns, abort, &seen);
    // a timeout here means: slot still unacknowledged, the receiver is gone or too far behind
    record_abort(abort, res, kWaitSendAck, dir, need_ack, seen, rank, (int)seq);
    ok = res == kWaitOk ? 1 : 0;
  }
  __syncthreads();
  if (ok) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16;
         i += (long long)gridDim.x * blockDim.x)
      remote_dst[i] = src[i];
  }
  bool any_failed;
  const bool flagger = last_block_done(counter, !ok, &any_failed);
  if (flagger) st_release_sys(remote_flag, any_failed ? kPoison : seq);     // a poisoned flag releases the receiver
}

// `poison`: after a word has been copied out, the slot word is overwritten with kSlotPoison (a quiet NaN
// in fp32, bf16 and fp16) before the acknowledgement goes out.  A receiver that ever reads a slot the
// sender has not refilled then sees NaNs instead of the plausible values of an older message.
constexpr unsigned int kSlotPoison = 0x7fc07fc0u;
__global__ void p2p_recv_kernel(uint4* __restrict__ dst, uint4* __restrict__ local_slot, long long n16,
                                const unsigned int* local_flag, unsigned int seq, unsigned int* remote_ack,
                                unsigned int* counter, unsigned long long timeout_ns, int* abort, int rank,
                                int dir, int poison) {
  __shared__ int ok;
  if (threadIdx.x == 0) {
    WaitResult res = ld_volatile(abort) != 0 ? kWaitAborted : kWaitOk;
    unsigned int seen = 0;
    if (res == kWaitOk) res = wait_flag_ge(local_flag, seq, timeout_ns, abort, &seen);
    record_abort(abort, res, kWaitRecv, dir, seq, seen, rank, (int)seq);    // timeout: the message never arrived
    ok = res == kWaitOk ? 1 : 0;
  }
  __syncthreads();
  if (ok) {
    const uint4 bad = make_uint4(kSlotPoison, kSlotPoison, kSlotPoison, kSlotPoison);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16;
         i += (long long)gridDim.x * blockDim.x) {
      dst[i] = local_slot[i];
      if (poison) local_slot[i] = bad;
    }
  }
  bool any_failed;
  const bool acker = last_block_done(counter, !ok, &any_failed);
  if (acker && remote_ack != nullptr) st_release_sys(remote_ack, any_failed ? kPoison : seq);
}

// Each rank writes `epoch` into slot [rank] of every peer's pad and waits until all slots of its own
// pad reach `epoch`.  pads[p] is the address of rank p's pad (an array of `world` uint32).  One warp.
__global__ void peer_barrier_kernel(unsigned int* const* __restrict__ pads, int rank, int world, unsigned int epoch,
                                    unsigned long long timeout_ns, int* abort, int tag) {
  const int p = threadIdx.x;
  const bool dead = ld_volatile(abort) != 0;
  __threadfence_system();
  if (p < world && !dead) st_release_sys(pads[p] + rank, epoch);
  WaitResult res = dead ? kWaitAborted : kWaitOk;
  unsigned int seen = 0;
  if (p < world && !dead) res = wait_flag_ge(pads[rank] + p, epoch, timeout_ns, abort, &seen);
  record_abort(abort, res, kWaitBarrier, p, epoch, seen, rank, tag);
  // one failed wait poisons this rank's slot on every peer, so their barriers return at once
  if (__any_sync(0xffffffffu, res != kWaitOk) && p < world) st_release_sys(pads[p] + rank, kPoison);
}

template <typename T>
struct Vec8;
template <>
struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void unpack(const uint4& u, float (&f)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __low2float(h[i]);
      f[2 * i + 1] = __high2float(h[i]);
    }
  }
  static __device__ __forceinline__ uint4 pack(const float (&f)[8]) {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return u;
  }
};
template <>
struct Vec8<__half> {
  static __device__ __forceinline__ void unpack(const uint4& u, float (&f)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __low2float(h[i]);
      f[2 * i + 1] = __high2float(h[i]);
    }
  }
  static __device__ __forceinline__ uint4 pack(const float (&f)[8]) {
    uint4 u;
    __half2* h = reinterpret_cast<__half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    return u;
  }
};

// ---- small all-reduce / all-gather of a decode step (a few rows of activations) in ONE kernel that can
// be captured in a CUDA graph: the epoch is not a launch argument but a counter in device memory that the
// kernel itself advances, so a replayed graph keeps the flag protocol intact.  Every rank stores its
// vector into slot [rank] of every peer's buffer (two buffers, alternating with the epoch: a rank can be
// at most one collective ahead of the slowest, because it needs that rank's flag of the current one),
// raises flag [rank] on every peer, waits for all flags of its own pad, then sums (or concatenates) the
// `world` slots of its own buffer in rank order - the same order on every rank, so all ranks hold
// identical results.  One CTA; n16 = number of 16-byte words of the vector.
//   bufs[p]  : rank p's buffer, 2 * world * slot16 words      pads[p] : rank p's flags, `world` uint32
template <typename T, bool GATHER>
__global__ void small_collective_kernel(const uint4* __restrict__ x, uint4* __restrict__ out,
                                        uint4* const* __restrict__ bufs, unsigned int* const* __restrict__ pads,
                                        unsigned int* __restrict__ counter, int rank, int world, int n16,
                                        int slot16, int rows, unsigned long long timeout_ns, int* abort) {
  __shared__ unsigned int s_epoch;
  __shared__ int s_fail;
  if (threadIdx.x == 0) {
    s_epoch = *counter + 1;
    s_fail = ld_volatile(abort) != 0 ? 1 : 0;
  }
  __syncthreads();
  const unsigned int epoch = s_epoch;
  const long long half = (long long)(epoch & 1u) * world * slot16;
  if (!s_fail) {
    for (int p = 0; p < world; ++p) {
      uint4* dst = bufs[p] + half + (long long)rank * slot16;
      for (int i = threadIdx.x; i < n16; i += blockDim.x) dst[i] = x[i];
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < 32) {
    const int p = threadIdx.x;
    WaitResult res = s_fail ? kWaitAborted : kWaitOk;
    unsigned int seen = 0;
    if (p < world && !s_fail) {
      st_release_sys(pads[p] + rank, epoch);
      res = wait_flag_ge(pads[rank] + p, epoch, timeout_ns, abort, &seen);
    }
    record_abort(abort, res, kWaitBarrier, p, epoch, seen, rank, 0x5c);
    if (__any_sync(0xffffffffu, res != kWaitOk)) {
      if (p < world) st_release_sys(pads[p] + rank, kPoison);
      if (p == 0) s_fail = 1;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) *counter = epoch;
  if (s_fail) return;
  const uint4* mine = bufs[rank] + half;
  if (GATHER) {
    // slot r holds [rows, n16 / rows] words; the result is [rows, world * n16 / rows]
    const int w = n16 / rows;
    for (int i = threadIdx.x; i < n16 * world; i += blockDim.x) {
      const int row = i / (w * world), c = i - row * (w * world);
      const int r = c / w, j = c - r * w;
      out[i] = mine[(long long)r * slot16 + row * w + j];
    }
  } else {
    for (int i = threadIdx.x; i < n16; i += blockDim.x) {
      float acc[8];
      Vec8<T>::unpack(mine[i], acc);
      for (int r = 1; r < world; ++r) {
        float f[8];
        Vec8<T>::unpack(mine[(long long)r * slot16 + i], f);
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] += f[k];
      }
      out[i] = Vec8<T>::pack(acc);
    }
  }
}

// 16-bit element types: 8 elements per 16-byte word.  bufs[p] = address of rank p's copy.
// Rank r owns words [r * slice16, (r + 1) * slice16) of the n16-word buffer.
template <typename T>
__global__ void allreduce_sumsq_16bit_kernel(uint4* const* __restrict__ bufs, int rank, int world, long long n16,
                                             long long slice16, float scale, double* __restrict__ sumsq,
                                             const int* abort) {
  __shared__ float scratch[32];
  if (block_sees_abort(abort)) return;
  const long long lo = (long long)rank * slice16;
  const long long hi = min(n16, lo + slice16);
  float ss = 0.f;
  for (long long i = lo + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < hi;
       i += (long long)gridDim.x * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int p = 0; p < world; ++p) {
      const int src = (rank + p) % world;          // start with the local copy, then walk the peers
      float f[8];
      Vec8<T>::unpack(bufs[src][i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      acc[j] *= scale;
      ss += acc[j] * acc[j];
    }
    const uint4 out = Vec8<T>::pack(acc);
    for (int p = 0; p < world; ++p) bufs[(rank + p) % world][i] = out;
  }
  ss = block_sum(ss, scratch);
  if (threadIdx.x == 0 && sumsq != nullptr) atomicAdd(sumsq, (double)ss);
}

__global__ void allreduce_sumsq_f32_kernel(float4* const* __restrict__ bufs, int rank, int world, long long n16,
                                           long long slice16, float scale, double* __restrict__ sumsq,
                                           const int* abort) {
  __shared__ float scratch[32];
  if (block_sees_abort(abort)) return;
  const long long lo = (long long)rank * slice16;
  const long long hi = min(n16, lo + slice16);
  float ss = 0.f;
  for (long long i = lo + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < hi;
       i += (long long)gridDim.x * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p = 0; p < world; ++p) {
      const float4 f = bufs[(rank + p) % world][i];
      acc.x += f.x; acc.y += f.y; acc.z += f.z; acc.w += f.w;
    }
    acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
    ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
    for (int p = 0; p < world; ++p) bufs[(rank + p) % world][i] = acc;
  }
  ss = block_sum(ss, scratch);
  if (threadIdx.x == 0 && sumsq != nullptr) atomicAdd(sumsq, (double)ss);
}

// Per-parameter sharding (parallel/fsdp.py): rank r's shard is the concatenation of piece r of every
// parameter, while gradients and gathered parameters are laid out in natural order.  `table` holds one
// row (shard_offset, piece, offset) per parameter; all three are multiples of 64 elements, so a
// 16-byte vector never straddles two pieces.  Returns the natural-order index of shard element `i`
// of rank `rank`.
constexpr int kMaxPieces = 96;
struct PieceMap {
  long long shard_end[kMaxPieces];     // shard_offset + piece
  long long delta[kMaxPieces];         // offset + rank * piece - shard_offset
};
__device__ __forceinline__ void load_piece_map(PieceMap* pm, const long long* __restrict__ table, int npieces,
                                               int rank) {
  for (int i = threadIdx.x; i < npieces; i += blockDim.x) {
    const long long so = table[3 * i], piece = table[3 * i + 1], off = table[3 * i + 2];
    pm->shard_end[i] = so + piece;
    pm->delta[i] = off + (long long)rank * piece - so;
  }
  __syncthreads();
}
__device__ __forceinline__ long long shard_to_natural(const PieceMap* pm, int npieces, long long i) {
  int lo = 0, hi = npieces - 1;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (i < pm->shard_end[mid]) hi = mid; else lo = mid + 1;
  }
  return i + pm->delta[lo];
}

// Reduce-scatter by pull: this rank sums ITS slice of every peer's staged buffer in fp32, scales it
// (gradient averaging), stores it to a local shard in the output dtype and accumulates the squared
// norm of what it stored.  One pass replaces reduce-scatter + cast/scale + the gradient-norm pass.
template <typename T, typename O>
__global__ void reduce_scatter_sumsq_kernel(const T* const* __restrict__ bufs, int rank, int world,
                                            long long shard_n, float scale, O* __restrict__ out,
                                            double* __restrict__ sumsq, bool accumulate, const int* abort,
                                            const long long* __restrict__ table, int npieces) {
  __shared__ float scratch[32];
  __shared__ PieceMap pm;
  if (block_sees_abort(abort)) return;
  if (table != nullptr) load_piece_map(&pm, table, npieces, rank);
  constexpr int kMaxWorld = 8;
  constexpr int kPer = 16 / sizeof(T);           // elements per 16-byte load
  const long long lo = table != nullptr ? 0 : (long long)rank * shard_n;
  const T* src[kMaxWorld];
#pragma unroll
  for (int p = 0; p < kMaxWorld; ++p) src[p] = p < world ? bufs[(rank + p) % world] + lo : nullptr;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long nvec = (world <= kMaxWorld) ? shard_n / kPer : 0;
  float ss = 0.f;
  // every peer's 16 bytes are requested before any is used: up to 8 remote loads in flight per thread,
  // 512-byte requests per warp on the link
  for (long long v = tid; v < nvec; v += stride) {
    uint4 raw[kMaxWorld];
    const long long at = table != nullptr ? shard_to_natural(&pm, npieces, v * kPer) : v * kPer;
    if (table != nullptr && !index_ok(at, kPer, (long long)world * shard_n, const_cast<int*>(abort), 3)) continue;
#pragma unroll
    for (int p = 0; p < kMaxWorld; ++p)
      if (p < world) raw[p] = __ldcv(reinterpret_cast<const uint4*>(src[p] + at));
    float acc[kPer];
#pragma unroll
    for (int j = 0; j < kPer; ++j) acc[j] = 0.f;
#pragma unroll
    for (int p = 0; p < kMaxWorld; ++p) {
      if (p < world) {
        const T* e = reinterpret_cast<const T*>(&raw[p]);
#pragma unroll
        for (int j = 0; j < kPer; ++j) acc[j] += to_f(e[j]);
      }
    }
    if constexpr (kPer == 8) {
      float prev[8];
      if (accumulate) load8(out + v * 8, prev);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        acc[j] = accumulate ? fmaf(acc[j], scale, prev[j]) : acc[j] * scale;
        ss = fmaf(acc[j], acc[j], ss);
      }
      store8(out + v * 8, acc);
    } else {
#pragma unroll
      for (int j = 0; j < kPer; ++j) {
        acc[j] *= scale;
        if (accumulate) acc[j] += to_f(out[v * kPer + j]);
        ss = fmaf(acc[j], acc[j], ss);
        out[v * kPer + j] = from_f<O>(acc[j]);
      }
    }
  }
  for (long long i = nvec * kPer + tid; i < shard_n; i += stride) {     // tail (and world > 8)
    float acc = 0.f;
    const long long at = table != nullptr ? shard_to_natural(&pm, npieces, i) : i;
    for (int p = 0; p < world; ++p) acc += to_f(bufs[(rank + p) % world][lo + at]);
    acc *= scale;
    if (accumulate) acc += to_f(out[i]);
    ss = fmaf(acc, acc, ss);
    out[i] = from_f<O>(acc);
  }
  ss = block_sum(ss, scratch);
  if (threadIdx.x == 0 && sumsq != nullptr) atomicAdd(sumsq, (double)ss);
}

// Reduce-scatter fused with the sharded AdamW update (for runs without global-norm clipping, where the
// update of a shard needs nothing but its own reduced gradient): pull this rank's slice of every peer's
// staged gradient, sum in fp32, apply the 1/dp scale, then update the fp32 master weights and both
// moments in place and write the compute-dtype copy that the next forward's all-gather reads.  The
// reduced gradient is never written to memory; `sumsq` still receives its squared norm for logging.
template <typename T, typename Lo>
__global__ void reduce_scatter_adamw_kernel(const T* const* __restrict__ bufs, int rank, int world, long long shard_n,
                                            float scale, float* __restrict__ p, float* __restrict__ m,
                                            float* __restrict__ v, Lo* __restrict__ low, double* __restrict__ sumsq,
                                            float lr, float beta1, float beta2, float eps, float wd, float bc1,
                                            float bc2_sqrt, const int* abort, const long long* __restrict__ table,
                                            int npieces) {
  __shared__ float scratch[32];
  __shared__ PieceMap pm;
  if (block_sees_abort(abort)) return;
  if (table != nullptr) load_piece_map(&pm, table, npieces, rank);
  constexpr int kMaxWorld = 8;
  static_assert(sizeof(T) == 2, "gradients are staged in a 16-bit type");
  const long long lo = table != nullptr ? 0 : (long long)rank * shard_n;
  const T* src[kMaxWorld];
#pragma unroll
  for (int q = 0; q < kMaxWorld; ++q) src[q] = q < world ? bufs[(rank + q) % world] + lo : nullptr;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long nvec = shard_n / 8;
  const float step = lr / bc1;
  const float decay = 1.f - lr * wd;
  float ss = 0.f;
  for (long long i = tid; i < nvec; i += stride) {
    uint4 raw[kMaxWorld];
    const long long at = table != nullptr ? shard_to_natural(&pm, npieces, i * 8) : i * 8;
    if (table != nullptr && !index_ok(at, 8, (long long)world * shard_n, const_cast<int*>(abort), 4)) continue;
#pragma unroll
    for (int q = 0; q < kMaxWorld; ++q)
      if (q < world) raw[q] = __ldcv(reinterpret_cast<const uint4*>(src[q] + at));
    float g[8], pv[8], mv[8], vv[8];
    load8(p + i * 8, pv);
    load8(m + i * 8, mv);
    load8(v + i * 8, vv);
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] = 0.f;
#pragma unroll
    for (int q = 0; q < kMaxWorld; ++q) {
      if (q < world) {
        const T* e = reinterpret_cast<const T*>(&raw[q]);
#pragma unroll
        for (int j = 0; j < 8; ++j) g[j] += to_f(e[j]);
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gj = g[j] * scale;
      ss = fmaf(gj, gj, ss);
      mv[j] = beta1 * mv[j] + (1.f - beta1) * gj;
      vv[j] = beta2 * vv[j] + (1.f - beta2) * gj * gj;
      pv[j] = pv[j] * decay - step * mv[j] / (sqrtf(vv[j]) / bc2_sqrt + eps);
    }
    store8(m + i * 8, mv);
    store8(v + i * 8, vv);
    store8(p + i * 8, pv);
    if (low != nullptr) store8(low + i * 8, pv);
  }
  ss = block_sum(ss, scratch);
  if (threadIdx.x == 0 && sumsq != nullptr) atomicAdd(sumsq, (double)ss);
}

// Parameter all-gather by pull into the natural layout.  The table may list all parameters of a unit
// or a subset (the rest being gathered by the GEMMs that consume them); the kernel walks the listed
// parameters back to back.  Word k of parameter p (0 <= k < world * piece) lives on rank k / piece at
// shard index shard_offset + k % piece and goes to natural index offset + k.  Four loads per thread
// are in flight before the first store.
struct NaturalMap {
  long long cum_end[kMaxPieces];       // elements of the listed parameters up to and including this one
  long long off[kMaxPieces], piece[kMaxPieces], soff[kMaxPieces];
};
__global__ void gather_pull_kernel(uint4* __restrict__ full, const uint4* const* __restrict__ peer_shards, int world,
                                   const long long* __restrict__ table, int npieces, int per, const int* abort,
                                   long long shard_numel, long long full_numel) {
  __shared__ NaturalMap nm;
  __shared__ long long total;
  if (block_sees_abort(abort)) return;
  if (threadIdx.x == 0) {
    long long cum = 0;
    for (int i = 0; i < npieces; ++i) {
      nm.soff[i] = table[3 * i]; nm.piece[i] = table[3 * i + 1]; nm.off[i] = table[3 * i + 2];
      cum += (long long)world * nm.piece[i];
      nm.cum_end[i] = cum;
    }
    total = cum;
  }
  __syncthreads();
  const long long nwords = total / per;
  constexpr int kUnroll = 4;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long w0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; w0 < nwords; w0 += stride * kUnroll) {
    uint4 v[kUnroll];
    long long dst[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const long long w = w0 + u * stride;
      dst[u] = -1;
      if (w < nwords) {
        const long long n = w * per;                      // element index within the listed parameters
        int lo = 0, hi = npieces - 1;
        while (lo < hi) {
          const int mid = (lo + hi) >> 1;
          if (n < nm.cum_end[mid]) hi = mid; else lo = mid + 1;
        }
        const long long rel = n - (nm.cum_end[lo] - (long long)world * nm.piece[lo]);
        const long long r = rel / nm.piece[lo];
        const long long j = rel - r * nm.piece[lo];
        if (index_ok(nm.soff[lo] + j, per, shard_numel, const_cast<int*>(abort), 1) &&
            index_ok(nm.off[lo] + rel, per, full_numel, const_cast<int*>(abort), 2)) {
          v[u] = __ldcv(peer_shards[r] + (nm.soff[lo] + j) / per);
          dst[u] = (nm.off[lo] + rel) / per;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
      if (dst[u] >= 0) full[dst[u]] = v[u];
  }
}

template <typename T>
__global__ void reduce_slots_kernel(const T* __restrict__ slots, T* __restrict__ out, long long n, int world) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    float acc = 0.f;
    for (int w = 0; w < world; ++w) acc += to_f(slots[(long long)w * n + i]);
    out[i] = from_f<T>(acc);
  }
}

// Kernels of this file run on side streams next to the persistent GEMM, whose CTAs need nearly all of
// an SM's shared memory.  An SM's L1 / shared-memory split is fixed while any CTA is resident on it,
// so a waiting CTA launched with the default (L1-heavy) split keeps a GEMM CTA off that SM until the
// wait ends, and a statically scheduled persistent kernel then runs at the pace of the CTA that
// started late.  Asking for the largest shared-memory carve-out makes the two co-resident.
template <typename K>
void prefer_max_shared(K kernel) {
  cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}

}  // namespace

void reduce_slots(const void* slots, void* out, long long n, int world, int dtype, cudaStream_t st) {
  if (n == 0) return;
  const int grid = (int)std::min<long long>(div_up(n, 256), 148LL * 16);
  MB_DISPATCH_DTYPE(dtype, (reduce_slots_kernel<scalar_t><<<grid, 256, 0, st>>>((const scalar_t*)slots, (scalar_t*)out,
                                                                             n, world)));
}

void reduce_scatter_sumsq(const void* const* bufs, int rank, int world, long long shard_n, float scale, void* out,
                          double* sumsq, bool accumulate, int in_dtype, int out_dtype, const int* abort,
                          const long long* table, int npieces, cudaStream_t st) {
  if (shard_n == 0) return;
  if (npieces > kMaxPieces) table = nullptr, npieces = -1;          // caller checks piece_table_limit()
  const int grid = (int)std::min<long long>(div_up(shard_n / 8 + 1, 256), 148LL * 4);
  MB_DISPATCH_DTYPE(in_dtype, {
    using T = scalar_t;
    if (out_dtype == kF32 && in_dtype != kF32) {
      prefer_max_shared(reduce_scatter_sumsq_kernel<T, float>);
      reduce_scatter_sumsq_kernel<T, float><<<grid, 256, 0, st>>>((const T* const*)bufs, rank, world, shard_n, scale,
                                                                 (float*)out, sumsq, accumulate, abort, table, npieces);
    } else {
      prefer_max_shared(reduce_scatter_sumsq_kernel<T, T>);
      reduce_scatter_sumsq_kernel<T, T><<<grid, 256, 0, st>>>((const T* const*)bufs, rank, world, shard_n, scale,
                                                             (T*)out, sumsq, accumulate, abort, table, npieces);
    }
  });
}

// shard_n must be a multiple of 8 and world <= 8; `low` may be null.  Returns false otherwise.
bool reduce_scatter_adamw(const void* const* bufs, int rank, int world, long long shard_n, float scale, float* p,
                          float* m, float* v, void* low, double* sumsq, float lr, float beta1, float beta2, float eps,
                          float wd, int step, int in_dtype, int low_dtype, const int* abort, const long long* table,
                          int npieces, cudaStream_t st) {
  if (shard_n == 0) return true;
  if (npieces > kMaxPieces) return false;
  if (shard_n % 8 != 0 || world > 8 || in_dtype == kF32 || (low != nullptr && low_dtype != in_dtype)) return false;
  const float bc1 = 1.f - powf(beta1, (float)step);
  const float bc2s = sqrtf(1.f - powf(beta2, (float)step));
  const int grid = (int)std::min<long long>(div_up(shard_n / 8, 256), 148LL * 4);
  if (in_dtype == kBF16) {
    prefer_max_shared(reduce_scatter_adamw_kernel<__nv_bfloat16, __nv_bfloat16>);
    reduce_scatter_adamw_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, st>>>(
        (const __nv_bfloat16* const*)bufs, rank, world, shard_n, scale, p, m, v, (__nv_bfloat16*)low, sumsq, lr, beta1,
        beta2, eps, wd, bc1, bc2s, abort, table, npieces);
  } else {
    prefer_max_shared(reduce_scatter_adamw_kernel<__half, __half>);
    reduce_scatter_adamw_kernel<__half, __half><<<grid, 256, 0, st>>>(
        (const __half* const*)bufs, rank, world, shard_n, scale, p, m, v, (__half*)low, sumsq, lr, beta1, beta2, eps, wd,
        bc1, bc2s, abort, table, npieces);
  }
  return true;
}

int piece_table_limit() { return kMaxPieces; }

void gather_pull(void* full, const void* const* peer_shards, int world, const long long* table, int npieces,
                 long long listed_numel, int esize, const int* abort, long long shard_numel, long long full_numel,
                 cudaStream_t st) {
  if (listed_numel == 0 || npieces == 0 || npieces > kMaxPieces) return;
  const int per = 16 / esize;
  const long long nwords = listed_numel / per;
  const int grid = (int)std::max<long long>(1, std::min<long long>(div_up(nwords, 256 * 4), 148LL * 4));
  prefer_max_shared(gather_pull_kernel);
  gather_pull_kernel<<<grid, 256, 0, st>>>((uint4*)full, (const uint4* const*)peer_shards, world, table, npieces, per,
                                           abort, shard_numel, full_numel);
}

void p2p_send(const void* src, void* remote_dst, long long nbytes, unsigned int* remote_flag, unsigned int seq,
              const unsigned int* local_ack, unsigned int need_ack, unsigned int* counter,
              unsigned long long timeout_ns, int* abort, int rank, int dir, cudaStream_t st) {
  const long long n16 = nbytes / 16;
  const int grid = (int)std::max<long long>(1, std::min<long long>(div_up(n16, 256), 16));
  prefer_max_shared(p2p_send_kernel);
  p2p_send_kernel<<<grid, 256, 0, st>>>((const uint4*)src, (uint4*)remote_dst, n16, remote_flag, seq, local_ack,
                                        need_ack, counter, timeout_ns, abort, rank, dir);
}

void p2p_recv(void* dst, void* local_slot, long long nbytes, const unsigned int* local_flag, unsigned int seq,
              unsigned int* remote_ack, unsigned int* counter, unsigned long long timeout_ns, int* abort, int rank,
              int dir, bool poison, cudaStream_t st) {
  const long long n16 = nbytes / 16;
  const int grid = (int)std::max<long long>(1, std::min<long long>(div_up(n16, 256), 16));
  prefer_max_shared(p2p_recv_kernel);
  p2p_recv_kernel<<<grid, 256, 0, st>>>((uint4*)dst, (uint4*)local_slot, n16, local_flag, seq, remote_ack,
                                        counter, timeout_ns, abort, rank, dir, poison ? 1 : 0);
}

void peer_barrier(unsigned int* const* pads, int rank, int world, unsigned int epoch, unsigned long long timeout_ns,
                  int* abort, int tag, cudaStream_t st) {
  prefer_max_shared(peer_barrier_kernel);
  peer_barrier_kernel<<<1, 32, 0, st>>>(pads, rank, world, epoch, timeout_ns, abort, tag);
}

void small_collective(const void* x, void* out, void* const* bufs, unsigned int* const* pads, unsigned int* counter,
                      int rank, int world, long long nbytes, long long slot_bytes, int rows, bool gather, int dtype,
                      unsigned long long timeout_ns, int* abort, cudaStream_t st) {
  const int n16 = (int)(nbytes / 16), slot16 = (int)(slot_bytes / 16);
  const int threads = 1024;
  if (gather) {
    prefer_max_shared(small_collective_kernel<__nv_bfloat16, true>);
    small_collective_kernel<__nv_bfloat16, true><<<1, threads, 0, st>>>(
        (const uint4*)x, (uint4*)out, (uint4* const*)bufs, pads, counter, rank, world, n16, slot16, rows, timeout_ns, abort);
  } else if (dtype == kBF16) {
    prefer_max_shared(small_collective_kernel<__nv_bfloat16, false>);
    small_collective_kernel<__nv_bfloat16, false><<<1, threads, 0, st>>>(
        (const uint4*)x, (uint4*)out, (uint4* const*)bufs, pads, counter, rank, world, n16, slot16, rows, timeout_ns, abort);
  } else {
    prefer_max_shared(small_collective_kernel<__half, false>);
    small_collective_kernel<__half, false><<<1, threads, 0, st>>>(
        (const uint4*)x, (uint4*)out, (uint4* const*)bufs, pads, counter, rank, world, n16, slot16, rows, timeout_ns, abort);
  }
}

void allreduce_sumsq(void* const* bufs, int rank, int world, long long nbytes, float scale, double* sumsq,
                     int dtype, const int* abort, cudaStream_t st) {
  const long long n16 = nbytes / 16;
  const long long slice16 = (n16 + world - 1) / world;
  const int grid = (int)std::max<long long>(1, std::min<long long>(div_up(slice16, 256), 148LL * 4));
  if (dtype == kBF16) {
    prefer_max_shared(allreduce_sumsq_16bit_kernel<__nv_bfloat16>);
    allreduce_sumsq_16bit_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((uint4* const*)bufs, rank, world, n16, slice16,
                                                                    scale, sumsq, abort);
  } else if (dtype == kF16) {
    prefer_max_shared(allreduce_sumsq_16bit_kernel<__half>);
    allreduce_sumsq_16bit_kernel<__half><<<grid, 256, 0, st>>>((uint4* const*)bufs, rank, world, n16, slice16, scale,
                                                             sumsq, abort);
  } else {
    prefer_max_shared(allreduce_sumsq_f32_kernel);
    allreduce_sumsq_f32_kernel<<<grid, 256, 0, st>>>((float4* const*)bufs, rank, world, n16, slice16, scale, sumsq,
                                                     abort);
  }
}

}  // namespace mb
