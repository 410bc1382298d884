// Launchers of the sm_100a kernels.  Plain C++ signatures over raw device
// pointers so the kernel translation units do not depend on libtorch.
#pragma once

#include <cuda_runtime.h>

namespace mb {

// ---- row-wise norms (norm_kernels.cu); weight dtype is fp32 or the activation dtype
void rms_norm_fwd(const void* x, const void* w, float w_off, void* y, float* rstd, long long M, int D,
                  float eps, int x_dtype, int w_dtype, cudaStream_t st);
// `colsum_ws`: kColsumRows * D floats (2 * kColsumRows * D for LayerNorm and TimestepNorm) or null.  With
// it, every CTA of the wide-row kernels stores its partial column sums (the weight / bias gradients) as one
// plain row and `colsum_finish` adds the rows up; without it the partial sums go out as atomics.  Either
// way the sums are ADDED to dw / db.
constexpr int kColsumRows = 296;
void colsum_finish(const float* ws, int rows, int D, float* out0, float* out1, cudaStream_t st);
// out[j] += sum over rows of a row-major 16-bit matrix [M, N] (bias gradients); false: shape not covered
bool colsum_16bit(const void* g, long long M, int N, float* ws, float* out, int dtype, cudaStream_t st);
void rms_norm_bwd(const void* dy, const void* x, const void* w, float w_off, const float* rstd, void* dx,
                  float* dw, long long M, int D, int x_dtype, int w_dtype, cudaStream_t st,
                  float* colsum_ws = nullptr);
void layer_norm_fwd(const void* x, const void* w, const void* b, float w_off, void* y, float* mean,
                    float* rstd, long long M, int D, float eps, int x_dtype, int w_dtype, cudaStream_t st);
void layer_norm_bwd(const void* dy, const void* x, const void* w, float w_off, const float* mean,
                    const float* rstd, void* dx, float* dw, float* db, long long M, int D, int x_dtype,
                    int w_dtype, cudaStream_t st, float* colsum_ws = nullptr);

// ---- TimestepNorm (timestep_norm_kernels.cu)
void timestep_norm_fwd(const void* x, const long long* prev_count, const void* prev_mean,
                       const void* prev_var, const void* gamma, float gamma_offset, const void* beta,
                       const bool* mask, void* y, long long* count_out, void* mean_out, void* var_out,
                       float* cummean, float* cumrstd, float* gu, float* gv, double* seg_scratch, int B, int L,
                       int H, int G, float eps, int x_dtype, int w_dtype, cudaStream_t st);
// scan segments per sequence; the forward pass needs 3 * B * nseg * G doubles of scratch, the backward
// pass 4 * B * nseg * G doubles (+ B * L ints when a padding mask is given)
int tsn_num_segments(int L);
void timestep_norm_bwd(const void* dy, const void* dmean_out, const void* dvar_out, const void* x,
                       const void* prev_mean, const long long* count_final, const float* cummean,
                       const float* cumrstd, const void* gamma, float gamma_offset, const bool* mask,
                       void* dx, void* dprev_mean, void* dprev_var, float* dgamma, float* dbeta,
                       float* ux, float* ds, float* db, float* dux, float* dvx, double* seg_scratch,
                       int* cumvalid, int B, int L, int H, int G, int x_dtype, int w_dtype, cudaStream_t st,
                       float* colsum_ws = nullptr);

// ---- CEMA (cema_kernels.cu); complex tensors are interleaved (re, im) fp32
constexpr int kCemaSegLen = 128;
bool cema_supported_ndim(int N);
int cema_num_segments(int L);
// carry: scratch of B * S * N * D complex (S = cema_num_segments(L)); unused when S == 1
void cema_fwd(const void* x, const float* p, const float* q, const float* gamma, const float* omega,
              const float* hx, void* y, float* h_last, float* carry, int B, int L, int D, int N,
              int x_dtype, cudaStream_t st);
// dp [D,N], dq/dgamma [D,N,2], domega [D] must be zero-initialised (accumulated with atomics)
void cema_bwd(const void* dy, const void* x, const float* p, const float* q, const float* gamma,
              const float* omega, const float* hx, const float* dh_last, void* dx, float* dp, float* dq,
              float* dgamma, float* domega, float* dhx, float* carry_a, float* carry_b, int B, int L,
              int D, int N, int x_dtype, cudaStream_t st);

// ---- element-wise (elementwise_kernels.cu)
void swiglu_fwd(const void* a, const void* b, void* out, long long n, int dtype, cudaStream_t st);
void silu_bwd(const void* g, const void* a, void* da, long long n, int dtype, cudaStream_t st);
void swiglu_bwd(const void* g, const void* a, const void* b, void* da, void* db, long long n, int dtype,
                cudaStream_t st);
void rotary_apply(const void* x, const float* freqs, void* out, long long rows, int L, int H, int Dh,
                  bool conj, int dtype, cudaStream_t st);
// q, k = rotary(z * (gamma + 1) / sqrt(Dh) + beta) for the two rows of gamma / beta [2, S]; z [rows, S], S = H * Dh a
// multiple of 8 (and at most 8192), position of a row = row % P, freqs [P, Dh / 2] (cos, sin); 16-bit activations
void qk_rotary_fwd(const void* z, const void* gamma, const void* beta, const float* freqs, void* q, void* k,
                   long long rows, int S, int Dh, int P, int dtype, int w_dtype, cudaStream_t st);
int qk_rotary_bwd_ctas(long long rows);
void qk_rotary_bwd(const void* dq, const void* dk, const void* z, const void* gamma, const float* freqs, void* dz,
                   float* partial, long long rows, int S, int Dh, int P, int dtype, int w_dtype, cudaStream_t st);
void cross_entropy_fwd(const void* logits, const long long* target, float* loss, float* lse, long long rows,
                       int V, long long ignore_index, int dtype, cudaStream_t st);
void cross_entropy_bwd(const void* logits, const long long* target, const float* lse, const float* dloss,
                       void* dlogits, long long rows, int V, long long ignore_index, int dtype,
                       cudaStream_t st);
void adamw_step(float* p, const void* g, float* m, float* v, void* low, long long n, float lr, float beta1,
                float beta2, float eps, float wd, int step, float grad_scale, const float* scale_ptr,
                int g_dtype, int low_dtype, cudaStream_t st);
void sum_squares(const void* g, long long n, double* out, int dtype, cudaStream_t st);
void scale_by_ptr(void* g, long long n, const float* scale, int dtype, cudaStream_t st);
void clip_coef(const double* sumsq, float max_norm, float* norm_out, float* coef_out, cudaStream_t st);

// ---- tcgen05 GEMM (gemm_sm100.cu): C[M,N] = act(A B^T + bias)
// lda / ldb / ldc: row strides in elements (multiples of 8).  mode: 0 dense, 1..3 causal tile structure
// (see gemm_sm100.cu).  The result is scaled by alpha before bias / activation.  `batch` independent
// problems of the same shape are addressed through the batch strides a_bs / b_bs / c_bs (elements).
// Operands / results spread over peer GPUs (fused all-gather -> GEMM and GEMM -> reduce-scatter):
//   a_parts > 1: A = [A_0 | A_1 | ...] along K, piece i at a_ptrs[i] (row stride lda, K / a_parts columns
//                each), possibly in a peer's memory; the K walk starts at piece a_first (the local one)
//   c_nparts > 1: column block i of the result (N / c_nparts columns) is stored to c_ptrs[i], laid out
//                [M, N / c_nparts]; nothing is written to C
struct GemmPeerSpec {
  int a_parts = 1, a_first = 0;
  const void* a_ptrs[8] = {};
  int c_nparts = 1;
  void* c_ptrs[8] = {};
};
// Parameter all-gather fused into the GEMM that first consumes the weight (forward of a linear layer,
// B = w [N, K] K-major).  The weight's rows are sharded over `world` ranks in blocks of N / world rows
// (per-parameter FSDP sharding); src[r] is rank r's block - peer memory for r != rank - and dst the local
// full matrix, which must also be the GEMM's B pointer.  Copy warps inside the GEMM kernel pull the blocks
// over NVLink into dst 128 rows at a time while the tensor cores already work on the rows that have
// arrived, starting with the rank's own; every byte crosses the link once, and dst is complete when
// the kernel ends.  `flags`: gemm_gather_flag_words(N) uint32 of device scratch.
struct GemmGatherSpec {
  int world = 0, rank = 0;
  const void* src[8] = {};
  void* dst = nullptr;
  unsigned int* flags = nullptr;
};
// Softmax of chunk-local attention fused into the epilogues of its matrix products (no softmax kernel, the
// logits never leave tensor memory in fp32).  Row vectors are fp32 [batch, M].  With mode == 1, column j of
// row i takes part iff j <= i + causal_off.
//   kind 1: row_out[i] = max(row_out[i], alpha acc[i, :])               nothing stored        (Q K^T, pass 1)
//   kind 2: C = exp(alpha acc - row_in[i]), row_out[i] += sum_j C[i, j]                        (Q K^T, pass 2)
//   kind 3: C = alpha acc / row_in[i]                                                         (P V)
//   kind 4: C = aux / row_in[i] * (alpha acc - row_in2[i]); aux laid out like C, may be C      (dO V^T -> dS)
//   kind 0 with aux: the standard epilogue plus an addend, C = act(alpha acc + bias + aux)     (residual adds)
struct GemmSoftmaxSpec {
  int kind = 0;
  const float* row_in = nullptr;
  const float* row_in2 = nullptr;
  float* row_out = nullptr;
  const void* aux = nullptr;
  int causal_off = 0;
};
bool gemm_gather_supported(int M, int N, int K, int world);
int gemm_gather_flag_words(int N);
int gemm_bf16_tcgen05(const void* A, const void* B, void* C, void* preact, const void* bias, int bias_dtype,
                      int act, int M, int N, int K, long long lda, long long ldb, long long ldc, bool a_mn,
                      bool b_mn, int mode, float alpha, int batch, long long a_bs, long long b_bs, long long c_bs,
                      int in_dtype, int out_dtype, int* err, int num_sms, cudaStream_t st,
                      const GemmPeerSpec* peers = nullptr, bool accumulate = false,
                      const GemmGatherSpec* gather = nullptr, const GemmSoftmaxSpec* softmax = nullptr);
// ---- FFT long convolution (fftconv_kernels.cu); spectra are [rows, N2/2 + 1] complex, N2 = 1 << fftconv_logn(L)
int fftconv_logn(int L);
bool fftconv_supported(int L);          // L <= 16384
// `packed`: -1 choose (packed half-size transform above 8192 samples), 0 plain, 1 packed
void rfft_rows(const void* x, float* out_spec, long long rows, int L, bool flip, int dtype, cudaStream_t st,
               int packed = -1);
void irfft_rows(const float* spec, float* out, long long rows, int L, cudaStream_t st, int packed = -1);
void fftconv_rows(const void* x, const float* kf, void* y, long long rows, int L, int D, bool conj_k, int dtype,
                  cudaStream_t st, int packed = -1);
// the gradient w.r.t. the kernel in one pass; rows of at most 8192 samples (longer: rfft_rows + irfft_rows)
void fftconv_dk(const void* dy, const void* x, float* acc_spec, float* dk, long long rows, int L, int D, int dtype,
                cudaStream_t st);
// y = act(alpha x w^T + bias) for M <= 16 rows of x (gemv_kernels.cu); false if the shapes do not qualify
bool gemv_small_m(const void* x, const void* w, const void* bias, int bias_dtype, void* y, int M, int N, int K,
                  long long ldx, long long ldw, long long ldy, float alpha, int act, int in_dtype, int out_dtype,
                  cudaStream_t st);
// reduce-scatter fused with the sharded AdamW update (comm_kernels.cu); false if the shapes do not qualify
bool reduce_scatter_adamw(const void* const* bufs, int rank, int world, long long shard_n, float scale, float* p,
                          float* m, float* v, void* low, double* sumsq, float lr, float beta1, float beta2, float eps,
                          float wd, int step, int in_dtype, int low_dtype, const int* abort, const long long* table,
                          int npieces, cudaStream_t st);
// Whether GEMMs with more than 128 rows run on CTA pairs (tcgen05 cta_group::2, 256 x 256 tiles); on by default.
void gemm_set_cta_pairs(bool on);
int gemm_pair_max_active_clusters();
// out[i] = sum over `world` slots of slot_w[i] (slots are consecutive, `n` elements each)
void reduce_slots(const void* slots, void* out, long long n, int world, int dtype, cudaStream_t st);

// ---- attention softmax (attention_kernels.cu)
void attn_softmax_fwd(void* s_inout, float* lse, long long rows, int L1, int L2, long long ld, bool causal,
                      float dropkey_p, unsigned long long seed, unsigned long long offset, int dtype,
                      cudaStream_t st);
void attn_softmax_bwd(const void* p, void* dp_inout, long long rows, int L1, int L2, long long ld, bool causal,
                      int dtype, cudaStream_t st);
// one decode step against fixed key / value buffers [BH, C, dk] / [BH, C, dv], keys 0 .. *pos valid (device scalar);
// dk a multiple of 8, 16-bit types; out [BH, dv]
void decode_attention(const void* q, const void* kb, const void* vb, const long long* pos, void* out, int BH, int C,
                      int dk, int dv, float scale, int dtype, cudaStream_t st);
// delta[b, h, l] = dO . O and dO' = dO / rowsum[b, h, l] over rows of dv values (dv a multiple of 8, 16-bit types)
void attn_bwd_prep(const void* dout, const void* out, const float* rowsum, void* dos, float* delta, int B, int L,
                   int H, int dv, int dtype, cudaStream_t st);

// ---- SequenceNorm pieces and dropout (sequence_norm_kernels.cu)
void time_sums(const void* u, const void* v, const bool* mask, float* s1, float* s2, int B, int L, int H,
               bool length_last, int dtype, cudaStream_t st);
void affine_apply(const void* p, const void* q, const float* a, const float* c, const float* d, const bool* mask,
                  void* out, int B, int L, int H, bool length_last, int dtype, cudaStream_t st);
void dropout_apply(const void* x, void* out, long long n, float p, unsigned long long seed,
                   unsigned long long offset, int dtype, cudaStream_t st);

// ---- explicit CEMA kernel / bias (ema_kernels.cu); complex arrays are interleaved fp32
void ema_parameters_fwd(const float* p, const float* logq, const float* gamma, const float* h, float* k,
                        float* bias, int B, int D, int N, int L, cudaStream_t st);
void ema_parameters_bwd(const float* dk, const float* dbias, const float* p, const float* logq, const float* gamma,
                        const float* h, float* dp, float* dq, float* dgamma, float* dh, int B, int D, int N, int L,
                        cudaStream_t st);

// ---- peer-memory communication (comm_kernels.cu); pointers may address a peer GPU's memory.
// `abort` is the device's abort record (kCommAbortWords ints, zero = healthy): the first bounded wait
// that runs out describes itself there, later waits return at once, and peers are released with
// poisoned flags.  `rank` / `dir` / `tag` only label the record.
constexpr int kCommAbortWords = 16;
void p2p_send(const void* src, void* remote_dst, long long nbytes, unsigned int* remote_flag, unsigned int seq,
              const unsigned int* local_ack, unsigned int need_ack, unsigned int* counter,
              unsigned long long timeout_ns, int* abort, int rank, int dir, cudaStream_t st);
// `poison`: overwrite the slot with NaN patterns once it has been read (debug aid, see comm_kernels.cu)
void p2p_recv(void* dst, void* local_slot, long long nbytes, const unsigned int* local_flag, unsigned int seq,
              unsigned int* remote_ack, unsigned int* counter, unsigned long long timeout_ns, int* abort, int rank,
              int dir, bool poison, cudaStream_t st);
// all-reduce (sum) or all-gather along the last dimension of a small 16-bit vector in one kernel whose
// epoch lives in device memory (`counter`), so that it can be captured in a CUDA graph; see the kernel
void small_collective(const void* x, void* out, void* const* bufs, unsigned int* const* pads, unsigned int* counter,
                      int rank, int world, long long nbytes, long long slot_bytes, int rows, bool gather, int dtype,
                      unsigned long long timeout_ns, int* abort, cudaStream_t st);
void peer_barrier(unsigned int* const* pads, int rank, int world, unsigned int epoch, unsigned long long timeout_ns,
                  int* abort, int tag, cudaStream_t st);
// out[i] (+)= scale * sum_p bufs[p][rank * shard_n + i]; out dtype = in dtype or fp32; sumsq += |out|^2
void reduce_scatter_sumsq(const void* const* bufs, int rank, int world, long long shard_n, float scale, void* out,
                          double* sumsq, bool accumulate, int in_dtype, int out_dtype, const int* abort,
                          const long long* table, int npieces, cudaStream_t st);
// `table` (optional, device int64 [npieces, 3] rows (shard_offset, piece, offset)): the staged buffers are in
// natural parameter order and rank r owns piece r of every parameter (per-parameter sharding); without it
// rank r owns the contiguous range [r * shard_n, (r + 1) * shard_n).  At most piece_table_limit() rows.
int piece_table_limit();
// Parameter all-gather by pull: full (natural order) <- piece r of every parameter listed in `table` from
// rank r's shard (peer_shards[r], possibly peer memory), for all r.  `listed_numel` = world * sum of the
// listed pieces (only sizes the grid).  Element size `esize` bytes (2 or 4).  Every computed index is checked
// against `shard_numel` / `full_numel` (elements; <= 0 disables): a bad one is recorded in `abort` (code 30)
// and skipped, never dereferenced.
void gather_pull(void* full, const void* const* peer_shards, int world, const long long* table, int npieces,
                 long long listed_numel, int esize, const int* abort, long long shard_numel, long long full_numel,
                 cudaStream_t st);
void allreduce_sumsq(void* const* bufs, int rank, int world, long long nbytes, float scale, double* sumsq,
                     int dtype, const int* abort, cudaStream_t st);

}  // namespace mb
