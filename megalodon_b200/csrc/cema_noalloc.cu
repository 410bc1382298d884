// Allocation-free CEMA forward: the segmented-scan kernels of cema_kernels.cu
// run with their carry buffer in a file-scope device array instead of a
// caller-allocated tensor.  See cema_noalloc.h for the contract.
#include "cema_noalloc.h"

#include <mutex>

#include "kernels.h"

namespace {

// The scratch itself.  In host code this name is only a handle for the runtime
// (it is not a device address); the address the kernels need is obtained per
// device with cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_cema_scratch[MB_CEMA_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
float* g_scratch_ptr[kMaxDevices] = {};   // device address of g_cema_scratch, per device

// Device address of the scratch array on the current device (looked up once per device).
int scratch_for_current_device(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return MB_NOALLOC_CUDA_ERROR;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_cema_scratch) != cudaSuccess || ptr == nullptr) return MB_NOALLOC_CUDA_ERROR;
    g_scratch_ptr[dev] = static_cast<float*>(ptr);
  }
  *out = g_scratch_ptr[dev];
  return MB_NOALLOC_OK;
}

}  // namespace

extern "C" unsigned long long mb_cema_noalloc_scratch_needed(int B, int L, int D, int N) {
  if (B <= 0 || L <= 0 || D <= 0 || N <= 0) return 0;
  const int S = mb::cema_num_segments(L);
  if (S <= 1) return 0;
  return (unsigned long long)B * S * N * D * 2ull * sizeof(float);
}

extern "C" int mb_cema_fwd_noalloc(const void* x, const float* p, const float* q, const float* gamma,
                                   const float* omega, const float* hx, void* y, float* h_last, int B, int L,
                                   int D, int N, int dtype, cudaStream_t stream) {
  if (x == nullptr || p == nullptr || q == nullptr || gamma == nullptr || omega == nullptr || y == nullptr)
    return MB_NOALLOC_BAD_ARGUMENT;
  if (B <= 0 || L <= 0 || D <= 0 || !mb::cema_supported_ndim(N) || dtype < 0 || dtype > 2)
    return MB_NOALLOC_BAD_ARGUMENT;
  if (mb_cema_noalloc_scratch_needed(B, L, D, N) > MB_CEMA_NOALLOC_SCRATCH_BYTES) return MB_NOALLOC_TOO_LARGE;
  float* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != MB_NOALLOC_OK) return rc;
  mb::cema_fwd(x, p, q, gamma, omega, hx, y, h_last, scratch, B, L, D, N, dtype, stream);
  return cudaGetLastError() == cudaSuccess ? MB_NOALLOC_OK : MB_NOALLOC_CUDA_ERROR;
}
