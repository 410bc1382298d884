// Allocation-free entry point for the CEMA forward pass.
//
// This entry point has no counterpart in the reference implementation.
//
// Who needs it: code that drives these kernels from a place where device memory
// cannot be allocated - for example a real-time inference loop that must not
// touch the allocator (allocation can synchronise the device and take an
// unbounded time), a host process that was handed a fixed memory budget, or a
// plain C / ctypes caller that has no tensor library to allocate scratch with.
// The regular path (`mb::cema_fwd`) asks its caller for a scratch buffer of
// B * S * N * D complex numbers; here that scratch lives in a fixed array inside
// the library instead, so the caller passes only inputs and outputs.
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Capacity of the built-in scratch array in bytes (32 MiB).  Every GPU on which
// the library is loaded holds this much device memory until the process exits.
#define MB_CEMA_NOALLOC_SCRATCH_BYTES (32u << 20)

// Status codes returned by mb_cema_fwd_noalloc.
#define MB_NOALLOC_OK 0
#define MB_NOALLOC_TOO_LARGE 1        // problem needs more scratch than the built-in array holds
#define MB_NOALLOC_BAD_ARGUMENT 2     // unsupported N / dtype or a null required pointer
#define MB_NOALLOC_CUDA_ERROR 3       // a CUDA runtime call failed (see cudaGetLastError)

// Scratch bytes a problem of this shape needs (0 when the sequence fits one segment).
unsigned long long mb_cema_noalloc_scratch_needed(int B, int L, int D, int N);

// y[B, L, D] = CEMA(x[B, L, D]) with coefficients p[D, N] (fp32), q / gamma
// [D, N] complex as interleaved fp32 pairs, omega[D] (fp32); optional carried
// state hx[B, D, N] complex (may be null); optional output h_last[B, D, N]
// complex (may be null).  `dtype`: 0 = fp32, 1 = bf16, 2 = fp16 activations.
// All pointers are device pointers on the current device; work is enqueued on
// `stream`.
//
// * Allocates nothing: no cudaMalloc / cudaFree, no library allocator.
// * Shapes whose scratch need exceeds MB_CEMA_NOALLOC_SCRATCH_BYTES are
//   rejected with MB_NOALLOC_TOO_LARGE and nothing is launched.
// * The first call on each device looks up the device address of the scratch
//   array (cudaGetSymbolAddress).  Make that first call before starting any
//   stream capture on that device.
// * All calls on one device share the one scratch array, which keeps whatever
//   the previous call left in it (this operator overwrites every element it
//   later reads, so nothing needs clearing).  Two calls whose kernels can
//   overlap on the GPU - different streams without an ordering between them -
//   race on it; serialise them.
int mb_cema_fwd_noalloc(const void* x, const float* p, const float* q, const float* gamma, const float* omega,
                        const float* hx, void* y, float* h_last, int B, int L, int D, int N, int dtype,
                        cudaStream_t stream);

#ifdef __cplusplus
}
#endif
