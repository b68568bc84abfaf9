// Split-K bf16 GEMM for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference; it exists for hosts of this library that cannot call
// cudaMalloc themselves and cannot let a library do it for them: code running while a CUDA graph is being
// captured, real-time serving loops that forbid allocator traffic after start-up, and plugins living inside
// another runtime's memory pool. The regular entry point (b2_gemm_bf16) needs a caller-supplied workspace for
// its split-K partial sums; here that workspace is a fixed array compiled into the library.
//
//   Y[M, N] = X[M, K] * W[N, K]^T      bf16 in, f32 accumulate, bf16 out, row strides in elements.
//
// Limits and rules:
//   * The scratch is B2_NOALLOC_SCRATCH_BYTES (8 MiB) per GPU, resident from the moment the library is loaded on
//     that GPU until the process exits. A problem whose split-K partials need more is rejected with
//     -b2::kTooLarge before anything is launched; nothing is ever allocated as a fallback.
//   * The first call on each device looks up the array's device address (cudaGetSymbolAddress) and clears its
//     semaphore words. Make that first call outside any stream capture; later calls only launch the kernel.
//     That first call may come from several host threads at once (the set-up is serialised by a mutex).
//   * All calls on a device share the one array. Calls that may overlap on the GPU (different streams without an
//     ordering between them) race on it; keep them on one stream or order them with events.
//   * The semaphore words are returned to zero by every launch, and partial sums are fully rewritten before they
//     are read, so stale contents from the previous call are harmless.
//   * The call returns as soon as the kernel is queued, so it cannot tell whether a bounded wait inside the kernel
//     ran out. `b2_gemm_bf16_noalloc_status(stream)` can: it waits for `stream`, returns 0 or the negative
//     b2::StatusCode a kernel of this entry point recorded on the current device since the last query (-kTimeout),
//     and after such a failure puts the semaphore words back to zero so later calls count correctly. It copies
//     32 bytes to the host and allocates nothing.
// Returns 0, a negative b2::StatusCode (kBadArgument, kTooLarge), or -(1000 + cudaError_t) if the CUDA runtime
// refused the launch or the one-time set-up (b2/launch.h).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

#define B2_NOALLOC_SCRATCH_BYTES (8 * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

int b2_gemm_bf16_noalloc(const void* x, const void* w, void* y, int M, int N, int K, int64_t ldx, int64_t ldw,
                         int64_t ldy, cudaStream_t stream);
int b2_gemm_bf16_noalloc_status(cudaStream_t stream);

#ifdef __cplusplus
}
#endif
