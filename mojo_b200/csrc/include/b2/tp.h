// C API of the fused tensor-parallel kernels (csrc/kernels/tp_fused.cu).
//
// A "region" is one symmetric allocation: the same number of bytes on every rank, each rank holding the device
// addresses at which it can reach every peer's copy. The layout struct says where the staging buffers, gathered
// buffers and flag arrays live inside it; the Python side builds both once per communicator.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>
#include "b2/status.h"

#ifdef __cplusplus
extern "C" {
#endif

struct B2TpRegion {
  int rank, tp;
  void* peer[8];
  void* mc_base;   // multicast (NVLS) mapping of the same region on all ranks, or null: kernels that can reduce in the switch use it
};

struct B2TpLayout {
  int64_t off_staging, staging_half_bytes;  // reduce-scatter staging, two halves (launch parity)
  int64_t off_yall, yall_half_bytes;        // all-reduce result, two halves
  int64_t off_xall, xall_half_bytes;        // all-gather destination, two halves
  int64_t off_rs_flags, rs_flags_bytes;     // u32 [units][tp]
  int64_t off_ag_flags, ag_flags_bytes;     // u32 [tp][chunks]
  int64_t off_res_flags;                    // u32 [8]
  int64_t off_done;                         // u32
  int64_t off_barrier;                      // u32 [8]
  int64_t off_epoch_rs, off_epoch_ag, off_epoch_bar;  // u32 [2] each: launch epoch + finished-CTA counter (local use)
  int64_t total_bytes;
};

// `slot` (0/1) picks the half of each double-buffered area; callers alternate it per launch of an op kind.
// Launch epochs are kept in device memory (see EpochCtl in tp_fused.cu), so the calls can sit in a CUDA graph.
// mode 0: reduce-scatter (out = this rank's M/tp rows, M % tp == 0). mode 1: all-reduce (result in yall half).
int b2_tp_gemm_rs_bf16(const void* x, const void* w, const struct B2TpRegion* reg, const struct B2TpLayout* lay, void* out,
                       const void* residual, int M, int N, int K, int64_t ldx, int64_t ldw, int mode, int slot,
                       uint64_t timeout_ns, int config, b2::Status* status, cudaStream_t stream);
// Same fused reduction with the block-scaled fp8 mainloop (xq/wq e4m3, xs [M, K/128], ws [N/128, K/128] f32 scales).
int b2_tp_gemm_rs_fp8(const void* xq, const float* xs, const void* wq, const float* ws, const struct B2TpRegion* reg,
                      const struct B2TpLayout* lay, void* out, const void* residual, int M, int N, int K, int mode, int slot,
                      uint64_t timeout_ns, b2::Status* status, cudaStream_t stream);
// X rows of this rank must already be in its own xall half at rows [rank * M/tp, (rank + 1) * M/tp).
int b2_tp_ag_gemm_bf16(const void* w, const struct B2TpRegion* reg, const struct B2TpLayout* lay, void* y, int M, int N, int K,
                       int64_t ldw, int64_t ldy, int slot, uint64_t timeout_ns, int n_comm, int config,
                       b2::Status* status, cudaStream_t stream);
// fp8 variant: the gathered half holds e4m3 rows [M][K], then (next 1024-byte boundary) f32 scales [M][K/128].
int b2_tp_ag_gemm_fp8(const void* wq, const float* ws, const struct B2TpRegion* reg, const struct B2TpLayout* lay, void* y, int M, int N,
                      int K, int64_t ldy, int slot, uint64_t timeout_ns, int n_comm, b2::Status* status, cudaStream_t stream);
int b2_tp_all_gather(const struct B2TpRegion* reg, const struct B2TpLayout* lay, int M, int K, int slot,
                     uint64_t timeout_ns, b2::Status* status, cudaStream_t stream);
int b2_symm_barrier(const struct B2TpRegion* reg, const struct B2TpLayout* lay, uint64_t timeout_ns, b2::Status* status,
                    cudaStream_t stream);
// Waits (bounded) for *flag >= want; used by the timeout tests with a flag nobody raises.
int b2_wait_flag(const uint32_t* flag, uint32_t want, uint64_t timeout_ns, b2::Status* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
