// C API of the expert-parallel MoE kernels (csrc/kernels/moe_ep.cu).
//
// One symmetric region per rank (see b2/tp.h for B2TpRegion) laid out as described by B2EpLayout:
//   recv_x      bf16 [e_local][cap][hidden]   rows dispatched to this rank, packed densely per local expert
//   recv_meta   i32  [e_local][cap]           (source rank << 24) | (token * top_k + k) for each received row
//   recv_count  u32  [2][e_local]             rows received per expert; two banks alternate per layer (`slot`),
//                                             the dispatch kernel clears the bank of the *next* launch
//   ret_y       bf16 [t_cap * top_k][hidden]  expert outputs returned to the rank that owns the token
//   disp_done / comb_done  u32 [8]            per-source epoch flags
//   epoch       u32 [8]                       launch epochs and CTA counters (device-resident: graph replay safe)
#pragma once
#include <cstdint>
#include <cuda_runtime.h>
#include "b2/status.h"
#include "b2/tp.h"

#ifdef __cplusplus
extern "C" {
#endif

struct B2EpLayout {
  int64_t off_recv_x, off_recv_meta, off_recv_count, off_ret_y, off_disp_done, off_comb_done, off_epoch, total_bytes;
  int cap, e_local, hidden, top_k, t_cap;
};

// Router (softmax + top-k over `E` logits per token, optional renormalisation, scaling) fused with the token
// permutation and the all-to-all: writes weights_out/ids_out [T, top_k] and fills the owners' receive buffers.
int b2_ep_dispatch(const void* x, const void* logits, float* weights_out, int32_t* ids_out, const struct B2TpRegion* reg,
                   const struct B2EpLayout* lay, int T, int E, int top_k, int norm_topk, float route_scale, int slot,
                   uint64_t timeout_ns, b2::Status* status, cudaStream_t stream);
// y[e][m][:] = x[e][m][:] W[e]^T for m < counts[e]; x [e_local * cap, K], w [e_local * N, K], optional SwiGLU epilogue
// (w rows interleaved gate/up in blocks of 16, y then has N / 2 columns).
int b2_moe_grouped_gemm(const void* x, const void* w, const uint32_t* counts, void* y, int e_local, int cap, int N, int K,
                        int64_t ldy, int swiglu, int bn, b2::Status* status, cudaStream_t stream);
// out[t] = sum_k weights[t, k] * expert_out(t, k) (+ shared[t]); y_local [e_local][cap][hidden] is this rank's output.
int b2_ep_combine(const void* y_local, const float* weights, const void* shared, void* out, const struct B2TpRegion* reg,
                  const struct B2EpLayout* lay, int T, int top_k, int slot, uint64_t timeout_ns, b2::Status* status,
                  cudaStream_t stream);

#ifdef __cplusplus
}
#endif
