// C API of the standalone symmetric-memory collectives (csrc/kernels/symm_coll.cu): all-reduce (one-shot,
// two-shot, in-switch reduction), reduce-scatter, all-gather, all-to-all with per-peer row counts, and the
// vocabulary-parallel arg-max merge. They are the small-message / test counterparts of the collectives that
// the fused GEMM and MoE kernels carry inside them. No counterpart in the reference, which has no
// multi-device communication at all.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>
#include "b2/status.h"
#include "b2/tp.h"

#ifdef __cplusplus
extern "C" {
#endif

struct B2CollLayout {
  int64_t off_buf, buf_half_bytes;  // input that peers read, two halves (launch parity)
  int64_t off_out, out_half_bytes;  // results / received data that peers write, two halves
  int64_t off_flags_a;              // u32 [8]: "my input of epoch e is in place, my previous results are consumed"
  int64_t off_flags_b;              // u32 [8]: "my writes of epoch e into your memory are complete"
  int64_t off_counts;               // u32 [2][8]: rows received from each peer by all-to-all
  int64_t off_done;                 // u32: CTAs of this launch that finished writing (local use)
  int64_t off_epoch;                // u32 [2]: launch epoch + finished-CTA counter (local use)
  int64_t total_bytes;
};

// All sizes in elements of bf16 unless stated; `slot` alternates 0/1 per launch of any of these collectives.
// The input of all_reduce / reduce_scatter must already be in this rank's `buf` half.
// algo: 0 one-shot (every rank reads all peers, result to `out`), 1 two-shot (each rank reduces a slice and writes
// it into every peer's `out` half; result is read there), 2 two-shot through the multicast mapping `mc_base`.
int b2_coll_all_reduce_bf16(const struct B2TpRegion* reg, const struct B2CollLayout* lay, void* mc_base, void* out, int64_t n,
                            int algo, int slot, uint64_t timeout_ns, b2::Status* status, cudaStream_t stream);
// One-shot all-reduce of the [rows, hidden] partials in `buf`, fused with the layer's residual add and RMSNorm:
// residual (bf16 [rows, hidden], may be null) += bf16(sum); out = rmsnorm(residual) * weight. hidden <= 16384.
int b2_coll_all_reduce_rmsnorm_bf16(const struct B2TpRegion* reg, const struct B2CollLayout* lay, void* residual, const void* weight,
                                    void* out, int rows, int hidden, float eps, int slot, uint64_t timeout_ns, b2::Status* status,
                                    cudaStream_t stream);
// The same through the NVLink switch: each rank reduces 1 / tp of the rows with multimem.ld_reduce on the multicast
// mapping `mc_base` and multimem.st's its normalised rows and new residual rows into every rank's `out` half, which
// then holds bf16 [rows, hidden] normalised followed by bf16 [rows, hidden] residual. `residual` (may be null) is
// only read. 2 * rows * hidden * 2 bytes must fit in an `out` half.
int b2_coll_all_reduce_rmsnorm_nvls_bf16(const struct B2TpRegion* reg, const struct B2CollLayout* lay, void* mc_base, const void* residual,
                                         const void* weight, int rows, int hidden, float eps, int slot, uint64_t timeout_ns,
                                         b2::Status* status, cudaStream_t stream);
// out = this rank's n / tp elements of the sum.
int b2_coll_reduce_scatter_bf16(const struct B2TpRegion* reg, const struct B2CollLayout* lay, void* out, int64_t n, int slot,
                                uint64_t timeout_ns, b2::Status* status, cudaStream_t stream);
// Pushes `bytes` (multiple of 16) from `in` (any local memory) into slot [rank] of every peer's `out` half.
int b2_coll_all_gather(const struct B2TpRegion* reg, const struct B2CollLayout* lay, const void* in, int64_t bytes, int slot,
                       uint64_t timeout_ns, b2::Status* status, cudaStream_t stream);
// in: [tp][max_rows][row_bytes] local; rows [0, send_counts[j]) of block j go to peer j's `out` half block [rank];
// the receiver finds the counts at off_counts[slot][src]. row_bytes is a multiple of 16.
int b2_coll_all_to_all(const struct B2TpRegion* reg, const struct B2CollLayout* lay, const void* in, const int* send_counts,
                       int max_rows, int64_t row_bytes, int slot, uint64_t timeout_ns, b2::Status* status, cudaStream_t stream);
// Greedy sampling over a vocabulary split across ranks: `local_idx[s]` is the arg-max of row s of this rank's
// logits shard [S, v_local] (leading dimension ld); tokens[s] = global index of the largest logit over all ranks
// (ties: smallest index); rank r's column c is global index r * v_stride + c. S * tp * 8 bytes must fit in an `out` half.
int b2_coll_vocab_argmax(const struct B2TpRegion* reg, const struct B2CollLayout* lay, const void* logits, int64_t ld,
                         const int64_t* local_idx, int64_t* tokens, int S, int v_local, int v_stride, int slot,
                         uint64_t timeout_ns, b2::Status* status, cudaStream_t stream);

// Link bandwidth probe built from the same peer loads / stores the collectives use: every rank whose bit is set in
// `senders` moves `bytes` (multiple of 16, at most one `buf` half) to (push) or from (pull) each of its next `n_peers`
// ranks, with `ctas` CTAs of 256 threads. The launch returns when every byte has been delivered on every rank.
int b2_coll_p2p_probe(const struct B2TpRegion* reg, const struct B2CollLayout* lay, int64_t bytes, int n_peers, uint32_t senders,
                      int pull, int ctas, int slot, uint64_t timeout_ns, b2::Status* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
