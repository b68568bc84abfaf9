// C launch API of the sm_100a kernel library.
//
// Every kernel is reachable through a plain C function taking raw device pointers and a stream, so the
// library can be driven from the PyTorch bindings, from ctypes, or from another C++ runtime. All
// functions return 0 on success or a negative b2::StatusCode for rejected arguments; device-side
// problems are reported through the `b2::Status*` word passed in (may be null).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>
#include "b2/status.h"

#ifdef __cplusplus
extern "C" {
#endif

// ---- elementwise / normalisation ---------------------------------------------------------------
// out = rmsnorm(x (+ residual)) * weight. If `residual` is non-null it is updated in place to x + residual.
// If `q_out`/`q_scale` are non-null the normalised row is also emitted as e4m3 with one f32 scale per
// 128 columns (dynamic activation quantisation for the fp8 GEMM).
int b2_rmsnorm_bf16(const void* x, void* residual, const void* weight, void* out, void* q_out, float* q_scale,
                    int rows, int hidden, float eps, cudaStream_t stream);
// Per-row 1x128 e4m3 quantisation of a bf16 matrix: q[r, c] = x[r, c] / s[r, c/128], s = amax/448.
int b2_quant_e4m3_1x128(const void* x, void* q_out, float* scale_out, int rows, int cols, cudaStream_t stream);
// Rotary embedding on q and k (in place) + scatter of k, v into the paged cache.
// q: [T, n_q, D] with row stride q_stride (elements); k, v likewise. cos_sin: f32 [max_pos, rot_dim]
// (cos in the first half of a row, sin in the second). slot < 0 skips the cache write.
// cache layout: [num_pages, n_kv, page_size, D].
int b2_rope_kvwrite_bf16(void* q, void* k, const void* v, const float* cos_sin, const int32_t* positions,
                         const int64_t* slots, void* k_cache, void* v_cache, int tokens, int n_q, int n_kv,
                         int head_dim, int rot_dim, int interleaved, int64_t q_stride, int64_t k_stride,
                         int64_t v_stride, int page_size, int64_t num_slots, int max_pos, b2::Status* status,
                         cudaStream_t stream);
// out[t, j] = silu(gate_up[t, j]) * gate_up[t, F + j]
int b2_swiglu_bf16(const void* gate_up, void* out, int rows, int ffn, int interleaved, cudaStream_t stream);
// out[t, :] = table[ids[t] - vocab_start, :] for ids inside [vocab_start, vocab_start + vocab_rows), else 0.
// tok[rows[i]] = prev[src[i]], i < n (int32 row / source indices, int64 token ids): feeds the tokens sampled by the
// previous step straight into the next step's input while the host is still one step behind.
int b2_patch_tokens(int64_t* tok, const int32_t* rows, const int32_t* src, const int64_t* prev, int n, int64_t tok_rows,
                    int64_t prev_rows, b2::Status* status, cudaStream_t stream);
int b2_embedding_bf16(const int64_t* ids, const void* table, void* out, int tokens, int hidden, int64_t vocab_start,
                      int64_t vocab_rows, cudaStream_t stream);
// out[i, :] = src[index[i], :] (row gather, 16-byte vectorised; used for last-token selection).
int b2_gather_rows_bf16(const void* src, const int64_t* index, void* out, int rows_out, int cols, int64_t rows_src,
                        b2::Status* status, cudaStream_t stream);
// dst[slots[i], :] = src[i, :] for slots[i] >= 0 (negative slots are padding and skipped).
int b2_scatter_rows_bf16(const void* src, const int64_t* slots, void* dst, int rows, int cols, int64_t rows_dst,
                         b2::Status* status, cudaStream_t stream);
// Copy whole KV pages inside a cache tensor: dst_page[i] <- src_page[i] (preemption swap / prefix share).
int b2_copy_pages(void* cache, const int64_t* src_pages, const int64_t* dst_pages, int n, int64_t page_bytes,
                  int64_t num_pages, b2::Status* status, cudaStream_t stream);

// ---- sampling ----------------------------------------------------------------------------------
// Greedy: ids[r] = argmax_j logits[r, j] (lowest index on ties); also writes the max value.
int b2_argmax(const void* logits, int is_bf16, int64_t* ids, float* max_out, int rows, int vocab, int64_t row_stride,
              cudaStream_t stream);
// Temperature / top-k / top-p sampling. Per-row parameters; top_k <= 0 disables, top_p >= 1 disables,
// temperature == 0 means greedy. u = Philox4x32-10(seed, row, step) unless `uniforms` is given.
int b2_sample(const void* logits, int is_bf16, int64_t* ids, const float* temperature, const int32_t* top_k,
              const float* top_p, const float* uniforms, uint64_t seed, uint64_t step, int rows, int vocab,
              int64_t row_stride, cudaStream_t stream);

// ---- attention ---------------------------------------------------------------------------------
// Causal GQA attention over a paged KV cache for a ragged batch of query chunks.
// q/out: [T, n_q, D]; cache: [num_pages, n_kv, page_size, D]; cu_q: [B+1] query offsets; ctx_lens: [B]
// total context (cached prefix + this chunk); block_tables: [B, max_blocks]. D == 128 or 64.
int b2_attn_prefill_bf16(const void* q, const void* k_cache, const void* v_cache, void* out, const int32_t* cu_q,
                         const int32_t* ctx_lens, const int32_t* block_tables, int batch, int max_blocks, int n_q,
                         int n_kv, int head_dim, int page_size, int max_q_len, float scale, int64_t q_stride,
                         int64_t out_stride, int64_t num_pages, b2::Status* status, cudaStream_t stream);
// bf16 GEMM on CTA pairs (tcgen05 cta_group::2, 256 x 256 tiles; csrc/kernels/gemm_bf16_pair.cu). Epilogue NONE or SWIGLU.
int b2_gemm_bf16_pair(const void* x, const void* w, void* y, int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldy,
                      int epilogue, int bn, b2::Status* status, cudaStream_t stream);
// The same attention on tcgen05 / TMEM (csrc/kernels/attention_tc.cu): head_dim 128 and page_size 128 only.
// q_rows = rows of the q matrix (for the tensor map); variant = descriptor variant of the V operand (0 = default).
int b2_attn_prefill_tc_bf16(const void* q, const void* k_cache, const void* v_cache, void* out, const int32_t* cu_q,
                            const int32_t* ctx_lens, const int32_t* block_tables, int batch, int max_blocks, int n_q,
                            int n_kv, int max_q_len, float scale, int64_t q_rows, int64_t q_stride, int64_t out_stride,
                            int64_t num_pages, int variant, const int32_t* work, const int32_t* n_work, int work_items,
                            b2::Status* status, cudaStream_t stream);
// One query token per sequence, split over the KV length. workspace: f32, size from b2_attn_decode_workspace.
// `counters` (may be null): u32 [batch * n_kv], zero before the first use and left at zero by every launch; with it
// (and page sizes that are multiples of 32) the split that finishes last merges the partials itself, otherwise a
// second small kernel does.
int b2_attn_decode_bf16(const void* q, const void* k_cache, const void* v_cache, void* out, const int32_t* ctx_lens,
                        const int32_t* block_tables, float* workspace, int batch, int max_blocks, int n_q, int n_kv,
                        int head_dim, int page_size, int num_splits, float scale, int64_t q_stride,
                        int64_t out_stride, int64_t num_pages, uint32_t* counters, b2::Status* status, cudaStream_t stream);
int64_t b2_attn_decode_counter_bytes(int batch, int n_kv);
int64_t b2_attn_decode_workspace(int batch, int n_q, int head_dim, int num_splits);
// MLA decode with absorbed weights: q_lat [B, H, 512], q_rope [B, H, 64]; cache [num_pages, page, 576]
// (512 latent + 64 rope); out_lat [B, H, 512].
int b2_mla_decode_bf16(const void* q_lat, const void* q_rope, const void* kv_cache, void* out_lat,
                       const int32_t* ctx_lens, const int32_t* block_tables, float* workspace, int batch,
                       int max_blocks, int n_heads, int page_size, int num_splits, float scale, int64_t num_pages,
                       b2::Status* status, cudaStream_t stream);
int64_t b2_mla_decode_workspace(int batch, int n_heads, int num_splits);
// The same kernel over arbitrary query rows (decode tokens and the tokens of prefill chunks in one launch): row r
// reads q_lat + r * q_lat_stride and q_rope + r * q_rope_stride (element strides, multiples of 8), sees the first
// row_ctx[r] cache positions of sequence row_seq[r] (row r itself when row_seq is null) and writes out_lat [rows, H, 512].
int b2_mla_attend_bf16(const void* q_lat, const void* q_rope, const void* kv_cache, void* out_lat, const int32_t* row_ctx,
                       const int32_t* block_tables, const int32_t* row_seq, float* workspace, int rows, int max_blocks,
                       int n_heads, int page_size, int num_splits, float scale, int64_t num_pages, int64_t q_lat_stride,
                       int64_t q_rope_stride, b2::Status* status, cudaStream_t stream);
// row_ctx[t] / row_seq[t] for every token t of a batch described by cu_q [num_seqs + 1] and ctx_lens [num_seqs]:
// token i of a sequence's chunk sees ctx - q_len + i + 1 positions (causal mask of chunked prefill; decode rows: ctx).
int b2_mla_rows_meta(const int32_t* cu_q, const int32_t* ctx_lens, int num_seqs, int32_t* row_ctx, int32_t* row_seq,
                     cudaStream_t stream);

// ---- GEMM (tcgen05 / TMEM / TMA) ---------------------------------------------------------------
// Epilogue selector for the tcgen05 GEMMs.
enum B2Epilogue { B2_EPI_NONE = 0, B2_EPI_ADD_RESIDUAL = 1, B2_EPI_SWIGLU = 2 };
// Y[M, N] = X[M, K] * W[N, K]^T (+ residual), bf16 in, f32 accumulate, bf16 out.
// ldx/ldw/ldy are row strides in elements. `workspace`/`counters` are split-K scratch (may be null when
// the chosen configuration does not split); sizes from b2_gemm_workspace_bytes.
int b2_gemm_bf16(const void* x, const void* w, void* y, const void* residual, int M, int N, int K, int64_t ldx,
                 int64_t ldw, int64_t ldy, int epilogue, int config, void* workspace, int64_t workspace_bytes,
                 b2::Status* status, cudaStream_t stream);
int64_t b2_gemm_workspace_bytes(int M, int N, int K);
// fp8 block-scaled: X e4m3 [M, K] with f32 scales [M, K/128]; W e4m3 [N, K] with f32 scales [N/128, K/128].
int b2_gemm_fp8_block(const void* xq, const float* xs, const void* wq, const float* ws, void* y, int M, int N, int K,
                      int64_t ldy, int config, b2::Status* status, cudaStream_t stream);
// The same with a split-K workspace (layout and size rule of the bf16 GEMM's: 256 KiB of zeroed per-tile semaphores,
// then f32 partial tiles). config bits 16..23 = split count; config 0 splits K when the tiles alone would leave
// half of the SMs idle (decode-sized M against a narrow tensor-parallel weight shard).
int b2_gemm_fp8_block_ws(const void* xq, const float* xs, const void* wq, const float* ws, void* y, int M, int N, int K,
                         int64_t ldy, int config, void* workspace, int64_t workspace_bytes, b2::Status* status,
                         cudaStream_t stream);
// GGUF: W stored as Q4_K (type 12) or Q6_K (type 14) super-blocks, row-major [N, K/256 blocks].
int b2_gemm_gguf(const void* x, const void* wq, int ggml_type, void* y, int M, int N, int K, b2::Status* status,
                 cudaStream_t stream);
int b2_dequant_gguf(const void* wq, int ggml_type, void* out_bf16, int64_t n_elems, cudaStream_t stream);

// ---- device capability probe -------------------------------------------------------------------
struct B2DeviceCaps {
  int cc_major, cc_minor, sm_count, smem_per_block_optin, l2_bytes, max_cluster;
  int64_t total_mem;
  int can_map_peer, multicast_supported, clock_khz, mem_clock_khz;
  char name[128];
};
int b2_device_caps(int device, struct B2DeviceCaps* out);

#ifdef __cplusplus
}
#endif
