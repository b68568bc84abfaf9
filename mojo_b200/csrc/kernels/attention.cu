// Paged GQA attention: causal chunked prefill and split-KV decode.
//
// Both kernels pack the query heads that share one KV head into the row dimension of the MMA tile
// (row = token * group + head_in_group), so a K/V tile fetched from the paged cache is used by the whole
// group. Softmax is the online form in f32 with exp(x) = 2^(x * log2e) and the scale folded into the
// exponent argument, the rewrite the reference applies to `exp` on NVIDIA targets
// (stdlib/src/math/math.mojo:577-582 with ex2.approx at :373-401).
//
// Tensor-core path: warp-level mma.sync m16n8k16 (bf16 in, f32 accumulate) fed by ldmatrix from XOR-swizzled
// shared memory that cp.async fills page by page. Decode is bandwidth-bound, so its four warps stream
// disjoint KV tiles through warp-private double buffers and merge their partial softmax states at the end.
#include <cstdint>
#include <cuda_bf16.h>
#include "b2/api.h"
#include "b2/launch.h"
#include "b2/ptx.cuh"
#include "b2/tma.h"
#include "b2/vec.cuh"

namespace b2 {
namespace {

__device__ __forceinline__ void cp_async_16(uint32_t smem, const void* gmem, bool valid) {
  const int sz = valid ? 16 : 0;  // src-size 0 => 16 bytes of zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem), "l"(gmem), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                                  uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Shared-memory tile of bf16 in 16-byte chunks. Two layouts:
//   ROWS == 0  [rows][D], chunk index XOR-swizzled by (row & 7)              (filled by cp.async)
//   ROWS  > 0  D/64 sub-tiles of [ROWS][64] with 128-byte rows and the 128-byte TMA swizzle: exactly what a
//              SWIZZLE_128B box of 64 columns x ROWS rows leaves in shared memory (base 1024-byte aligned)
template <int D, int ROWS = 0>
__device__ __forceinline__ uint32_t tile_addr(uint32_t base, int row, int chunk) {
  if constexpr (ROWS == 0) {
    constexpr int CPR = D / 8;  // chunks per row
    return base + static_cast<uint32_t>((row * CPR + (chunk ^ (row & 7))) * 16);
  } else {
    return base + static_cast<uint32_t>((chunk >> 3) * (ROWS * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
  }
}

struct PagedKV {
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  const int32_t* table;  // block table of this sequence
  int n_kv, kvh, page_size, ctx_len;
  int64_t num_pages;
};

// Stage `ROWS` consecutive KV positions starting at kv0 into swizzled tiles (K and V) using `NT` threads.
template <int D, int ROWS, int NT>
__device__ __forceinline__ void load_kv_tile(const PagedKV& kv, int kv0, uint32_t k_sm, uint32_t v_sm, int tid,
                                             Status* status) {
  constexpr int CPR = D / 8;
  constexpr int TOTAL = ROWS * CPR;
#pragma unroll
  for (int i = tid; i < TOTAL; i += NT) {
    const int row = i / CPR, chunk = i % CPR;
    const int pos = kv0 + row;
    bool valid = pos < kv.ctx_len;
    int64_t page = 0;
    if (valid) {
      page = kv.table[pos / kv.page_size];
      if (!B2_ASSERT(status, page >= 0 && page < kv.num_pages, kSiteKvIndex, page, kv.num_pages)) {
        valid = false;
        page = 0;
      }
    }
    const int64_t off = ((page * kv.n_kv + kv.kvh) * kv.page_size + (valid ? pos % kv.page_size : 0)) * D + chunk * 8;
    cp_async_16(tile_addr<D>(k_sm, row, chunk), kv.k + off, valid);
    cp_async_16(tile_addr<D>(v_sm, row, chunk), kv.v + off, valid);
  }
}

// One warp: S = Q K^T on a BN-token tile, online softmax, O += P V.
//   qf      Q fragments of this warp's 16 rows (D/16 k-steps x 4 regs)
//   max_lo  highest KV position visible to row g, max_hi to row g + 8 (causal + context limit)
template <int D, int BN, int TROWS = 0>
__device__ __forceinline__ void warp_attend(const uint32_t (&qf)[D / 16][4], uint32_t k_sm, uint32_t v_sm, int kv0,
                                            int max_lo, int max_hi, float scale_log2, float (&o)[D / 8][4],
                                            float (&m)[2], float (&l)[2], int lane) {
  constexpr int NT_S = BN / 8;
  float s[NT_S][4];
#pragma unroll
  for (int j = 0; j < NT_S; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
    for (int jp = 0; jp < NT_S / 2; ++jp) {
      uint32_t b0, b1, b2, b3;
      const int row = jp * 16 + (lane & 7) + ((lane >> 4) << 3);
      const int chunk = kk * 2 + ((lane >> 3) & 1);
      ldmatrix_x4(tile_addr<D, TROWS>(k_sm, row, chunk), b0, b1, b2, b3);
      mma_bf16(s[2 * jp], qf[kk], b0, b1);
      mma_bf16(s[2 * jp + 1], qf[kk], b2, b3);
    }
  }
  // mask + running max
  const int t = lane & 3;
  float mx_lo = m[0], mx_hi = m[1];
#pragma unroll
  for (int j = 0; j < NT_S; ++j) {
    const int col = kv0 + j * 8 + 2 * t;
    s[j][0] = col <= max_lo ? s[j][0] * scale_log2 : -INFINITY;
    s[j][1] = col + 1 <= max_lo ? s[j][1] * scale_log2 : -INFINITY;
    s[j][2] = col <= max_hi ? s[j][2] * scale_log2 : -INFINITY;
    s[j][3] = col + 1 <= max_hi ? s[j][3] * scale_log2 : -INFINITY;
    mx_lo = fmaxf(mx_lo, fmaxf(s[j][0], s[j][1]));
    mx_hi = fmaxf(mx_hi, fmaxf(s[j][2], s[j][3]));
  }
  mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
  mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
  mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
  mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
  // rows that have seen nothing yet keep m = -inf; use 0 as the subtrahend so exp2 gives 0, not NaN
  const float sub_lo = mx_lo == -INFINITY ? 0.0f : mx_lo;
  const float sub_hi = mx_hi == -INFINITY ? 0.0f : mx_hi;
  const float corr_lo = ptx::ex2(m[0] - sub_lo), corr_hi = ptx::ex2(m[1] - sub_hi);
  m[0] = mx_lo;
  m[1] = mx_hi;
  float sum_lo = 0.0f, sum_hi = 0.0f;
  uint32_t pf[NT_S][2];
#pragma unroll
  for (int j = 0; j < NT_S; ++j) {
    const float p0 = ptx::ex2(s[j][0] - sub_lo), p1 = ptx::ex2(s[j][1] - sub_lo);
    const float p2 = ptx::ex2(s[j][2] - sub_hi), p3 = ptx::ex2(s[j][3] - sub_hi);
    sum_lo += p0 + p1;
    sum_hi += p2 + p3;
    pf[j][0] = ptx::pack_bf16x2(p0, p1);
    pf[j][1] = ptx::pack_bf16x2(p2, p3);
  }
  l[0] = l[0] * corr_lo + sum_lo;
  l[1] = l[1] * corr_hi + sum_hi;
#pragma unroll
  for (int d = 0; d < D / 8; ++d) {
    o[d][0] *= corr_lo; o[d][1] *= corr_lo;
    o[d][2] *= corr_hi; o[d][3] *= corr_hi;
  }
#pragma unroll
  for (int kk = 0; kk < BN / 16; ++kk) {
    const uint32_t a[4] = {pf[2 * kk][0], pf[2 * kk][1], pf[2 * kk + 1][0], pf[2 * kk + 1][1]};
#pragma unroll
    for (int dp = 0; dp < D / 16; ++dp) {
      uint32_t b0, b1, b2, b3;
      const int row = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
      const int chunk = dp * 2 + (lane >> 4);
      ldmatrix_x4_trans(tile_addr<D, TROWS>(v_sm, row, chunk), b0, b1, b2, b3);
      mma_bf16(o[2 * dp], a, b0, b1);
      mma_bf16(o[2 * dp + 1], a, b2, b3);
    }
  }
}

// Load this warp's 16 packed query rows into fragments. Row r -> (token = r / group, head = r % group).
template <int D>
__device__ __forceinline__ void load_q_frags(const __nv_bfloat16* q, int64_t q_stride, int tok0, int n_tok, int group,
                                             int kvh, int row0, uint32_t q_sm, uint32_t (&qf)[D / 16][4], int lane) {
  constexpr int CPR = D / 8;
  // warp-private staging: 16 rows x D
  for (int i = lane; i < 16 * CPR; i += 32) {
    const int r = i / CPR, chunk = i % CPR;
    const int pr = row0 + r;
    const int tok = pr / group, hg = pr % group;
    const bool valid = tok < n_tok;
    const __nv_bfloat16* src = q + static_cast<int64_t>(tok0 + (valid ? tok : 0)) * q_stride +
                               static_cast<int64_t>(kvh * group + hg) * D + chunk * 8;
    cp_async_16(tile_addr<D>(q_sm, r, chunk), src, valid);
  }
  cp_async_commit();
  cp_async_wait<0>();
  __syncwarp();
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    const int row = lane & 15, chunk = kk * 2 + (lane >> 4);
    ldmatrix_x4(tile_addr<D>(q_sm, row, chunk), qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
  }
  __syncwarp();
}

// ------------------------------------------------------------------------------------------------
// Prefill: CTA = 4 warps x 16 packed rows = 64 rows; KV tiles of 64 tokens, double buffered, shared by
// the four warps.
// ------------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(128) attn_prefill_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
    const __nv_bfloat16* __restrict__ v_cache, __nv_bfloat16* __restrict__ out, const int32_t* __restrict__ cu_q,
    const int32_t* __restrict__ ctx_lens, const int32_t* __restrict__ block_tables, int max_blocks, int n_q, int n_kv,
    int page_size, float scale_log2, int64_t q_stride, int64_t out_stride, int64_t num_pages, Status* status) {
  ptx::grid_dep_sync();
  constexpr int BM = 64, BN = 64;
  constexpr int TILE_BYTES = BN * D * 2;
  extern __shared__ __align__(128) uint8_t smem[];
  const int seq = blockIdx.z, kvh = blockIdx.y;
  const int group = n_q / n_kv;
  const int tok0 = cu_q[seq];
  const int q_len = cu_q[seq + 1] - tok0;
  const int ctx = ctx_lens[seq];
  const int row_base = blockIdx.x * BM;
  if (row_base >= q_len * group) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t sbase = ptx::smem_u32(smem);
  const uint32_t q_sm = sbase + warp * (16 * D * 2);
  const uint32_t kv_sm = sbase + 4 * (16 * D * 2);  // [2 stages][K, V]

  PagedKV kv{k_cache, v_cache, block_tables + static_cast<int64_t>(seq) * max_blocks, n_kv, kvh, page_size, ctx, num_pages};

  uint32_t qf[D / 16][4];
  const int row0 = row_base + warp * 16;
  load_q_frags<D>(q, q_stride, tok0, q_len, group, kvh, row0, q_sm, qf, lane);

  const int g = lane >> 2;
  const int past = ctx - q_len;  // tokens already in the cache before this chunk
  const int tok_lo = (row0 + g) / group, tok_hi = (row0 + g + 8) / group;
  const int max_lo = tok_lo < q_len ? past + tok_lo : -1;
  const int max_hi = tok_hi < q_len ? past + tok_hi : -1;
  // the CTA needs KV positions [0, last visible position of its last row]
  const int last_tok = min(q_len - 1, (row_base + BM - 1) / group);
  const int kv_end = min(ctx, past + last_tok + 1);
  const int n_tiles = (kv_end + BN - 1) / BN;

  float o[D / 8][4];
#pragma unroll
  for (int d = 0; d < D / 8; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.0f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};

  if (n_tiles > 0) {
    load_kv_tile<D, BN, 128>(kv, 0, kv_sm, kv_sm + TILE_BYTES, threadIdx.x, status);
    cp_async_commit();
  }
  for (int t = 0; t < n_tiles; ++t) {
    const int stage = t & 1;
    if (t + 1 < n_tiles) {
      const uint32_t nb = kv_sm + (stage ^ 1) * 2 * TILE_BYTES;
      load_kv_tile<D, BN, 128>(kv, (t + 1) * BN, nb, nb + TILE_BYTES, threadIdx.x, status);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint32_t kb = kv_sm + stage * 2 * TILE_BYTES;
    // a warp whose rows cannot see this tile yet skips the math (causal upper triangle)
    const int warp_max = min(q_len - 1, (row0 + 15) / group) + past;
    if (t * BN <= warp_max && row0 < q_len * group)
      warp_attend<D, BN>(qf, kb, kb + TILE_BYTES, t * BN, max_lo, max_hi, scale_log2, o, m, l, lane);
    __syncthreads();
  }
  // finalise: O / l
  l[0] += __shfl_xor_sync(0xffffffffu, l[0], 1);
  l[0] += __shfl_xor_sync(0xffffffffu, l[0], 2);
  l[1] += __shfl_xor_sync(0xffffffffu, l[1], 1);
  l[1] += __shfl_xor_sync(0xffffffffu, l[1], 2);
  const float inv_lo = l[0] > 0.0f ? 1.0f / l[0] : 0.0f, inv_hi = l[1] > 0.0f ? 1.0f / l[1] : 0.0f;
  const int t4 = lane & 3;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int pr = row0 + g + half * 8;
    const int tok = pr / group, hg = pr % group;
    if (tok >= q_len) continue;
    __nv_bfloat16* dst = out + static_cast<int64_t>(tok0 + tok) * out_stride + static_cast<int64_t>(kvh * group + hg) * D;
    const float inv = half ? inv_hi : inv_lo;
#pragma unroll
    for (int d = 0; d < D / 8; ++d) {
      const uint32_t pk = ptx::pack_bf16x2(o[d][half * 2] * inv, o[d][half * 2 + 1] * inv);
      *reinterpret_cast<uint32_t*>(dst + d * 8 + 2 * t4) = pk;
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Decode: CTA = (split, kv head, sequence); 4 warps stream disjoint 32-token tiles of the split's KV
// range through warp-private double buffers; rows = the `group` query heads (<= 16).
// ------------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(128) attn_decode_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
    const __nv_bfloat16* __restrict__ v_cache, __nv_bfloat16* __restrict__ out, const int32_t* __restrict__ ctx_lens,
    const int32_t* __restrict__ block_tables, float* __restrict__ workspace, int max_blocks, int n_q, int n_kv,
    int page_size, int num_splits, float scale_log2, int64_t q_stride, int64_t out_stride, int64_t num_pages,
    Status* status) {
  ptx::grid_dep_sync();
  constexpr int BN = 32;
  constexpr int TILE_BYTES = BN * D * 2;
  extern __shared__ __align__(128) uint8_t smem[];
  const int split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
  const int group = n_q / n_kv;
  const int ctx = ctx_lens[seq];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t sbase = ptx::smem_u32(smem);
  // per warp: Q staging (16 x D) + 2 stages x (K, V)
  constexpr int WARP_BYTES = 16 * D * 2 + 4 * TILE_BYTES;
  const uint32_t q_sm = sbase + warp * WARP_BYTES;
  const uint32_t kv_sm = q_sm + 16 * D * 2;

  // KV range of this split, in whole tiles
  const int tiles_total = (ctx + BN - 1) / BN;
  const int tiles_per_split = (tiles_total + num_splits - 1) / num_splits;
  const int tile_begin = split * tiles_per_split;
  const int tile_end = min(tiles_total, tile_begin + tiles_per_split);

  PagedKV kv{k_cache, v_cache, block_tables + static_cast<int64_t>(seq) * max_blocks, n_kv, kvh, page_size, ctx, num_pages};
  uint32_t qf[D / 16][4];
  load_q_frags<D>(q, q_stride, seq, 1, group, kvh, 0, q_sm, qf, lane);

  float o[D / 8][4];
#pragma unroll
  for (int d = 0; d < D / 8; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.0f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
  const int g = lane >> 2;
  const int max_lo = g < group ? ctx - 1 : -1;
  const int max_hi = g + 8 < group ? ctx - 1 : -1;

  int t = tile_begin + warp;
  if (t < tile_end) {
    load_kv_tile<D, BN, 32>(kv, t * BN, kv_sm, kv_sm + TILE_BYTES, lane, status);
    cp_async_commit();
  }
  int stage = 0;
  for (; t < tile_end; t += 4) {
    if (t + 4 < tile_end) {
      const uint32_t nb = kv_sm + (stage ^ 1) * 2 * TILE_BYTES;
      load_kv_tile<D, BN, 32>(kv, (t + 4) * BN, nb, nb + TILE_BYTES, lane, status);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncwarp();
    const uint32_t kb = kv_sm + stage * 2 * TILE_BYTES;
    warp_attend<D, BN>(qf, kb, kb + TILE_BYTES, t * BN, max_lo, max_hi, scale_log2, o, m, l, lane);
    __syncwarp();
    stage ^= 1;
  }
  l[0] += __shfl_xor_sync(0xffffffffu, l[0], 1);
  l[0] += __shfl_xor_sync(0xffffffffu, l[0], 2);
  l[1] += __shfl_xor_sync(0xffffffffu, l[1], 1);
  l[1] += __shfl_xor_sync(0xffffffffu, l[1], 2);

  // ---- merge the four warps through shared memory (reusing the KV buffers) ----
  __syncthreads();
  float* red = reinterpret_cast<float*>(smem);  // [4 warps][16 rows][D + 2]
  constexpr int RS = D + 2;
  const int t4 = lane & 3;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    float* dst = red + (warp * 16 + g + half * 8) * RS;
#pragma unroll
    for (int d = 0; d < D / 8; ++d) {
      dst[d * 8 + 2 * t4] = o[d][half * 2];
      dst[d * 8 + 2 * t4 + 1] = o[d][half * 2 + 1];
    }
    if (t4 == 0) {
      dst[D] = m[half];
      dst[D + 1] = l[half];
    }
  }
  __syncthreads();
  // 128 threads: thread -> (row = tid / 8, 16-wide column slice = tid % 8) for D = 128
  constexpr int COLS_PER_THREAD = D / 8;
  const int row = threadIdx.x >> 3, cs = (threadIdx.x & 7) * COLS_PER_THREAD;
  if (row < group) {
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, red[(w * 16 + row) * RS + D]);
    const float sub = mm == -INFINITY ? 0.0f : mm;
    float ll = 0.0f, acc[COLS_PER_THREAD];
#pragma unroll
    for (int c = 0; c < COLS_PER_THREAD; ++c) acc[c] = 0.0f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float* src = red + (w * 16 + row) * RS;
      const float f = ptx::ex2(src[D] - sub);
      ll += src[D + 1] * f;
#pragma unroll
      for (int c = 0; c < COLS_PER_THREAD; ++c) acc[c] += src[cs + c] * f;
    }
    const int head = kvh * group + row;
    if (num_splits == 1) {
      const float inv = ll > 0.0f ? 1.0f / ll : 0.0f;
      __nv_bfloat16* dst = out + static_cast<int64_t>(seq) * out_stride + static_cast<int64_t>(head) * D + cs;
#pragma unroll
      for (int c = 0; c < COLS_PER_THREAD; c += 2)
        *reinterpret_cast<uint32_t*>(dst + c) = ptx::pack_bf16x2(acc[c] * inv, acc[c + 1] * inv);
    } else {
      float* dst = workspace + ((static_cast<int64_t>(seq) * n_q + head) * num_splits + split) * RS;
#pragma unroll
      for (int c = 0; c < COLS_PER_THREAD; ++c) dst[cs + c] = acc[c];
      if ((threadIdx.x & 7) == 0) {
        dst[D] = mm;
        dst[D + 1] = ll;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Decode, TMA path (page_size % 32 == 0): one warp per (split, kv head, sequence). K/V tiles of 32 tokens
// arrive as SWIZZLE_128B boxes through a STAGES-deep mbarrier ring issued by lane 0, so the address work per
// 16 KB tile is four instructions instead of a page-table walk per 16-byte chunk, and several small CTAs per
// SM keep ~200 KB of loads in flight. The cache is addressed as a 2-D matrix [(page, kv head, token), D].
// ------------------------------------------------------------------------------------------------
template <int D, int STAGES>
__global__ void __launch_bounds__(32) attn_decode_tma_kernel(
    const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
    const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out, const int32_t* __restrict__ ctx_lens,
    const int32_t* __restrict__ block_tables, float* __restrict__ workspace, int max_blocks, int n_q, int n_kv,
    int page_size, int num_splits, float scale_log2, int64_t q_stride, int64_t out_stride, int64_t num_pages,
    uint32_t* __restrict__ split_counters, Status* status) {
  ptx::grid_dep_sync();
  constexpr int BN = 32;
  constexpr int HALVES = D / 64;
  constexpr int SUB_BYTES = BN * 128;              // one [32][64] box
  constexpr int TILE_BYTES = HALVES * SUB_BYTES;   // K or V tile
  constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_sm = sbase + STAGES * STAGE_BYTES;
  const uint32_t bar0 = q_sm + 16 * D * 2;
  const int split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
  const int lane = threadIdx.x;
  const int group = n_q / n_kv;
  const int ctx = ctx_lens[seq];
  const int32_t* table = block_tables + static_cast<int64_t>(seq) * max_blocks;

  const int tiles_total = (ctx + BN - 1) / BN;
  const int tiles_per_split = (tiles_total + num_splits - 1) / num_splits;
  const int tile_begin = split * tiles_per_split;
  const int tile_end = min(tiles_total, tile_begin + tiles_per_split);
  const int n_tiles = max(0, tile_end - tile_begin);

  if (lane == 0) {
    ptx::prefetch_tensormap(&tmap_k);
    ptx::prefetch_tensormap(&tmap_v);
    for (int s = 0; s < STAGES; ++s) ptx::mbar_init(bar0 + 8 * s, 1);
    ptx::fence_mbar_init();
  }
  __syncwarp();

  auto issue = [&](int i) {  // lane 0 only: start the loads of this CTA's i-th tile
    const int t = tile_begin + i;
    const int pos = t * BN;
    int64_t page = table[pos / page_size];
    if (!B2_ASSERT(status, page >= 0 && page < num_pages, kSiteKvIndex, page, num_pages)) page = 0;
    const int row = static_cast<int>((page * n_kv + kvh) * page_size + pos % page_size);
    const int s = i % STAGES;
    const uint32_t dst = sbase + s * STAGE_BYTES;
    const uint32_t bar = bar0 + 8 * s;
    ptx::mbar_arrive_expect_tx(bar, STAGE_BYTES);
#pragma unroll
    for (int h = 0; h < HALVES; ++h) {
      ptx::tma_load_2d(dst + h * SUB_BYTES, &tmap_k, bar, h * 64, row, ptx::kEvictFirst);
      ptx::tma_load_2d(dst + TILE_BYTES + h * SUB_BYTES, &tmap_v, bar, h * 64, row, ptx::kEvictFirst);
    }
  };
  if (lane == 0) {
    for (int i = 0; i < STAGES - 1 && i < n_tiles; ++i) issue(i);
  }

  uint32_t qf[D / 16][4];
  load_q_frags<D>(q, q_stride, seq, 1, group, kvh, 0, q_sm, qf, lane);

  float o[D / 8][4];
#pragma unroll
  for (int d = 0; d < D / 8; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.0f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
  const int g = lane >> 2;
  const int max_lo = g < group ? ctx - 1 : -1;
  const int max_hi = g + 8 < group ? ctx - 1 : -1;

  bool ok = true;
  for (int i = 0; i < n_tiles; ++i) {
    const int s = i % STAGES;
    // the stage being refilled was consumed in iteration i - 1 (program order within the warp)
    if (lane == 0 && i + STAGES - 1 < n_tiles) issue(i + STAGES - 1);
    if (!__all_sync(0xffffffffu, ptx::mbar_wait(bar0 + 8 * s, (i / STAGES) & 1))) {
      if (lane == 0) status_record(status, kTimeout, kSiteAttn, seq, i);
      ok = false;
      break;
    }
    const uint32_t kb = sbase + s * STAGE_BYTES;
    const int kv0 = (tile_begin + i) * BN;
    if (kv0 + BN > ctx) {
      // rows past the context hold whatever the page held before: clear V there so 0 * garbage stays 0
      for (int r = ctx - kv0 + (lane >> 4); r < BN; r += 2)
#pragma unroll
        for (int c = (lane & 15); c < D / 8; c += 16) {
          const uint32_t a = tile_addr<D, BN>(kb + TILE_BYTES, r, c);
          asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(a), "r"(0u) : "memory");
        }
      __syncwarp();
    }
    warp_attend<D, BN, BN>(qf, kb, kb + TILE_BYTES, kv0, max_lo, max_hi, scale_log2, o, m, l, lane);
    __syncwarp();
  }
  if (!ok) {
    // let outstanding copies land before the CTA's shared memory is released
    for (int i = 0; i < STAGES; ++i) ptx::mbar_wait(bar0 + 8 * i, 0, 20000000ull) || ptx::mbar_wait(bar0 + 8 * i, 1, 20000000ull);
    return;
  }
  l[0] += __shfl_xor_sync(0xffffffffu, l[0], 1);
  l[0] += __shfl_xor_sync(0xffffffffu, l[0], 2);
  l[1] += __shfl_xor_sync(0xffffffffu, l[1], 1);
  l[1] += __shfl_xor_sync(0xffffffffu, l[1], 2);
  const int t4 = lane & 3;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int row = g + half * 8;
    if (row >= group) continue;
    const int head = kvh * group + row;
    if (num_splits == 1) {
      const float inv = l[half] > 0.0f ? 1.0f / l[half] : 0.0f;
      __nv_bfloat16* dst = out + static_cast<int64_t>(seq) * out_stride + static_cast<int64_t>(head) * D;
#pragma unroll
      for (int d = 0; d < D / 8; ++d)
        *reinterpret_cast<uint32_t*>(dst + d * 8 + 2 * t4) = ptx::pack_bf16x2(o[d][half * 2] * inv, o[d][half * 2 + 1] * inv);
    } else {
      float* dst = workspace + ((static_cast<int64_t>(seq) * n_q + head) * num_splits + split) * (D + 2);
#pragma unroll
      for (int d = 0; d < D / 8; ++d)
        *reinterpret_cast<float2*>(dst + d * 8 + 2 * t4) = make_float2(o[d][half * 2], o[d][half * 2 + 1]);
      if (t4 == 0) {
        dst[D] = m[half];
        dst[D + 1] = l[half];
      }
    }
  }
  if (num_splits > 1 && split_counters != nullptr) {
    // The split that finishes last merges the partials of its (sequence, kv head): no second launch. Its own stores
    // and the others' are ordered by the fence on each side of the counter.
    __threadfence();
    __syncwarp();
    uint32_t old = 0;
    if (lane == 0) old = atomicAdd(split_counters + static_cast<int64_t>(seq) * n_kv + kvh, 1u);
    old = __shfl_sync(0xffffffffu, old, 0);
    if (old != static_cast<uint32_t>(num_splits - 1)) return;
    if (lane == 0) split_counters[static_cast<int64_t>(seq) * n_kv + kvh] = 0;   // ready for the next launch
    __threadfence();
    constexpr int RS = D + 2;
    for (int row = 0; row < group; ++row) {
      const int head = kvh * group + row;
      const float* base = workspace + (static_cast<int64_t>(seq) * n_q + head) * num_splits * RS;
      float mm = -INFINITY;
      for (int sp = 0; sp < num_splits; ++sp) mm = fmaxf(mm, __ldcg(base + sp * RS + D));
      const float sub = mm == -INFINITY ? 0.0f : mm;
      float ll = 0.0f;
      float acc[D / 32];
#pragma unroll
      for (int c = 0; c < D / 32; ++c) acc[c] = 0.0f;
      for (int sp = 0; sp < num_splits; ++sp) {
        const float f = ptx::ex2(__ldcg(base + sp * RS + D) - sub);
        ll += __ldcg(base + sp * RS + D + 1) * f;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) acc[c] += __ldcg(base + sp * RS + c * 32 + lane) * f;
      }
      const float inv = ll > 0.0f ? 1.0f / ll : 0.0f;
      __nv_bfloat16* dst = out + static_cast<int64_t>(seq) * out_stride + static_cast<int64_t>(head) * D;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) dst[c * 32 + lane] = __float2bfloat16(acc[c] * inv);
    }
  }
}

// Merge split partials: one warp per (sequence, head).
template <int D>
__global__ void attn_decode_reduce_kernel(const float* __restrict__ workspace, __nv_bfloat16* __restrict__ out,
                                          int n_q, int num_splits, int64_t out_stride, int total) {
  ptx::grid_dep_sync();
  constexpr int RS = D + 2;
  const int idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (idx >= total) return;
  const int seq = idx / n_q, head = idx % n_q;
  const float* base = workspace + static_cast<int64_t>(idx) * num_splits * RS;
  float mm = -INFINITY;
  for (int s = 0; s < num_splits; ++s) mm = fmaxf(mm, base[s * RS + D]);
  const float sub = mm == -INFINITY ? 0.0f : mm;
  float ll = 0.0f;
  float acc[D / 32];
#pragma unroll
  for (int c = 0; c < D / 32; ++c) acc[c] = 0.0f;
  for (int s = 0; s < num_splits; ++s) {
    const float f = ptx::ex2(base[s * RS + D] - sub);
    ll += base[s * RS + D + 1] * f;
#pragma unroll
    for (int c = 0; c < D / 32; ++c) acc[c] += base[s * RS + c * 32 + lane] * f;
  }
  const float inv = ll > 0.0f ? 1.0f / ll : 0.0f;
  __nv_bfloat16* dst = out + static_cast<int64_t>(seq) * out_stride + static_cast<int64_t>(head) * D;
#pragma unroll
  for (int c = 0; c < D / 32; ++c) dst[c * 32 + lane] = __float2bfloat16(acc[c] * inv);
}

}  // namespace
}  // namespace b2

using namespace b2;

extern "C" int b2_attn_prefill_bf16(const void* q, const void* k_cache, const void* v_cache, void* out,
                                    const int32_t* cu_q, const int32_t* ctx_lens, const int32_t* block_tables,
                                    int batch, int max_blocks, int n_q, int n_kv, int head_dim, int page_size,
                                    int max_q_len, float scale, int64_t q_stride, int64_t out_stride,
                                    int64_t num_pages, Status* status, cudaStream_t stream) {
  if (batch <= 0 || max_q_len <= 0) return 0;
  if (n_kv <= 0 || n_q % n_kv != 0 || (head_dim != 128 && head_dim != 64) || q_stride % 8 != 0 || out_stride % 2 != 0)
    return -kBadArgument;
  const int group = n_q / n_kv;
  dim3 grid((max_q_len * group + 63) / 64, n_kv, batch);
  const float scale_log2 = scale * ptx::kLog2e;
  auto qp = static_cast<const __nv_bfloat16*>(q);
  auto kp = static_cast<const __nv_bfloat16*>(k_cache);
  auto vp = static_cast<const __nv_bfloat16*>(v_cache);
  auto op = static_cast<__nv_bfloat16*>(out);
  if (head_dim == 128) {
    constexpr int SMEM = 4 * 16 * 128 * 2 + 4 * 64 * 128 * 2;
    static DeviceOnce attr_once;
    if (const int rc = attr_once.run([&] { return cudaFuncSetAttribute(attn_prefill_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM); })) return rc;
    launch_pdl(attn_prefill_kernel<128>, dim3(grid), dim3(128), SMEM, stream, qp, kp, vp, op, cu_q, ctx_lens, block_tables, max_blocks, n_q,
                                                          n_kv, page_size, scale_log2, q_stride, out_stride, num_pages,
                                                          status);
  } else {
    constexpr int SMEM = 4 * 16 * 64 * 2 + 4 * 64 * 64 * 2;
    static DeviceOnce attr_once;
    if (const int rc = attr_once.run([&] { return cudaFuncSetAttribute(attn_prefill_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM); })) return rc;
    launch_pdl(attn_prefill_kernel<64>, dim3(grid), dim3(128), SMEM, stream, qp, kp, vp, op, cu_q, ctx_lens, block_tables, max_blocks, n_q,
                                                         n_kv, page_size, scale_log2, q_stride, out_stride, num_pages,
                                                         status);
  }
  return last_launch_rc();
}

extern "C" int64_t b2_attn_decode_workspace(int batch, int n_q, int head_dim, int num_splits) {
  return static_cast<int64_t>(batch) * n_q * num_splits * (head_dim + 2) * 4;
}

// Split decode on the TMA path merges its partials in the split that finishes last, counted per (sequence, kv head) in
// `counters` (u32, zero before the first launch; every launch leaves them at zero). Bytes needed for `batch` sequences:
extern "C" int64_t b2_attn_decode_counter_bytes(int batch, int n_kv) { return static_cast<int64_t>(batch) * n_kv * 4; }

extern "C" int b2_attn_decode_bf16(const void* q, const void* k_cache, const void* v_cache, void* out,
                                   const int32_t* ctx_lens, const int32_t* block_tables, float* workspace, int batch,
                                   int max_blocks, int n_q, int n_kv, int head_dim, int page_size, int num_splits,
                                   float scale, int64_t q_stride, int64_t out_stride, int64_t num_pages,
                                   uint32_t* counters, Status* status, cudaStream_t stream) {
  if (batch <= 0) return 0;
  if (n_kv <= 0 || n_q % n_kv != 0 || n_q / n_kv > 16 || (head_dim != 128 && head_dim != 64) || q_stride % 8 != 0 ||
      num_splits < 1 || (num_splits > 1 && workspace == nullptr))
    return -kBadArgument;
  dim3 grid(num_splits, n_kv, batch);
  const float scale_log2 = scale * ptx::kLog2e;
  auto qp = static_cast<const __nv_bfloat16*>(q);
  auto kp = static_cast<const __nv_bfloat16*>(k_cache);
  auto vp = static_cast<const __nv_bfloat16*>(v_cache);
  auto op = static_cast<__nv_bfloat16*>(out);
  const int total = batch * n_q;
  if (page_size % 32 == 0) {
    // TMA path: cache as a 2-D matrix [(page, kv head, token), D], boxes of 32 tokens x 64 columns
    CUtensorMap tk, tv;
    const uint64_t rows = static_cast<uint64_t>(num_pages) * n_kv * page_size;
    if (!make_tmap_2d(&tk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, k_cache, rows, head_dim, head_dim * 2, 32, 64, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !make_tmap_2d(&tv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, v_cache, rows, head_dim, head_dim * 2, 32, 64, CU_TENSOR_MAP_SWIZZLE_128B))
      return -kBadArgument;
    constexpr int STAGES = 3;
    if (head_dim == 128) {
      constexpr int SMEM = STAGES * 2 * 32 * 128 * 2 + 16 * 128 * 2 + 64 + 1024;
      static DeviceOnce attr_once;
    if (const int rc = attr_once.run([&] { return cudaFuncSetAttribute(attn_decode_tma_kernel<128, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM); })) return rc;
      launch_pdl(attn_decode_tma_kernel<128, STAGES>, dim3(grid), dim3(32), SMEM, stream, tk, tv, qp, op, ctx_lens, block_tables, workspace, max_blocks,
                                                                    n_q, n_kv, page_size, num_splits, scale_log2, q_stride,
                                                                    out_stride, num_pages, counters, status);
      if (num_splits > 1 && counters == nullptr)
        launch_pdl(attn_decode_reduce_kernel<128>, dim3((total + 3) / 4), dim3(128), 0, stream, workspace, op, n_q, num_splits, out_stride, total);
    } else {
      constexpr int SMEM = STAGES * 2 * 32 * 64 * 2 + 16 * 64 * 2 + 64 + 1024;
      static DeviceOnce attr_once;
    if (const int rc = attr_once.run([&] { return cudaFuncSetAttribute(attn_decode_tma_kernel<64, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM); })) return rc;
      launch_pdl(attn_decode_tma_kernel<64, STAGES>, dim3(grid), dim3(32), SMEM, stream, tk, tv, qp, op, ctx_lens, block_tables, workspace, max_blocks,
                                                                   n_q, n_kv, page_size, num_splits, scale_log2, q_stride,
                                                                    out_stride, num_pages, counters, status);
      if (num_splits > 1 && counters == nullptr)
        launch_pdl(attn_decode_reduce_kernel<64>, dim3((total + 3) / 4), dim3(128), 0, stream, workspace, op, n_q, num_splits, out_stride, total);
    }
    return last_launch_rc();
  }
  if (head_dim == 128) {
    constexpr int SMEM = 4 * (16 * 128 * 2 + 4 * 32 * 128 * 2);
    static DeviceOnce attr_once;
    if (const int rc = attr_once.run([&] { return cudaFuncSetAttribute(attn_decode_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM); })) return rc;
    launch_pdl(attn_decode_kernel<128>, dim3(grid), dim3(128), SMEM, stream, qp, kp, vp, op, ctx_lens, block_tables, workspace, max_blocks,
                                                         n_q, n_kv, page_size, num_splits, scale_log2, q_stride,
                                                         out_stride, num_pages, status);
    if (num_splits > 1)
      launch_pdl(attn_decode_reduce_kernel<128>, dim3((total + 3) / 4), dim3(128), 0, stream, workspace, op, n_q, num_splits, out_stride, total);
  } else {
    constexpr int SMEM = 4 * (16 * 64 * 2 + 4 * 32 * 64 * 2);
    static DeviceOnce attr_once;
    if (const int rc = attr_once.run([&] { return cudaFuncSetAttribute(attn_decode_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM); })) return rc;
    launch_pdl(attn_decode_kernel<64>, dim3(grid), dim3(128), SMEM, stream, qp, kp, vp, op, ctx_lens, block_tables, workspace, max_blocks,
                                                        n_q, n_kv, page_size, num_splits, scale_log2, q_stride,
                                                        out_stride, num_pages, status);
    if (num_splits > 1)
      launch_pdl(attn_decode_reduce_kernel<64>, dim3((total + 3) / 4), dim3(128), 0, stream, workspace, op, n_q, num_splits, out_stride, total);
  }
  return last_launch_rc();
}
