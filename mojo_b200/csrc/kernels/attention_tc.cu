// Causal GQA prefill attention on the 5th-generation tensor cores: S = Q K^T and O_j = P_j V_j are tcgen05.mma
// instructions with S and O_j in TMEM; Q, K and V tiles arrive by TMA; the online softmax runs in registers.
// Head dimension 128, KV pages of 128 tokens (one KV tile = one page of one KV head, a contiguous 32 KB block).
// The reference has no attention of any kind, and no tensor-core code (its newest gate is sm_90a,
// stdlib/src/sys/info.mojo:423-434).
//
// One CTA = 128 query rows of one query head, 320 threads:
//   warp 0      TMA producer: the Q tile once (two 128 x 64 boxes), then K and V of each KV tile into a 2-deep ring
//   warp 1      owns TMEM (512 columns: two S buffers, two O buffers); one lane issues the MMAs
//                 S_j   = Q K_j^T    A = Q  (K-major, 128-byte swizzle), B = K_j (K-major: head dim is contiguous)
//                 O_j   = P_j V_j    A = P_j (K-major, written by the softmax warps), B = V_j (MN-major: V rows are
//                                    KV tokens, so the N = head-dim index is the contiguous one)
//   warps 2-9   compute, two threads per query row (64 columns each): tcgen05.ld the half row of S_j, causal mask,
//               running max (halves exchanged through shared memory), exp2, row sum; write P_j as bf16 into shared
//               memory in the swizzled operand layout; then O = O * alpha_{j-1} + O_{j-1} for their 64 columns of
//               the accumulator (tcgen05.ld); at the end O / l as bf16
// S_{j+1} is issued before P_j V_j, so the softmax of tile j + 1 overlaps the second MMA of tile j, and the
// accumulation of O_j runs after the softmax of tile j + 1.
// Every mbarrier wait is bounded; a role that gives up records TIMEOUT, raises a CTA-wide flag and leaves its
// loop, the others follow at their next wait, and the CTA still frees TMEM and exits.
#include <cstdint>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "b2/api.h"
#include "b2/launch.h"
#include "b2/config.h"
#include "b2/gemm_tc.cuh"
#include "b2/ptx.cuh"
#include "b2/status.h"
#include "b2/tma.h"

namespace b2 {
namespace {

constexpr int kD = 128;            // head dimension
constexpr int kTile = 128;         // query rows per CTA = KV tokens per tile = page size
constexpr int kThreadsAttn = 320;
constexpr int kHalfBytes = kTile * 64 * 2;     // one 128 x 64 bf16 box: 16 KB
constexpr int kTileBytes = 2 * kHalfBytes;     // 128 x 128 bf16: 32 KB
constexpr int kStages = 2;
// shared memory: Q | P | K[2] | V[2] | barriers | alpha ring | l
constexpr int kOffQ = 0;
constexpr int kOffP = kOffQ + kTileBytes;
constexpr int kOffK = kOffP + kTileBytes;
constexpr int kOffV = kOffK + kStages * kTileBytes;
constexpr int kOffBar = kOffV + kStages * kTileBytes;      // 192 KB
constexpr int kNumBars = 1 + 4 * kStages + 2 + 2 + 2 + 2 + 1;  // q_full, k/v full+empty, s full/empty, p full/empty, o full/empty, drain
constexpr int kOffAlpha = kOffBar + 8 * kNumBars + 16;     // float [2][2][128]: partial row maxima
constexpr int kOffL = kOffAlpha + 4 * kTile * 4;           // float [2][128]
constexpr int kOffFlags = kOffL + 2 * kTile * 4;           // tmem holder, fail flag
constexpr int kSmemAttn = kOffFlags + 16 + 1024;           // + alignment slack

struct AttnTcParams {
  __nv_bfloat16* out;
  int64_t ld_out;
  const int* cu_q;
  const int* ctx_lens;
  const int* block_tables;
  int max_blocks, n_q, n_kv;
  int64_t num_pages;
  float scale_log2;   // softmax scale * log2(e)
  // descriptor of the MN-major V operand (bytes): stride between 64-column groups, stride between 8-row groups
  uint32_t v_lbo, v_sbo;
  // Optional work list: item i = (sequence, query tile) as two ints, for grids of (items, heads). `n_work` (device
  // memory) is the number of valid items, so that a captured launch with a fixed grid serves any batch; null means
  // every CTA of the grid has an item. Without a list the grid is (query tiles, heads, sequences).
  const int* work;
  const int* n_work;
};

// Shared-memory descriptor with explicit leading / stride byte offsets, 128-byte swizzle.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

__global__ void __launch_bounds__(kThreadsAttn, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                       const __grid_constant__ CUtensorMap tmap_v, AttnTcParams prm, Status* status) {
  ptx::grid_dep_sync();
  int seq = blockIdx.z, qt = blockIdx.x;
  const int head = blockIdx.y;
  if (prm.work != nullptr) {
    if (prm.n_work != nullptr && static_cast<int>(blockIdx.x) >= *prm.n_work) return;
    seq = prm.work[2 * blockIdx.x];
    qt = prm.work[2 * blockIdx.x + 1];
  }
  const int q_begin = prm.cu_q[seq], q_len = prm.cu_q[seq + 1] - q_begin;
  if (qt * kTile >= q_len) return;                       // uniform per CTA: before any barrier or allocation
  const int ctx = prm.ctx_lens[seq];
  const int pos0 = ctx - q_len + qt * kTile;              // absolute position of this tile's first query row
  const int rows = min(kTile, q_len - qt * kTile);
  const int n_tiles = min((pos0 + rows + kTile - 1) / kTile, (ctx + kTile - 1) / kTile);  // KV tiles with a visible token
  const int kvh = head / (prm.n_q / prm.n_kv);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - ptx::smem_u32(smem_raw));
  auto bar = [&](int i) { return base + kOffBar + 8u * i; };
  const uint32_t q_full = bar(0);
  auto k_full = [&](int s) { return bar(1 + s); };
  auto v_full = [&](int s) { return bar(1 + kStages + s); };
  auto k_empty = [&](int s) { return bar(1 + 2 * kStages + s); };
  auto v_empty = [&](int s) { return bar(1 + 3 * kStages + s); };
  auto s_full = [&](int a) { return bar(1 + 4 * kStages + a); };
  auto s_empty = [&](int a) { return bar(3 + 4 * kStages + a); };
  const uint32_t p_full = bar(5 + 4 * kStages), p_empty = bar(6 + 4 * kStages);
  auto o_full = [&](int a) { return bar(7 + 4 * kStages + a); };
  auto o_empty = [&](int a) { return bar(9 + 4 * kStages + a); };
  const uint32_t drain_bar = bar(11 + 4 * kStages);
  float* alpha_ring = reinterpret_cast<float*>(smem + kOffAlpha);
  float* l_final = reinterpret_cast<float*>(smem + kOffL);
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + kOffFlags);
  volatile uint32_t* fail = reinterpret_cast<volatile uint32_t*>(smem + kOffFlags + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    ptx::prefetch_tensormap(&tmap_q);
    ptx::prefetch_tensormap(&tmap_k);
    ptx::prefetch_tensormap(&tmap_v);
    ptx::mbar_init(q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(k_full(s), 1);
      ptx::mbar_init(v_full(s), 1);
      ptx::mbar_init(k_empty(s), 1);
      ptx::mbar_init(v_empty(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(s_full(a), 1);
      ptx::mbar_init(s_empty(a), 8);
      ptx::mbar_init(o_full(a), 1);
      ptx::mbar_init(o_empty(a), 8);
    }
    ptx::mbar_init(p_full, 8);
    ptx::mbar_init(p_empty, 1);
    ptx::mbar_init(drain_bar, 1);
    ptx::fence_mbar_init();
    *fail = 0;
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_holder), 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  auto give_up = [&](int site_a, int site_b) {
    status_record(status, kTimeout, kSiteAttn, site_a, site_b);
    *fail = 1;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (ptx::elect_one()) {
      ptx::mbar_arrive_expect_tx(q_full, kTileBytes);
      ptx::tma_load_2d(base + kOffQ, &tmap_q, q_full, head * kD, q_begin + qt * kTile, ptx::kEvictFirst);
      ptx::tma_load_2d(base + kOffQ + kHalfBytes, &tmap_q, q_full, head * kD + 64, q_begin + qt * kTile, ptx::kEvictFirst);
      int issued_k = 0, issued_v = 0;
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j % kStages;
        const uint32_t ph = static_cast<uint32_t>((j / kStages) & 1);
        int page = prm.block_tables[static_cast<int64_t>(seq) * prm.max_blocks + j];
        if (page < 0 || page >= prm.num_pages) {
          status_record(status, kOutOfBounds, kSiteKvIndex, seq, page);
          page = 0;
        }
        const int row = (page * prm.n_kv + kvh) * kTile;
        if (!ptx::mbar_wait(k_empty(s), ph ^ 1u)) { give_up(1, j); ok = false; break; }
        ptx::mbar_arrive_expect_tx(k_full(s), kTileBytes);
        ptx::tma_load_2d(base + kOffK + s * kTileBytes, &tmap_k, k_full(s), 0, row, ptx::kEvictLast);
        ptx::tma_load_2d(base + kOffK + s * kTileBytes + kHalfBytes, &tmap_k, k_full(s), 64, row, ptx::kEvictLast);
        ++issued_k;
        if (!ptx::mbar_wait(v_empty(s), ph ^ 1u)) { give_up(2, j); ok = false; break; }
        ptx::mbar_arrive_expect_tx(v_full(s), kTileBytes);
        ptx::tma_load_2d(base + kOffV + s * kTileBytes, &tmap_v, v_full(s), 0, row, ptx::kEvictLast);
        ptx::tma_load_2d(base + kOffV + s * kTileBytes + kHalfBytes, &tmap_v, v_full(s), 64, row, ptx::kEvictLast);
        ++issued_v;
      }
      if (!ok) {
        // let the copies this thread started land before the CTA gives up its shared memory
        ptx::mbar_wait(q_full, 0, 200000000ull);
        for (int j = max(0, issued_k - kStages); j < issued_k; ++j) ptx::mbar_wait(k_full(j % kStages), (j / kStages) & 1, 200000000ull);
        for (int j = max(0, issued_v - kStages); j < issued_v; ++j) ptx::mbar_wait(v_full(j % kStages), (j / kStages) & 1, 200000000ull);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (ptx::elect_one()) {
      constexpr uint32_t idesc_s = ptx::make_idesc(1, 1, 128, 128);                 // bf16 x bf16, both K-major
      constexpr uint32_t idesc_o = ptx::make_idesc(1, 1, 128, 128) | (1u << 16);    // B (= V) is MN-major
      bool ok = true;
      auto issue_s = [&](int j) -> bool {
        const int s = j % kStages, a = j & 1;
        if (!ptx::mbar_wait(k_full(s), (j / kStages) & 1)) { give_up(3, j); return false; }
        if (!ptx::mbar_wait(s_empty(a), ((j >> 1) & 1) ^ 1u)) { give_up(4, j); return false; }
        ptx::tc_fence_after();
        const uint32_t d = tmem_base + a * 128;
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
          const uint64_t da = ptx::make_smem_desc_sw128(base + kOffQ + kb * kHalfBytes);
          const uint64_t db = ptx::make_smem_desc_sw128(base + kOffK + s * kTileBytes + kb * kHalfBytes);
#pragma unroll
          for (int k = 0; k < 4; ++k) ptx::tc_mma_f16(d, da + 2u * k, db + 2u * k, idesc_s, (kb | k) ? 1u : 0u);
        }
        ptx::tc_commit(k_empty(s));    // K_j can be overwritten once S_j has read it
        ptx::tc_commit(s_full(a));
        return true;
      };
      if (!ptx::mbar_wait(q_full, 0)) { give_up(5, 0); ok = false; }
      if (ok && n_tiles > 0) ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles && !issue_s(j + 1)) { ok = false; break; }
        const int s = j % kStages, a = j & 1;
        if (!ptx::mbar_wait(v_full(s), (j / kStages) & 1)) { give_up(6, j); ok = false; break; }
        if (!ptx::mbar_wait(p_full, j & 1)) { give_up(7, j); ok = false; break; }
        if (!ptx::mbar_wait(o_empty(a), ((j >> 1) & 1) ^ 1u)) { give_up(8, j); ok = false; break; }
        ptx::tc_fence_after();
        const uint32_t d = tmem_base + 256 + a * 128;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          // A: 16 KV columns of P = 32 bytes inside the swizzled row (+2 per step, next 64-column block after four)
          const uint64_t da = ptx::make_smem_desc_sw128(base + kOffP + (k >> 2) * kHalfBytes) + 2u * (k & 3);
          // B: 16 KV rows of V = two 8-row groups of 1 KB each; the two 64-column halves of the head dim are v_lbo apart
          const uint64_t db = smem_desc(base + kOffV + s * kTileBytes + k * 2048, prm.v_lbo, prm.v_sbo);
          ptx::tc_mma_f16(d, da, db, idesc_o, k ? 1u : 0u);
        }
        ptx::tc_commit(v_empty(s));
        ptx::tc_commit(p_empty);
        ptx::tc_commit(o_full(a));
      }
      if (!ok) {
        ptx::tc_commit(drain_bar);
        ptx::mbar_wait(drain_bar, 0, 200000000ull);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ compute warps
    // Eight warps, two threads per query row: thread (r, g) owns columns [64 g, 64 g + 64) of the row's S tile and
    // the same columns of its O accumulator. Two warps per scheduler hide each other's dependency stalls, which one
    // warp per scheduler cannot. Per KV tile: softmax of S_j and the write of P_j, then (software pipelining) the
    // accumulation of O_{j-1}, whose MMA ran while this tile's softmax did.
    const int g = (warp - 2) >> 2;          // column half
    const int quarter = warp & 3;           // TMEM lane quarter this warp may access
    const int r = quarter * 32 + lane;
    const int qpos = pos0 + r;
    const uint32_t lane_bits = static_cast<uint32_t>(quarter * 32) << 16;
    float* pmax = alpha_ring;               // [2 tiles in flight][2 halves][128 rows]
    float m_run = -INFINITY, l_part = 0.0f, alpha_prev = 1.0f;
    float o[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) o[i] = 0.0f;
    // A warp that gives up keeps walking the loop (every compute warp must reach the named barrier of every tile)
    // but no longer waits, reads TMEM or arrives anywhere; the other roles then run into their own limits.
    bool ok = true;
    auto wait_all = [&](uint32_t bar_addr, uint32_t parity, int code, int j) -> bool {
      if (!ok || *fail != 0) return false;
      if (__all_sync(0xffffffffu, ptx::mbar_wait(bar_addr, parity))) return true;
      if (lane == 0) give_up(code, j);
      return false;
    };
    auto accumulate = [&](int j, float alpha) {
      const int a = j & 1;
      ok = wait_all(o_full(a), (j >> 1) & 1, 11, j);
      if (!ok) return;
      ptx::tc_fence_after();
      const uint32_t taddr = tmem_base + 256 + a * 128 + g * 64 + lane_bits;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t v[32];
        ptx::tmem_ld_32x32(taddr + c * 32, v);
        ptx::tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c * 32 + i] = fmaf(o[c * 32 + i], alpha, __uint_as_float(v[i]));
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(o_empty(a));
    };
    for (int j = 0; j < n_tiles; ++j) {
      const int a = j & 1;
      float s[64];
      ok = wait_all(s_full(a), (j >> 1) & 1, 9, j);
      if (ok) {
        ptx::tc_fence_after();
        const uint32_t taddr = tmem_base + a * 128 + g * 64 + lane_bits;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t v[32];
          ptx::tmem_ld_32x32(taddr + c * 32, v);
          ptx::tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) s[c * 32 + i] = __uint_as_float(v[i]);
        }
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(s_empty(a));     // S buffer free for tile j + 2
      } else {
#pragma unroll
        for (int c = 0; c < 64; ++c) s[c] = 0.0f;
      }
      const int kv0 = j * kTile + g * 64;
      if (kv0 + 63 > pos0) {                             // some row of this tile masks some of these columns
#pragma unroll
        for (int c = 0; c < 64; ++c)
          if (kv0 + c > qpos) s[c] = -INFINITY;
      }
      // row maximum of the raw scores: eight independent chains, then the partner's half through shared memory
      float mx[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) mx[i] = s[i];
#pragma unroll
      for (int c = 8; c < 64; ++c) mx[c & 7] = fmaxf(mx[c & 7], s[c]);
      const float mloc = fmaxf(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])), fmaxf(fmaxf(mx[4], mx[5]), fmaxf(mx[6], mx[7])));
      pmax[(a * 2 + g) * kTile + r] = mloc;
      ptx::named_barrier_sync(5, 256);
      const float m_new = fmaxf(m_run, fmaxf(mloc, pmax[(a * 2 + (g ^ 1)) * kTile + r]));
      const float m_use = m_new == -INFINITY ? 0.0f : m_new;   // a row with nothing visible yet
      const float alpha = ptx::ex2((m_run - m_use) * prm.scale_log2);
      const float neg_m = -m_use * prm.scale_log2;
      m_run = m_new;
      if (j > 0) ok = wait_all(p_empty, (j - 1) & 1, 10, j);
      if (ok) {
        float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          float p[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            p[i] = ptx::ex2(fmaf(s[ch * 8 + i], prm.scale_log2, neg_m));
            sum[i & 3] += p[i];
          }
          uint4 pk;
          pk.x = ptx::pack_bf16x2(p[0], p[1]);
          pk.y = ptx::pack_bf16x2(p[2], p[3]);
          pk.z = ptx::pack_bf16x2(p[4], p[5]);
          pk.w = ptx::pack_bf16x2(p[6], p[7]);
          *reinterpret_cast<uint4*>(smem + kOffP + g * kHalfBytes + gemm::sw128_offset(r, ch)) = pk;
        }
        l_part = l_part * alpha + ((sum[0] + sum[1]) + (sum[2] + sum[3]));
        ptx::fence_proxy_async_smem();   // generic-proxy writes of P -> visible to the tensor core's async proxy
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(p_full);
      }
      // O_{j-1} = P_{j-1} V_{j-1} has had this tile's softmax to finish in
      if (j > 0) accumulate(j - 1, alpha_prev);
      alpha_prev = alpha;
    }
    if (n_tiles > 0) accumulate(n_tiles - 1, alpha_prev);
    l_final[g * kTile + r] = l_part;
    ptx::named_barrier_sync(5, 256);
    if (ok && *fail == 0 && r < rows) {
      const float l = l_final[r] + l_final[kTile + r];
      const float inv = l > 0.0f ? 1.0f / l : 0.0f;
      __nv_bfloat16* dst = prm.out + static_cast<int64_t>(q_begin + qt * kTile + r) * prm.ld_out + head * kD + g * 64;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint4 pk;
        pk.x = ptx::pack_bf16x2(o[c * 8 + 0] * inv, o[c * 8 + 1] * inv);
        pk.y = ptx::pack_bf16x2(o[c * 8 + 2] * inv, o[c * 8 + 3] * inv);
        pk.z = ptx::pack_bf16x2(o[c * 8 + 4] * inv, o[c * 8 + 5] * inv);
        pk.w = ptx::pack_bf16x2(o[c * 8 + 6] * inv, o[c * 8 + 7] * inv);
        ptx::st_v4(dst + c * 8, pk);
      }
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace
}  // namespace b2

using namespace b2;

// Same contract as b2_attn_prefill_bf16 with head_dim = 128 and page_size = 128 fixed; out rows 16-byte aligned.
// `variant` is reserved (0). With `work` (device memory, `work_items` pairs of (sequence, query tile)) the grid is one
// CTA per item and head; `n_work` (device memory, may be null) bounds the valid items, for launches whose grid is
// fixed ahead of the batch (CUDA graphs). The caller orders the items, longest context first for an even finish.
extern "C" int b2_attn_prefill_tc_bf16(const void* q, const void* k_cache, const void* v_cache, void* out, const int32_t* cu_q,
                                       const int32_t* ctx_lens, const int32_t* block_tables, int batch, int max_blocks, int n_q,
                                       int n_kv, int max_q_len, float scale, int64_t q_rows, int64_t q_stride, int64_t out_stride,
                                       int64_t num_pages, int variant, const int32_t* work, const int32_t* n_work, int work_items,
                                       Status* status, cudaStream_t stream) {
  if (batch <= 0 || max_q_len <= 0) return 0;
  if (work != nullptr && work_items <= 0) return 0;
  if (n_q <= 0 || n_kv <= 0 || n_q % n_kv != 0 || q_stride % 8 != 0 || out_stride % 8 != 0 ||
      (reinterpret_cast<uintptr_t>(q) & 15) != 0 || (reinterpret_cast<uintptr_t>(out) & 15) != 0)
    return -kBadArgument;
  CUtensorMap tq, tk, tv;
  const int64_t kv_rows = num_pages * n_kv * kTile;
  if (!make_tmap_2d(&tq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, q, q_rows, static_cast<int64_t>(n_q) * kD, q_stride * 2, kTile, 64,
                    CU_TENSOR_MAP_SWIZZLE_128B) ||
      !make_tmap_2d(&tk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, k_cache, kv_rows, kD, kD * 2, kTile, 64, CU_TENSOR_MAP_SWIZZLE_128B) ||
      !make_tmap_2d(&tv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, v_cache, kv_rows, kD, kD * 2, kTile, 64, CU_TENSOR_MAP_SWIZZLE_128B))
    return -kBadArgument;
  AttnTcParams prm{};
  prm.out = static_cast<__nv_bfloat16*>(out);
  prm.ld_out = out_stride;
  prm.cu_q = cu_q;
  prm.ctx_lens = ctx_lens;
  prm.block_tables = block_tables;
  prm.max_blocks = max_blocks;
  prm.n_q = n_q;
  prm.n_kv = n_kv;
  prm.num_pages = num_pages;
  prm.scale_log2 = scale * 1.4426950408889634f;
  prm.v_lbo = kHalfBytes;   // the second 64 columns of the head dimension are the second TMA box
  prm.v_sbo = 1024;         // 8 KV rows of 128 bytes
  prm.work = work;
  prm.n_work = work != nullptr ? n_work : nullptr;
  (void)variant;
  static DeviceOnce attr_once;
  if (const int rc = attr_once.run([&] {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemAttn);
        return e;
      }))
    return rc;
  dim3 grid((max_q_len + kTile - 1) / kTile, n_q, batch);
  if (work != nullptr) grid = dim3(work_items, n_q, 1);
  launch_pdl(attn_prefill_tc_kernel, dim3(grid), dim3(kThreadsAttn), kSmemAttn, stream, tq, tk, tv, prm, status);
  return last_launch_rc();
}
