// Multi-head latent attention with absorbed projections: decode, and prefill chunks as one row group per query token.
//
// Per token the cache stores one row [c (512 latent dims) | k_rope (64 dims)] shared by all heads. With W_UK
// folded into the query and W_UV applied after the kernel, attention for 16 heads is
//     s[h, t] = (q_lat[h] . c[t] + q_rope[h] . k_rope[t]) * scale,   o_lat[h] = sum_t softmax(s)[h, t] * c[t]
// i.e. one 16-row MMA tile against a 576-wide key that doubles as a 512-wide value: every cache byte is read
// once and used twice.
//
// CTA = 4 warps on one (KV split, head group, sequence). A 32-token tile (36 KB) arrives as nine SWIZZLE_128B
// TMA boxes through a 3-stage mbarrier ring. The 576-wide dot product is split four ways across the warps and
// summed through shared memory (one __syncthreads per tile, parity double-buffered); each warp then owns 128
// of the 512 output columns, so the f32 accumulator is 64 registers per thread.
//
// A "row group" (grid z) is one query token: its 16 heads, the context length it may see and the block table of
// its sequence. In decode there is one row group per sequence. A prefill chunk contributes one row group per
// token, with context = cached prefix + position in the chunk + 1 (that is the causal mask) and `row_seq` naming
// the sequence whose block table it reads; the chunk's latents are in the cache before the kernel runs, and the
// tiles shared by the tokens of a sequence are served by L2.
#include <cstdint>
#include <cstdlib>
#include <cuda.h>
#include <cuda_bf16.h>
#include "b2/api.h"
#include "b2/launch.h"
#include "b2/ptx.cuh"
#include "b2/tma.h"

namespace b2 {
namespace {

constexpr int kLat = 512, kRope = 64, kRow = kLat + kRope;  // 576
constexpr int BN = 32;
constexpr int kSub = kRow / 64;                 // 9 boxes of 64 columns
constexpr int kTileBytes = kSub * BN * 128;     // 36864

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 16-byte chunk `chunk` of row `row` in a tile made of [BN][64] sub-tiles with the 128-byte TMA swizzle
__device__ __forceinline__ uint32_t kv_addr(uint32_t base, int row, int chunk) {
  return base + static_cast<uint32_t>((chunk >> 3) * (BN * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

// STAGES = 2 (110 KB of shared memory) lets two CTAs share an SM: eight warps instead of four hide each other's
// ldmatrix / mma / barrier latency. Measured against the three-stage ring (146 KB, one CTA per SM, one warp per
// scheduler, tensor pipe 11 % active): prefill rows 612 -> 408 us for 8 x 512 tokens, decode 45.9 -> 35.7 us for
// 64 sequences x 768 tokens. Two is therefore the default for both; B2_MLA_STAGES=3 selects the deep ring.
template <int STAGES>
__global__ void __launch_bounds__(128, STAGES == 2 ? 2 : 1) mla_decode_kernel(
    const __grid_constant__ CUtensorMap tmap_kv, const __nv_bfloat16* __restrict__ q_lat,
    const __nv_bfloat16* __restrict__ q_rope, __nv_bfloat16* __restrict__ out_lat, const int32_t* __restrict__ ctx_lens,
    const int32_t* __restrict__ block_tables, const int32_t* __restrict__ row_seq, float* __restrict__ workspace,
    int max_blocks, int n_heads, int page_size, int num_splits, float scale_log2, int64_t num_pages, int64_t q_lat_stride,
    int64_t q_rope_stride, Status* status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ int sh_fail;  // set by any thread whose wait ran out; read after the per-tile barrier so all agree
  const uint32_t sbase = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_sm = sbase + STAGES * kTileBytes;        // [16][576] bf16, rows of 1152 bytes (72 chunks)
  const uint32_t s_sm = q_sm + 16 * kRow * 2;               // [2][4 warps][16][32] f32
  const uint32_t bar0 = s_sm + 2 * 4 * 16 * 32 * 4;
  uint8_t* gen = smem_raw + (sbase - ptx::smem_u32(smem_raw));
  float* s_red = reinterpret_cast<float*>(gen + STAGES * kTileBytes + 16 * kRow * 2);
  __nv_bfloat16* q_gen = reinterpret_cast<__nv_bfloat16*>(gen + STAGES * kTileBytes);

  const int split = blockIdx.x, hg = blockIdx.y, seq = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ctx = ctx_lens[seq];
  const int32_t* table = block_tables + static_cast<int64_t>(row_seq != nullptr ? row_seq[seq] : seq) * max_blocks;
  const int head0 = hg * 16;
  const int rows = min(16, n_heads - head0);

  const int tiles_total = (ctx + BN - 1) / BN;
  const int tiles_per_split = (tiles_total + num_splits - 1) / num_splits;
  const int tile_begin = split * tiles_per_split;
  const int tile_end = min(tiles_total, tile_begin + tiles_per_split);
  const int n_tiles = max(0, tile_end - tile_begin);

  if (threadIdx.x == 0) {
    sh_fail = 0;
    ptx::prefetch_tensormap(&tmap_kv);
    for (int s = 0; s < STAGES; ++s) ptx::mbar_init(bar0 + 8 * s, 1);
    ptx::fence_mbar_init();
  }
  auto issue = [&](int i) {
    const int pos = (tile_begin + i) * BN;
    int64_t page = table[pos / page_size];
    if (!B2_ASSERT(status, page >= 0 && page < num_pages, kSiteKvIndex, page, num_pages)) page = 0;
    const int row = static_cast<int>(page * page_size + pos % page_size);
    const int s = i % STAGES;
    const uint32_t bar = bar0 + 8 * s;
    ptx::mbar_arrive_expect_tx(bar, kTileBytes);
#pragma unroll
    for (int c = 0; c < kSub; ++c)
      ptx::tma_load_2d(sbase + s * kTileBytes + c * (BN * 128), &tmap_kv, bar, c * 64, row, ptx::kEvictFirst);
  };
  // stage Q: row r = head head0 + r; columns [0, 512) from q_lat, [512, 576) from q_rope; rows >= `rows` are zero
  for (int i = threadIdx.x; i < 16 * (kRow / 8); i += blockDim.x) {
    const int r = i / (kRow / 8), c = i % (kRow / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < rows) {
      // row strides in elements: the two query parts may be column slices of one wider projection output
      v = c < kLat / 8 ? reinterpret_cast<const uint4*>(q_lat + seq * q_lat_stride + static_cast<int64_t>(head0 + r) * kLat)[c]
                       : reinterpret_cast<const uint4*>(q_rope + seq * q_rope_stride + static_cast<int64_t>(head0 + r) * kRope)[c - kLat / 8];
    }
    // plain row-major with an XOR on the low 3 chunk bits to spread ldmatrix rows over banks
    reinterpret_cast<uint4*>(q_gen)[r * (kRow / 8) + ((c & ~7) | ((c & 7) ^ (r & 7)))] = v;
  }
  __syncthreads();
  if (threadIdx.x == 0)
    for (int i = 0; i < STAGES - 1 && i < n_tiles; ++i) issue(i);

  // this warp's slice of the 576-wide dot product: 9 k-steps of 16
  uint32_t qf[9][4];
#pragma unroll
  for (int kk = 0; kk < 9; ++kk) {
    const int row = lane & 15, chunk = (warp * 9 + kk) * 2 + (lane >> 4);
    const uint32_t a = q_sm + static_cast<uint32_t>((row * (kRow / 8) + ((chunk & ~7) | ((chunk & 7) ^ (row & 7)))) * 16);
    ldsm_x4(a, qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
  }
  float o[16][4];
#pragma unroll
  for (int d = 0; d < 16; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.0f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
  const int g = lane >> 2, t4 = lane & 3;
  const int max_lo = g < rows ? ctx - 1 : -1, max_hi = g + 8 < rows ? ctx - 1 : -1;

  bool ok = true;
  for (int i = 0; i < n_tiles; ++i) {
    const int st = i % STAGES;
    if (!ptx::mbar_wait(bar0 + 8 * st, (i / STAGES) & 1)) {
      status_record(status, kTimeout, kSiteAttn, seq, i);
      sh_fail = 1;
    }
    const uint32_t kb = sbase + st * kTileBytes;
    const int kv0 = (tile_begin + i) * BN;
    // ---- partial S over this warp's 144 dims ----
    float s[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
    {
#pragma unroll
      for (int kk = 0; kk < 9; ++kk) {
#pragma unroll
        for (int jp = 0; jp < 2; ++jp) {
          uint32_t b0, b1, b2, b3;
          const int row = jp * 16 + (lane & 7) + ((lane >> 4) << 3);
          const int chunk = (warp * 9 + kk) * 2 + ((lane >> 3) & 1);
          ldsm_x4(kv_addr(kb, row, chunk), b0, b1, b2, b3);
          mma16816(s[2 * jp], qf[kk], b0, b1);
          mma16816(s[2 * jp + 1], qf[kk], b2, b3);
        }
      }
    }
    float* mine = s_red + ((i & 1) * 4 + warp) * 512;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      *reinterpret_cast<float2*>(mine + g * 32 + j * 8 + 2 * t4) = make_float2(s[j][0], s[j][1]);
      *reinterpret_cast<float2*>(mine + (g + 8) * 32 + j * 8 + 2 * t4) = make_float2(s[j][2], s[j][3]);
    }
    __syncthreads();  // every warp has finished the previous tile's P.V as well: its stage can be refilled
    if (sh_fail != 0) { ok = false; break; }
    if (threadIdx.x == 0 && i + STAGES - 1 < n_tiles) issue(i + STAGES - 1);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 lo = make_float2(0.f, 0.f), hi = make_float2(0.f, 0.f);
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float* src = s_red + ((i & 1) * 4 + w) * 512;
        const float2 a = *reinterpret_cast<const float2*>(src + g * 32 + j * 8 + 2 * t4);
        const float2 b = *reinterpret_cast<const float2*>(src + (g + 8) * 32 + j * 8 + 2 * t4);
        lo.x += a.x; lo.y += a.y; hi.x += b.x; hi.y += b.y;
      }
      s[j][0] = lo.x; s[j][1] = lo.y; s[j][2] = hi.x; s[j][3] = hi.y;
    }
    // ---- online softmax (identical in all four warps) ----
    float mx_lo = m[0], mx_hi = m[1];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = kv0 + j * 8 + 2 * t4;
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
    const float sub_lo = mx_lo == -INFINITY ? 0.0f : mx_lo, sub_hi = mx_hi == -INFINITY ? 0.0f : mx_hi;
    const float corr_lo = ptx::ex2(m[0] - sub_lo), corr_hi = ptx::ex2(m[1] - sub_hi);
    m[0] = mx_lo;
    m[1] = mx_hi;
    float sum_lo = 0.0f, sum_hi = 0.0f;
    uint32_t pf[4][2];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
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
    for (int d = 0; d < 16; ++d) {
      o[d][0] *= corr_lo; o[d][1] *= corr_lo;
      o[d][2] *= corr_hi; o[d][3] *= corr_hi;
    }
    // ---- O[:, 128 w : 128 w + 128] += P . C ----
    const int valid = ctx - kv0;  // rows of the tile inside the context; beyond that the page holds stale data
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
      const uint32_t a[4] = {pf[2 * kk][0], pf[2 * kk][1], pf[2 * kk + 1][0], pf[2 * kk + 1][1]};
#pragma unroll
      for (int dp = 0; dp < 8; ++dp) {
        uint32_t b0, b1, b2, b3;
        const int row = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
        const int chunk = warp * 16 + dp * 2 + (lane >> 4);
        ldsm_x4_t(kv_addr(kb, row, chunk), b0, b1, b2, b3);
        if (valid < BN) {
          // P is exactly zero for masked tokens, but 0 * NaN is NaN: blank operand rows past the context.
          // After the transposing load, register b0/b2 hold tokens kk*16 + 2*t4 (+1), b1/b3 tokens +8.
          const int tk = kk * 16 + 2 * t4;
          const uint32_t keep0 = (tk < valid ? 0x0000ffffu : 0u) | (tk + 1 < valid ? 0xffff0000u : 0u);
          const uint32_t keep1 = (tk + 8 < valid ? 0x0000ffffu : 0u) | (tk + 9 < valid ? 0xffff0000u : 0u);
          b0 &= keep0; b2 &= keep0; b1 &= keep1; b3 &= keep1;
        }
        mma16816(o[2 * dp], a, b0, b1);
        mma16816(o[2 * dp + 1], a, b2, b3);
      }
    }
  }
  if (!ok) {
    for (int i = 0; i < STAGES; ++i) ptx::mbar_wait(bar0 + 8 * i, 0, 20000000ull) || ptx::mbar_wait(bar0 + 8 * i, 1, 20000000ull);
    return;
  }
  l[0] += __shfl_xor_sync(0xffffffffu, l[0], 1);
  l[0] += __shfl_xor_sync(0xffffffffu, l[0], 2);
  l[1] += __shfl_xor_sync(0xffffffffu, l[1], 1);
  l[1] += __shfl_xor_sync(0xffffffffu, l[1], 2);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = g + half * 8;
    if (r >= rows) continue;
    const int64_t h = static_cast<int64_t>(seq) * n_heads + head0 + r;
    if (num_splits == 1) {
      const float inv = l[half] > 0.0f ? 1.0f / l[half] : 0.0f;
      __nv_bfloat16* dst = out_lat + h * kLat + warp * 128;
#pragma unroll
      for (int d = 0; d < 16; ++d)
        *reinterpret_cast<uint32_t*>(dst + d * 8 + 2 * t4) = ptx::pack_bf16x2(o[d][half * 2] * inv, o[d][half * 2 + 1] * inv);
    } else {
      float* dst = workspace + (h * num_splits + split) * (kLat + 2);
#pragma unroll
      for (int d = 0; d < 16; ++d)
        *reinterpret_cast<float2*>(dst + warp * 128 + d * 8 + 2 * t4) = make_float2(o[d][half * 2], o[d][half * 2 + 1]);
      if (warp == 0 && t4 == 0) {
        dst[kLat] = m[half];
        dst[kLat + 1] = l[half];
      }
    }
  }
}

__global__ void mla_reduce_kernel(const float* __restrict__ workspace, __nv_bfloat16* __restrict__ out, int num_splits, int total) {
  constexpr int RS = kLat + 2;
  const int idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (idx >= total) return;
  const float* base = workspace + static_cast<int64_t>(idx) * num_splits * RS;
  float mm = -INFINITY;
  for (int s = 0; s < num_splits; ++s) mm = fmaxf(mm, base[s * RS + kLat]);
  const float sub = mm == -INFINITY ? 0.0f : mm;
  float ll = 0.0f, acc[kLat / 32];
#pragma unroll
  for (int c = 0; c < kLat / 32; ++c) acc[c] = 0.0f;
  for (int s = 0; s < num_splits; ++s) {
    const float f = ptx::ex2(base[s * RS + kLat] - sub);
    ll += base[s * RS + kLat + 1] * f;
#pragma unroll
    for (int c = 0; c < kLat / 32; ++c) acc[c] += base[s * RS + c * 32 + lane] * f;
  }
  const float inv = ll > 0.0f ? 1.0f / ll : 0.0f;
#pragma unroll
  for (int c = 0; c < kLat / 32; ++c) out[static_cast<int64_t>(idx) * kLat + c * 32 + lane] = __float2bfloat16(acc[c] * inv);
}

// One thread block per sequence: expand (cu_q, ctx_lens) into per-token rows for the attention kernel.
// Token i of a sequence with q_len new tokens and `ctx` tokens in total sees ctx - q_len + i + 1 positions.
__global__ void mla_rows_meta_kernel(const int32_t* __restrict__ cu_q, const int32_t* __restrict__ ctx_lens,
                                     int32_t* __restrict__ row_ctx, int32_t* __restrict__ row_seq) {
  const int b = blockIdx.x;
  const int t0 = cu_q[b], q_len = cu_q[b + 1] - t0, ctx = ctx_lens[b];
  for (int i = threadIdx.x; i < q_len; i += blockDim.x) {
    row_ctx[t0 + i] = max(0, ctx - q_len + i + 1);
    row_seq[t0 + i] = b;
  }
}

}  // namespace
}  // namespace b2

using namespace b2;

extern "C" int64_t b2_mla_decode_workspace(int batch, int n_heads, int num_splits) {
  return static_cast<int64_t>(batch) * n_heads * num_splits * (kLat + 2) * 4;
}

extern "C" int b2_mla_rows_meta(const int32_t* cu_q, const int32_t* ctx_lens, int num_seqs, int32_t* row_ctx, int32_t* row_seq,
                                cudaStream_t stream) {
  if (num_seqs <= 0) return 0;
  mla_rows_meta_kernel<<<num_seqs, 128, 0, stream>>>(cu_q, ctx_lens, row_ctx, row_seq);
  return last_launch_rc();
}

extern "C" int b2_mla_attend_bf16(const void* q_lat, const void* q_rope, const void* kv_cache, void* out_lat,
                                  const int32_t* row_ctx, const int32_t* block_tables, const int32_t* row_seq, float* workspace,
                                  int rows, int max_blocks, int n_heads, int page_size, int num_splits, float scale,
                                  int64_t num_pages, int64_t q_lat_stride, int64_t q_rope_stride, Status* status,
                                  cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (n_heads <= 0 || page_size % BN != 0 || num_splits < 1 || (num_splits > 1 && workspace == nullptr)) return -kBadArgument;
  // 16-byte vector loads of the query rows
  if (q_lat_stride % 8 != 0 || q_rope_stride % 8 != 0 || (reinterpret_cast<uintptr_t>(q_lat) & 15) != 0 ||
      (reinterpret_cast<uintptr_t>(q_rope) & 15) != 0)
    return -kBadArgument;
  CUtensorMap tk;
  const uint64_t cache_rows = static_cast<uint64_t>(num_pages) * page_size;
  if (!make_tmap_2d(&tk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, kv_cache, cache_rows, kRow, kRow * 2, BN, 64, CU_TENSOR_MAP_SWIZZLE_128B))
    return -kBadArgument;
  // two-stage ring (two CTAs per SM) unless B2_MLA_STAGES=3 asks for the deep one
  static const int forced = [] {
    const char* e = getenv("B2_MLA_STAGES");
    return e != nullptr ? atoi(e) : 0;
  }();
  const int stages = forced == 3 ? 3 : 2;
  const int SMEM = stages * kTileBytes + 16 * kRow * 2 + 2 * 4 * 16 * 32 * 4 + 64 + 1024;
  auto kern = stages == 2 ? mla_decode_kernel<2> : mla_decode_kernel<3>;
  static DeviceOnce attr_once[2];
  if (const int rc = attr_once[stages - 2].max_smem(kern, SMEM)) return rc;
  // grid z is limited to 65535: larger row counts go out in slices
  constexpr int kMaxZ = 65535;
  for (int r0 = 0; r0 < rows; r0 += kMaxZ) {
    const int n = rows - r0 < kMaxZ ? rows - r0 : kMaxZ;
    dim3 grid(num_splits, (n_heads + 15) / 16, n);
    float* ws = workspace == nullptr ? nullptr : workspace + static_cast<int64_t>(r0) * n_heads * num_splits * (kLat + 2);
    __nv_bfloat16* out = static_cast<__nv_bfloat16*>(out_lat) + static_cast<int64_t>(r0) * n_heads * kLat;
    kern<<<grid, 128, SMEM, stream>>>(
        tk, static_cast<const __nv_bfloat16*>(q_lat) + r0 * q_lat_stride, static_cast<const __nv_bfloat16*>(q_rope) + r0 * q_rope_stride,
        out, row_ctx + r0, row_seq == nullptr ? block_tables + static_cast<int64_t>(r0) * max_blocks : block_tables,
        row_seq == nullptr ? nullptr : row_seq + r0, ws, max_blocks, n_heads, page_size,
        num_splits, scale * ptx::kLog2e, num_pages, q_lat_stride, q_rope_stride, status);
    if (num_splits > 1) {
      const int total = n * n_heads;
      mla_reduce_kernel<<<(total + 3) / 4, 128, 0, stream>>>(ws, out, num_splits, total);
    }
  }
  return last_launch_rc();
}

extern "C" int b2_mla_decode_bf16(const void* q_lat, const void* q_rope, const void* kv_cache, void* out_lat,
                                  const int32_t* ctx_lens, const int32_t* block_tables, float* workspace, int batch,
                                  int max_blocks, int n_heads, int page_size, int num_splits, float scale,
                                  int64_t num_pages, Status* status, cudaStream_t stream) {
  return b2_mla_attend_bf16(q_lat, q_rope, kv_cache, out_lat, ctx_lens, block_tables, nullptr, workspace, batch, max_blocks,
                            n_heads, page_size, num_splits, scale, num_pages, static_cast<int64_t>(n_heads) * kLat,
                            static_cast<int64_t>(n_heads) * kRope, status, stream);
}
