// Block-scaled fp8 GEMM on tcgen05 (kind::f8f6f4):
//   Y[M, N] = sum over 128-wide K blocks kb of  sx[m, kb] * sw[n / 128, kb] * (Xq[m, kb-block] . Wq[n, kb-block])
// Xq: e4m3 [M, K] with one f32 scale per row per 128 columns (dynamic activation quantisation);
// Wq: e4m3 [N, K] with one f32 scale per 128 x 128 block (checkpoint format). bf16 out.
//
// A 128-byte shared-memory row holds exactly one scale block of K, so every pipeline stage is one scale block:
// the MMA warp issues its four K=32 instructions into a fresh TMEM slab (no accumulation across stages) and
// commits; the four promotion warps pull the slab out of TMEM, multiply by the two scales and accumulate in f32
// registers - the fp8 types accumulate in f32 (stdlib/src/utils/numerics.mojo:1031-1054). Slabs are
// multi-buffered so the promotion of block kb overlaps the MMA of block kb + 1. The reference rejects fp8 on this
// architecture outright (stdlib/src/builtin/simd.mojo:186-189), so there is no reference kernel to compare to.
//
// Operand assignment as in the bf16 GEMM: normal (tokens on the UMMA M side) or swapped (weight rows on the M
// side, tokens as UMMA N) for decode-sized M.
#include <cstdint>
#include <cuda.h>
#include <cuda_bf16.h>
#include "b2/api.h"
#include "b2/launch.h"
#include "b2/gemm_tc.cuh"
#include "b2/ptx.cuh"
#include "b2/tma.h"
#include "b2/tp.h"
#include "b2/tp_ag.cuh"
#include "b2/tp_rs.cuh"

namespace b2 {
namespace {

constexpr int kThreads = 192;

struct Fp8Params {
  __nv_bfloat16* y;
  int64_t ldy;
  const float* sx;  // [M, KB]
  const float* sw;  // [ceil(N / 128), KB]
  int M, N, KB;
  int p_blocks, q_blocks;
  // split-K (plain mode only): work item w = tile * splits + split covers k-blocks [split * KB / splits,
  // (split + 1) * KB / splits); partial tiles go to `partials` as f32 [tile][split][BN][128] and the CTA that
  // arrives last at the tile's counter adds them up in split order and stores the result
  int splits;
  float* partials;
  uint32_t* counters;   // [tiles], zero on entry and on exit
};

// What the tensor-parallel variants add to the plain kernel (see tp_fused.cu for the protocols).
struct Fp8Fused {
  tp::RsParams rs;     // kModeRs
  tp::AgParams ag;     // kModeAg
  tp::AgSched ag_sched;
  tp::EpochCtl ectl;
  int n_gemm;          // CTAs [0, n_gemm) run the GEMM; the rest only reduce (RS) or only move data (AG)
};
constexpr int kModePlain = 0;
// Row-parallel GEMM fused with reduce-scatter / all-reduce: finished tiles go to the owner rank's staging buffer,
// CTAs >= n_gemm only reduce, the others join the reduction after their tiles.
constexpr int kModeRs = 1;
// All-gather fused with the column-parallel GEMM: CTAs >= n_gemm push this rank's quantised rows and their scales
// to every peer chunk by chunk; the GEMM producer waits for the chunks a tile needs before its first load.
constexpr int kModeAg = 2;

// WG2 = true: eight promotion warps, two threads per accumulator row, each owning BN / 2 columns of every slab.
// Two warps per scheduler hide each other's tcgen05.ld and FMA latency, which one warp per scheduler cannot
// (measured: with four warps the tensor pipe idles 58 % of the time waiting for slabs to be promoted).
template <int BN, int STAGES, int SLABS, bool SWAP, int MODE, bool WG2>
__global__ void __launch_bounds__(WG2 ? kThreads + 128 : kThreads, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmap_p, const __grid_constant__ CUtensorMap tmap_q, Fp8Params prm,
                const __grid_constant__ tp::RsSched rs_sched, const __grid_constant__ Fp8Fused fz, Status* status) {
  ptx::grid_dep_sync();
  constexpr bool RS = MODE == kModeRs;
  constexpr bool AG = MODE == kModeAg;
  static_assert(!(RS && WG2), "the fused reduce-scatter epilogue is written for four epilogue warps");
  static_assert(!WG2 || BN >= 64, "column halves must be whole tcgen05.ld chunks");
  constexpr int NW = WG2 ? 8 : 4;            // promotion warps
  constexpr int COLS = WG2 ? BN / 2 : BN;    // accumulator columns per thread
  tp::RsParams rs = fz.rs;
  tp::AgParams ag = fz.ag;
  const tp::EpochCtl ectl = fz.ectl;
  const int n_gemm = fz.n_gemm;
  uint32_t epoch = 0;
  if (RS || AG) epoch = tp::epoch_begin(ectl);
  rs.epoch = epoch;
  ag.epoch = epoch;
  const int my_cta = static_cast<int>(blockIdx.x);
  const int n_ctas = (RS || AG) ? n_gemm : static_cast<int>(gridDim.x);
  if (AG && my_cta >= n_gemm) {
    extern __shared__ uint8_t smem_comm[];
    uint8_t* win = smem_comm + ((128 - (reinterpret_cast<uintptr_t>(smem_comm) & 127)) & 127);
    tp::ag_push(ag, my_cta - n_gemm, win, status);
    tp::epoch_end(ectl, epoch);
    return;
  }
  auto tile_of = [&](int w, int& pb, int& qb) {
    if (RS) {
      const gemm::WorkUnit u = rs_sched.get(w);
      pb = u.pb;
      qb = u.qb;
    } else if (AG) {
      const gemm::WorkUnit u = fz.ag_sched.get(w);
      pb = u.pb;
      qb = u.qb;
    } else {
      const int t = w / prm.splits;
      pb = t / prm.q_blocks;
      qb = t % prm.q_blocks;
    }
  };
  auto kb_range = [&](int w, int& kb0, int& kb1) {
    kb0 = 0;
    kb1 = prm.KB;
    if (MODE == kModePlain && prm.splits > 1) {
      const int sp = w % prm.splits;
      kb0 = sp * prm.KB / prm.splits;
      kb1 = (sp + 1) * prm.KB / prm.splits;
    }
  };
  if (!RS || my_cta < n_gemm) {
  constexpr int kPBytes = 128 * 128, kQBytes = BN * 128, kStageBytes = kPBytes + kQBytes;
  constexpr int kTmemCols = (SLABS * BN <= 32) ? 32 : (SLABS * BN <= 64) ? 64 : (SLABS * BN <= 128) ? 128 : (SLABS * BN <= 256) ? 256 : 512;
  constexpr int CH = BN >= 32 ? 32 : 16;
  constexpr int kRingAndBarriers = STAGES * kStageBytes + (2 * STAGES + 2 * SLABS + 1) * 8 + 16 + NW * BN * 4 + 1024 + 64;
  constexpr uint32_t idesc = ptx::make_idesc(0, 0, 128, BN);  // e4m3 x e4m3 -> f32
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + STAGES * kStageBytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto slab_full = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };
  auto slab_empty = [&](int s) { return bar_base + 8u * (2 * STAGES + SLABS + s); };
  const uint32_t drain_bar = bar_base + 8u * (2 * STAGES + 2 * SLABS);
  const uint32_t holder = bar_base + 8u * (2 * STAGES + 2 * SLABS + 1);
  uint32_t* holder_ptr = reinterpret_cast<uint32_t*>(smem_raw + (holder - ptx::smem_u32(smem_raw)));
  float* col_scale = reinterpret_cast<float*>(smem_raw + (holder + 16 - ptx::smem_u32(smem_raw)));  // [4 warps][BN], swapped layout

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    ptx::prefetch_tensormap(&tmap_p);
    ptx::prefetch_tensormap(&tmap_q);
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < SLABS; ++s) {
      ptx::mbar_init(slab_full(s), 1);
      ptx::mbar_init(slab_empty(s), NW);
    }
    ptx::mbar_init(drain_bar, 1);
    ptx::fence_mbar_init();
  }
  if (warp == 1) {
    ptx::tmem_alloc(holder, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *holder_ptr;
  const int total = prm.p_blocks * prm.q_blocks * (MODE == kModePlain ? prm.splits : 1);
  const int KB = prm.KB;

  if (warp == 0) {
    if (ptx::elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      long issued = 0;
      bool ok = true;
      for (int w = my_cta; ok && w < total; w += n_ctas) {
        int pb, qb;
        tile_of(w, pb, qb);
        if constexpr (AG) {
          gemm::WorkUnit u{};
          u.pb = pb;
          u.qb = qb;
          if (!tp::AgGate{ag, SWAP, BN}(u, status)) { ok = false; break; }
        }
        int kb0, kb1;
        kb_range(w, kb0, kb1);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1u)) {
            status_record(status, kTimeout, kSiteGemmEmpty, w, kb);
            ok = false;
            break;
          }
          const uint32_t sp = smem_base + stage * kStageBytes;
          ptx::mbar_arrive_expect_tx(full_bar(stage), kStageBytes);
          ptx::tma_load_2d(sp, &tmap_p, full_bar(stage), kb * 128, pb * 128, SWAP ? ptx::kEvictFirst : ptx::kEvictNormal);
          ptx::tma_load_2d(sp + kPBytes, &tmap_q, full_bar(stage), kb * 128, qb * BN, SWAP ? ptx::kEvictLast : ptx::kEvictNormal);
          ++issued;
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        long pending = issued < STAGES ? issued : STAGES;
        int s = stage;
        uint32_t ph = phase;
        for (long i = 0; i < pending; ++i) {
          if (--s < 0) { s = STAGES - 1; ph ^= 1u; }
          if (!ptx::mbar_wait(full_bar(s), ph, 200000000ull)) break;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (ptx::elect_one()) {
      int stage = 0, slab = 0;
      uint32_t phase = 0, slab_phase = 0;
      bool ok = true;
      for (int w = my_cta; ok && w < total; w += n_ctas) {
        int kb0, kb1;
        kb_range(w, kb0, kb1);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!ptx::mbar_wait(slab_empty(slab), slab_phase ^ 1u)) {
            status_record(status, kTimeout, kSiteGemmTmemEmpty, w, kb);
            ok = false;
            break;
          }
          if (!ptx::mbar_wait(full_bar(stage), phase)) {
            status_record(status, kTimeout, kSiteGemmFull, w, kb);
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          const uint32_t sp = smem_base + stage * kStageBytes;
          const uint64_t da = ptx::make_smem_desc_sw128(sp);
          const uint64_t db = ptx::make_smem_desc_sw128(sp + kPBytes);
          const uint32_t d_tmem = tmem_base + slab * BN;
#pragma unroll
          for (int k = 0; k < 4; ++k) ptx::tc_mma_f8(d_tmem, da + 2u * k, db + 2u * k, idesc, k > 0 ? 1u : 0u);
          ptx::tc_commit(empty_bar(stage));
          ptx::tc_commit(slab_full(slab));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          if (++slab == SLABS) { slab = 0; slab_phase ^= 1u; }
        }
      }
      if (!ok) {
        ptx::tc_commit(drain_bar);
        ptx::mbar_wait(drain_bar, 0, 200000000ull);
      }
    }
    __syncwarp();
  } else {
    // ---- promotion + epilogue warps ----
    const int quarter = warp & 3;
    const int p_local = quarter * 32 + lane;
    const int col_base = WG2 ? ((warp - 2) >> 2) * COLS : 0;   // first accumulator column of this thread
    int slab = 0;
    uint32_t slab_phase = 0;
    bool ok = true;
    for (int w = my_cta; ok && w < total; w += n_ctas) {
      int pb, qb;
      tile_of(w, pb, qb);
      float acc[COLS];
#pragma unroll
      for (int j = 0; j < COLS; ++j) acc[j] = 0.0f;
      const int row = pb * 128 + p_local;  // m (normal) or n (swapped)
      int kb0, kb1;
      kb_range(w, kb0, kb1);
      for (int kb = kb0; kb < kb1; ++kb) {
        // scale(s) for this k-block. With the fused all-gather the token scales of a tile arrive from peers and
        // are only known to be in place once the tile's first slab is full (the producer passed the chunk gate
        // before it loaded the operands), so they are read after the wait, past L1.
        float s_row = 0.0f, s_blk0 = 0.0f, s_blk1 = 0.0f;
        auto load_scales = [&]() {
          if constexpr (!SWAP) {
            if (row < prm.M) s_row = AG ? __ldcg(prm.sx + static_cast<int64_t>(row) * KB + kb) : prm.sx[static_cast<int64_t>(row) * KB + kb];
            const int nb = (qb * BN) >> 7;
            s_blk0 = prm.sw[static_cast<int64_t>(nb) * KB + kb];
            if (BN > 128) s_blk1 = ((qb * BN + 128) < prm.N) ? prm.sw[static_cast<int64_t>(nb + 1) * KB + kb] : 0.0f;
          } else {
            s_row = prm.sw[static_cast<int64_t>(pb) * KB + kb];  // 128 weight rows = one scale block
            // each warp stages the token scales it needs itself: no barrier that a failed warp could strand
            float* cs = col_scale + (warp - 2) * BN;
            __syncwarp();
            for (int j = lane; j < BN; j += 32) {
              const int m = qb * BN + j;
              const float* src = prm.sx + static_cast<int64_t>(m) * KB + kb;
              cs[j] = m < prm.M ? (AG ? __ldcg(src) : *src) : 0.0f;
            }
            __syncwarp();
          }
        };
        if constexpr (!AG) load_scales();
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(slab_full(slab), slab_phase))) {
          if (lane == 0) status_record(status, kTimeout, kSiteGemmTmemFull, w, kb);
          ok = false;
          break;
        }
        if constexpr (AG) load_scales();
        ptx::tc_fence_after();
        const uint32_t taddr = tmem_base + slab * BN + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll
        for (int c = 0; c < COLS / CH; ++c) {
          uint32_t r[CH];
          if constexpr (CH == 32) ptx::tmem_ld_32x32(taddr + col_base + c * CH, r);
          else ptx::tmem_ld_32x16(taddr + col_base + c * CH, r);
          ptx::tc_wait_ld();
          if constexpr (!SWAP) {
            const float s = s_row * ((col_base + c * CH) < 128 ? s_blk0 : s_blk1);
#pragma unroll
            for (int j = 0; j < CH; ++j) acc[c * CH + j] = fmaf(__uint_as_float(r[j]), s, acc[c * CH + j]);
          } else {
            const float* cs = col_scale + (warp - 2) * BN + col_base + c * CH;
#pragma unroll
            for (int j = 0; j < CH; ++j) acc[c * CH + j] = fmaf(__uint_as_float(r[j]), s_row * cs[j], acc[c * CH + j]);
          }
        }
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(slab_empty(slab));
        if (++slab == SLABS) { slab = 0; slab_phase ^= 1u; }
      }
      // the fused epilogue below synchronises the four warps, so they must agree on whether it runs
      if constexpr (RS) ok = ptx::named_barrier_and(3, 128, ok);
      if constexpr (MODE == kModePlain) {
        if (prm.splits > 1) ok = ptx::named_barrier_and(2, NW * 32, ok);   // the hand-over below synchronises all promotion warps
      }
      if (!ok) break;
      if constexpr (MODE == kModePlain) {
        if (prm.splits > 1) {
          const int tile = w / prm.splits, sp = w % prm.splits;
          float* ws_tile = prm.partials + static_cast<size_t>(tile) * prm.splits * BN * 128;
          float* mine = ws_tile + static_cast<size_t>(sp) * BN * 128 + p_local;
#pragma unroll
          for (int j = 0; j < COLS; ++j) __stcg(mine + (col_base + j) * 128, acc[j]);
          __threadfence();
          ptx::named_barrier_sync(2, NW * 32);
          if (threadIdx.x == 64) {  // first promotion thread
            const uint32_t old = atomicAdd(prm.counters + tile, 1u);
            const bool last = old == static_cast<uint32_t>(prm.splits - 1);
            if (last) prm.counters[tile] = 0;  // ready for the next launch
            __threadfence();
            holder_ptr[2] = last ? 1u : 0u;
          }
          ptx::named_barrier_sync(2, NW * 32);
          const bool last = holder_ptr[2] != 0;
          ptx::named_barrier_sync(2, NW * 32);  // the flag word is rewritten by the next work item
          if (!last) continue;
#pragma unroll
          for (int j = 0; j < COLS; ++j) acc[j] = 0.0f;
          for (int sidx = 0; sidx < prm.splits; ++sidx) {
            const float* src = ws_tile + static_cast<size_t>(sidx) * BN * 128 + p_local;
#pragma unroll
            for (int j = 0; j < COLS; ++j) acc[j] += __ldcg(src + (col_base + j) * 128);
          }
        }
      }
      // ---- store ----
      if constexpr (RS) {
        extern __shared__ uint8_t smem_dyn[];
        uint8_t* epi_buf = smem_dyn + kRingAndBarriers;
        epi_buf += (16 - (reinterpret_cast<uintptr_t>(epi_buf) & 15)) & 15;
        tp::RsEpilogue<BN, SWAP> writer{rs, epi_buf};
        gemm::WorkUnit u{};
        u.pb = pb;
        u.qb = qb;
        writer.write_tile(u, quarter, lane, [&](int col0, uint32_t (&r)[CH]) {
#pragma unroll
          for (int j = 0; j < CH; ++j) r[j] = __float_as_uint(acc[col0 + j]);
        });
      } else if constexpr (!SWAP) {
        if (row < prm.M) {
          __nv_bfloat16* dst = prm.y + static_cast<int64_t>(row) * prm.ldy + qb * BN + col_base;
#pragma unroll
          for (int g = 0; g < COLS / 8; ++g) {
            if (qb * BN + col_base + g * 8 >= prm.N) break;
            uint4 pk;
            pk.x = ptx::pack_bf16x2(acc[g * 8 + 0], acc[g * 8 + 1]);
            pk.y = ptx::pack_bf16x2(acc[g * 8 + 2], acc[g * 8 + 3]);
            pk.z = ptx::pack_bf16x2(acc[g * 8 + 4], acc[g * 8 + 5]);
            pk.w = ptx::pack_bf16x2(acc[g * 8 + 6], acc[g * 8 + 7]);
            ptx::st_v4(dst + g * 8, pk);
          }
        }
      } else {
        if (row < prm.N) {
#pragma unroll
          for (int j = 0; j < COLS; ++j) {
            const int m = qb * BN + col_base + j;
            if (m >= prm.M) break;
            prm.y[static_cast<int64_t>(m) * prm.ldy + row] = __float2bfloat16(acc[j]);
          }
        }
      }
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
  }  // GEMM CTAs
  if constexpr (RS) {
    tp::reduce_phase<BN, SWAP>(rs, status);
    tp::rs_epoch_end(ectl, rs);
  }
  if constexpr (AG) tp::epoch_end(ectl, epoch);
}

template <int BN, bool SWAP>
int launch_fp8(const void* xq, const float* xs, const void* wq, const float* ws, void* y, int M, int N, int K, int64_t ldy,
               int splits, void* workspace, int64_t workspace_bytes, Status* status, cudaStream_t stream) {
  constexpr int kStageBytes = 128 * 128 + BN * 128;
  constexpr int STAGES = (190 * 1024 / kStageBytes) > 8 ? 8 : (190 * 1024 / kStageBytes);
  constexpr int SLABS = BN <= 128 ? 4 : 2;
  constexpr bool WG2 = BN >= 64;
  constexpr int SMEM = STAGES * kStageBytes + (2 * STAGES + 2 * SLABS + 1) * 8 + 16 + (WG2 ? 8 : 4) * BN * 4 + 1024 + 64;
  const void* p_ptr = SWAP ? wq : xq;
  const void* q_ptr = SWAP ? xq : wq;
  const int rows_p = SWAP ? N : M, rows_q = SWAP ? M : N;
  CUtensorMap tp, tq;
  if (!make_tmap_2d(&tp, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p_ptr, rows_p, K, K, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B) ||
      !make_tmap_2d(&tq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, q_ptr, rows_q, K, K, BN, 128, CU_TENSOR_MAP_SWIZZLE_128B))
    return -kBadArgument;
  Fp8Params prm{};
  prm.y = static_cast<__nv_bfloat16*>(y);
  prm.ldy = ldy;
  prm.sx = xs;
  prm.sw = ws;
  prm.M = M;
  prm.N = N;
  prm.KB = K / 128;
  prm.p_blocks = (rows_p + 127) / 128;
  prm.q_blocks = (rows_q + BN - 1) / BN;
  prm.splits = 1;
  {
    const int64_t tiles = static_cast<int64_t>(prm.p_blocks) * prm.q_blocks;
    const int64_t counters_bytes = 65536 * 4;   // same workspace convention as the bf16 GEMM: semaphores, then partial tiles
    if (splits == 0) {
      // automatic: split only when the tiles leave at least half of the SMs idle, at least four k-blocks per split
      splits = 1;
      if (workspace != nullptr && tiles * 2 <= kNumSMs && prm.KB >= 8) {
        splits = static_cast<int>(kNumSMs / tiles);
        if (splits > prm.KB / 4) splits = prm.KB / 4;
        if (splits > 8) splits = 8;
      }
    }
    if (splits > prm.KB) splits = prm.KB;
    if (splits > 1) {
      const int64_t need = counters_bytes + tiles * splits * BN * 128 * 4;
      if (workspace == nullptr || workspace_bytes < need || tiles > 65536) return -kTooLarge;
      prm.splits = splits;
      prm.counters = static_cast<uint32_t*>(workspace);
      prm.partials = reinterpret_cast<float*>(static_cast<char*>(workspace) + counters_bytes);
    }
  }
  auto kern = gemm_fp8_kernel<BN, STAGES, SLABS, SWAP, kModePlain, WG2>;
  static DeviceOnce attr_once;
  if (const int rc = attr_once.run([&] {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        return e;
      }))
    return rc;
  const int total = prm.p_blocks * prm.q_blocks * prm.splits;
  static const tp::RsSched no_sched{};
  static const Fp8Fused no_fused{};
  launch_pdl(kern, dim3(total < kNumSMs ? total : kNumSMs), dim3(WG2 ? kThreads + 128 : kThreads), SMEM, stream, tp, tq, prm, no_sched, no_fused, status);
  return last_launch_rc();
}

template <int BN, bool SWAP>
int launch_fp8_rs(const void* xq, const float* xs, const void* wq, const float* ws, int M, int N, int K, tp::RsParams rs,
                  tp::EpochCtl ectl, Status* status, cudaStream_t stream) {
  constexpr int kStageBytes = 128 * 128 + BN * 128;
  constexpr int STAGES = (150 * 1024 / kStageBytes) > 8 ? 8 : (150 * 1024 / kStageBytes);
  constexpr int SLABS = BN <= 128 ? 4 : 2;
  constexpr int SMEM = STAGES * kStageBytes + (2 * STAGES + 2 * SLABS + 1) * 8 + 16 + 4 * BN * 4 + 1024 + 64 + tp::rs_epi_bytes<BN, SWAP>() + 16;
  const void* p_ptr = SWAP ? wq : xq;
  const void* q_ptr = SWAP ? xq : wq;
  const int rows_p = SWAP ? N : M, rows_q = SWAP ? M : N;
  CUtensorMap tmp, tmq;
  if (!make_tmap_2d(&tmp, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p_ptr, rows_p, K, K, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B) ||
      !make_tmap_2d(&tmq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, q_ptr, rows_q, K, K, BN, 128, CU_TENSOR_MAP_SWIZZLE_128B))
    return -kBadArgument;
  Fp8Params prm{};
  prm.sx = xs;
  prm.sw = ws;
  prm.M = M;
  prm.N = N;
  prm.KB = K / 128;
  prm.p_blocks = (rows_p + 127) / 128;
  prm.q_blocks = (rows_q + BN - 1) / BN;
  tp::RsSched sched{};
  sched.p_blocks = prm.p_blocks;
  sched.q_blocks = prm.q_blocks;
  sched.num_kb = prm.KB;
  sched.bn = BN;
  sched.swap = SWAP;
  constexpr int TM = SWAP ? BN : 128;
  sched.m_tiles = SWAP ? sched.q_blocks : sched.p_blocks;
  if (!tp::build_rs_order(sched, rs.tp, rs.rank, rs.R, TM)) return -kTooLarge;
  rs.p_blocks = prm.p_blocks;
  rs.q_blocks = prm.q_blocks;
  auto kern = gemm_fp8_kernel<BN, STAGES, SLABS, SWAP, kModeRs, false>;
  static DeviceOnce attr_once;
  if (const int rc = attr_once.run([&] {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        return e;
      }))
    return rc;
  const int total = prm.p_blocks * prm.q_blocks;
  int n_gemm = kNumSMs - (rs.tp > 1 ? (M >= 2048 ? 4 : 12) : 0);
  if (total < n_gemm) n_gemm = total;
  Fp8Fused fz{};
  fz.rs = rs;
  fz.ectl = ectl;
  fz.n_gemm = n_gemm;
  launch_pdl(kern, dim3(kNumSMs), dim3(kThreads), SMEM, stream, tmp, tmq, prm, sched, fz, status);
  return last_launch_rc();
}

template <int BN, bool SWAP>
int launch_fp8_ag(const void* xq_all, const float* xs_all, const void* wq, const float* ws, void* y, int M, int N, int K, int64_t ldy,
                  tp::AgParams ag, tp::EpochCtl ectl, Status* status, cudaStream_t stream) {
  constexpr int kStageBytes = 128 * 128 + BN * 128;
  constexpr int STAGES = (190 * 1024 / kStageBytes) > 8 ? 8 : (190 * 1024 / kStageBytes);
  constexpr int SLABS = BN <= 128 ? 4 : 2;
  constexpr bool WG2 = BN >= 64;
  constexpr int SMEM_GEMM = STAGES * kStageBytes + (2 * STAGES + 2 * SLABS + 1) * 8 + 16 + (WG2 ? 8 : 4) * BN * 4 + 1024 + 64;
  constexpr int SMEM_COMM = tp::kAgRingBytes + 64 + 128;
  constexpr int SMEM = SMEM_GEMM > SMEM_COMM ? SMEM_GEMM : SMEM_COMM;
  const void* p_ptr = SWAP ? wq : xq_all;
  const void* q_ptr = SWAP ? xq_all : wq;
  const int rows_p = SWAP ? N : M, rows_q = SWAP ? M : N;
  CUtensorMap tmp, tmq;
  if (!make_tmap_2d(&tmp, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p_ptr, rows_p, K, K, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B) ||
      !make_tmap_2d(&tmq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, q_ptr, rows_q, K, K, BN, 128, CU_TENSOR_MAP_SWIZZLE_128B))
    return -kBadArgument;
  Fp8Params prm{};
  prm.y = static_cast<__nv_bfloat16*>(y);
  prm.ldy = ldy;
  prm.sx = xs_all;
  prm.sw = ws;
  prm.M = M;
  prm.N = N;
  prm.KB = K / 128;
  prm.p_blocks = (rows_p + 127) / 128;
  prm.q_blocks = (rows_q + BN - 1) / BN;
  Fp8Fused fz{};
  fz.ag = ag;
  fz.ectl = ectl;
  fz.ag_sched.p_blocks = prm.p_blocks;
  fz.ag_sched.q_blocks = prm.q_blocks;
  fz.ag_sched.num_kb = prm.KB;
  fz.ag_sched.bn = BN;
  fz.ag_sched.swap = SWAP;
  constexpr int TM = SWAP ? BN : 128;
  fz.ag_sched.m_tiles = SWAP ? prm.q_blocks : prm.p_blocks;
  fz.ag_sched.first_tile = (ag.rank * ag.R / TM) % fz.ag_sched.m_tiles;
  const int total = prm.p_blocks * prm.q_blocks;
  int n_gemm = kNumSMs - ag.n_comm;
  if (total < n_gemm) n_gemm = total;
  fz.n_gemm = n_gemm;
  auto kern = gemm_fp8_kernel<BN, STAGES, SLABS, SWAP, kModeAg, WG2>;
  static DeviceOnce attr_once;
  if (const int rc = attr_once.run([&] {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        return e;
      }))
    return rc;
  static const tp::RsSched no_sched{};
  launch_pdl(kern, dim3(n_gemm + ag.n_comm), dim3(WG2 ? kThreads + 128 : kThreads), SMEM, stream, tmp, tmq, prm, no_sched, fz, status);
  return last_launch_rc();
}

}  // namespace
}  // namespace b2

using namespace b2;

extern "C" int b2_gemm_fp8_block_ws(const void* xq, const float* xs, const void* wq, const float* ws, void* y, int M, int N,
                                    int K, int64_t ldy, int config, void* workspace, int64_t workspace_bytes, Status* status,
                                    cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 128 != 0 || N % 8 != 0) return -kBadArgument;
  bool swap = M <= 64;
  int bn = swap ? (M <= 16 ? 16 : M <= 32 ? 32 : 64) : 128;
  int splits = 0;   // automatic
  if (config != 0) {
    swap = (config >> 30) & 1;
    bn = config & 0xffff;
    splits = (config >> 16) & 0xff;
    if (splits == 0) splits = 1;
  }
  if (!swap && ldy % 8 != 0) return -kBadArgument;
#define B2_FP8(BN_, SWAP_) return launch_fp8<BN_, SWAP_>(xq, xs, wq, ws, y, M, N, K, ldy, splits, workspace, workspace_bytes, status, stream)
  if (swap) {
    switch (bn) {
      case 16: B2_FP8(16, true);
      case 32: B2_FP8(32, true);
      case 64: B2_FP8(64, true);
      case 128: B2_FP8(128, true);
      default: return -kBadArgument;
    }
  }
  switch (bn) {
    case 64: B2_FP8(64, false);
    case 128: B2_FP8(128, false);
    default: return -kBadArgument;
  }
#undef B2_FP8
}

extern "C" int b2_gemm_fp8_block(const void* xq, const float* xs, const void* wq, const float* ws, void* y, int M, int N,
                                 int K, int64_t ldy, int config, Status* status, cudaStream_t stream) {
  // without a workspace: explicit split-K configurations are refused, the automatic rule does not split
  return b2_gemm_fp8_block_ws(xq, xs, wq, ws, y, M, N, K, ldy, config, nullptr, 0, status, stream);
}

extern "C" int b2_tp_gemm_rs_fp8(const void* xq, const float* xs, const void* wq, const float* ws, const B2TpRegion* reg,
                                 const B2TpLayout* lay, void* out, const void* residual, int M, int N, int K, int mode, int slot,
                                 uint64_t timeout_ns, b2::Status* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (reg == nullptr || lay == nullptr || reg->tp < 1 || reg->tp > tp::kMaxTp || K % 128 != 0 || N % 8 != 0) return -kBadArgument;
  const int ntp = reg->tp;
  const int R = (M + ntp - 1) / ntp;
  if (mode == 0 && M % ntp != 0) return -kBadArgument;
  tp::RsParams rs{};
  rs.rank = reg->rank;
  rs.tp = ntp;
  rs.M = M;
  rs.N = N;
  rs.R = R;
  rs.mode = mode;
  const int parity = slot & 1;
  for (int i = 0; i < ntp; ++i) rs.peer[i] = static_cast<uint8_t*>(reg->peer[i]);
  tp::EpochCtl ectl{reinterpret_cast<uint32_t*>(rs.peer[rs.rank] + lay->off_epoch_rs),
                    reinterpret_cast<uint32_t*>(rs.peer[rs.rank] + lay->off_epoch_rs + 4)};
  if (static_cast<int64_t>(ntp) * R * N * 2 > lay->staging_half_bytes || (mode == 1 && static_cast<int64_t>(M) * N * 2 > lay->yall_half_bytes))
    return -kTooLarge;
  rs.off_staging = lay->off_staging + parity * lay->staging_half_bytes;
  rs.off_yall = lay->off_yall + parity * lay->yall_half_bytes;
  rs.off_flags = lay->off_rs_flags;
  rs.off_resflags = lay->off_res_flags;
  rs.off_done = lay->off_done;
  rs.residual = static_cast<const __nv_bfloat16*>(residual);
  rs.out = static_cast<__nv_bfloat16*>(out);
  rs.timeout_ns = timeout_ns;
  rs.region_bytes = lay->total_bytes;
  rs.status = status;
  const bool swap = M <= 64;
  const int bn = swap ? (M <= 16 ? 16 : M <= 32 ? 32 : 64) : 128;
  const int tm = swap ? bn : 128;
  const int64_t units = static_cast<int64_t>((R + tm - 1) / tm + 1) * (swap ? (N + 127) / 128 : (N + bn - 1) / bn);
  if (units * ntp * 4 > lay->rs_flags_bytes) return -kTooLarge;
  if (swap) {
    switch (bn) {
      case 16: return launch_fp8_rs<16, true>(xq, xs, wq, ws, M, N, K, rs, ectl, status, stream);
      case 32: return launch_fp8_rs<32, true>(xq, xs, wq, ws, M, N, K, rs, ectl, status, stream);
      default: return launch_fp8_rs<64, true>(xq, xs, wq, ws, M, N, K, rs, ectl, status, stream);
    }
  }
  return launch_fp8_rs<128, false>(xq, xs, wq, ws, M, N, K, rs, ectl, status, stream);
}

// All-gather fused with the block-scaled fp8 column-parallel GEMM. The gathered buffer of this parity holds the
// e4m3 rows [M][K] followed (at the next 1024-byte boundary) by their f32 scales [M][K / 128]; this rank's rows
// and scales must already be there. K must be a multiple of 512 so that a chunk of scale rows is a whole number
// of 16-byte units.
extern "C" int b2_tp_ag_gemm_fp8(const void* wq, const float* ws, const B2TpRegion* reg, const B2TpLayout* lay, void* y, int M, int N,
                                 int K, int64_t ldy, int slot, uint64_t timeout_ns, int n_comm, b2::Status* status,
                                 cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (reg == nullptr || lay == nullptr || reg->tp < 1 || reg->tp > tp::kMaxTp || K % 512 != 0 || N % 8 != 0 || ldy % 8 != 0 ||
      M % reg->tp != 0)
    return -kBadArgument;
  const int ntp = reg->tp;
  tp::AgParams ag{};
  ag.rank = reg->rank;
  ag.tp = ntp;
  ag.M = M;
  ag.K = K;
  ag.R = M / ntp;
  ag.chunk_rows = tp::ag_chunk_rows(ag.R);
  ag.chunks_per_rank = (ag.R + ag.chunk_rows - 1) / ag.chunk_rows;
  const int parity = slot & 1;
  for (int i = 0; i < ntp; ++i) ag.peer[i] = static_cast<uint8_t*>(reg->peer[i]);
  tp::EpochCtl ectl{reinterpret_cast<uint32_t*>(ag.peer[ag.rank] + lay->off_epoch_ag),
                    reinterpret_cast<uint32_t*>(ag.peer[ag.rank] + lay->off_epoch_ag + 4)};
  const int64_t q_bytes = (static_cast<int64_t>(M) * K + 1023) / 1024 * 1024;
  const int64_t s_bytes = static_cast<int64_t>(M) * (K / 128) * 4;
  if (q_bytes + s_bytes > lay->xall_half_bytes) return -kTooLarge;
  if (static_cast<int64_t>(ntp) * ag.chunks_per_rank * 4 > lay->ag_flags_bytes) return -kTooLarge;
  ag.off_xall = lay->off_xall + parity * lay->xall_half_bytes;
  ag.row_bytes = K;
  ag.off_aux = ag.off_xall + q_bytes;
  ag.aux_row_bytes = static_cast<int64_t>(K / 128) * 4;
  ag.off_flags = lay->off_ag_flags;
  ag.n_comm = ntp > 1 ? (n_comm > 0 ? n_comm : 8) : 0;
  if (ag.n_comm > ag.chunks_per_rank && ntp > 1) ag.n_comm = ag.chunks_per_rank;
  ag.timeout_ns = timeout_ns;
  const void* xq_all = ag.peer[ag.rank] + ag.off_xall;
  const float* xs_all = reinterpret_cast<const float*>(ag.peer[ag.rank] + ag.off_aux);
  const bool swap = M <= 64;
  const int bn = swap ? (M <= 16 ? 16 : M <= 32 ? 32 : 64) : 128;
  if (swap) {
    switch (bn) {
      case 16: return launch_fp8_ag<16, true>(xq_all, xs_all, wq, ws, y, M, N, K, ldy, ag, ectl, status, stream);
      case 32: return launch_fp8_ag<32, true>(xq_all, xs_all, wq, ws, y, M, N, K, ldy, ag, ectl, status, stream);
      default: return launch_fp8_ag<64, true>(xq_all, xs_all, wq, ws, y, M, N, K, ldy, ag, ectl, status, stream);
    }
  }
  return launch_fp8_ag<128, false>(xq_all, xs_all, wq, ws, y, M, N, K, ldy, ag, ectl, status, stream);
}
