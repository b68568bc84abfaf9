// bf16 GEMM on CTA pairs (tcgen05 cta_group::2): Y[M, N] = X[M, K] * W[N, K]^T, f32 accumulate, bf16 out.
//
// Two CTAs of a cluster of 2 work on one 256 x 256 output tile. Each CTA stages 128 rows of X and 128 rows of W
// per 64-wide k-block (32 KB instead of the 48 KB a lone CTA needs for a 128 x 256 tile), the even CTA of the pair
// issues `tcgen05.mma.cta_group::2` (M = 256, N = 256, K = 16), which reads both CTAs' shared memory and writes
// 128 accumulator rows into each CTA's TMEM. Every W byte therefore crosses the L2 -> SM path once per two SMs:
// the single-CTA kernel is bound by exactly that path at large sizes (profiles/gemm_bf16_tcgen05_8192.md).
//
// Per CTA, 192 threads as in gemm_tc.cuh: warp 0 one TMA lane, warp 1 TMEM allocation and (even CTA only) the MMA
// lane, warps 2-5 the epilogue over this CTA's 128 rows. Barriers: `full` lives in the even CTA and counts the
// bytes of both CTAs' loads; `empty` and `tmem_full` exist in both CTAs and are signalled by one commit each from
// the MMA lane; `tmem_empty` lives in the even CTA and collects the eight epilogue warps of the pair. Loads carry
// no cluster broadcast: each CTA fetches its own half tiles. Every wait is bounded; a role that gives up records
// TIMEOUT and stops, the rest of the pair runs into its own limits, and both CTAs meet at the cluster barrier
// before TMEM is freed. The reference has no tensor-core code at all (stdlib/src/sys/info.mojo:423-434).
#include <cstdint>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "b2/api.h"
#include "b2/launch.h"
#include "b2/config.h"
#include "b2/ptx.cuh"
#include "b2/status.h"
#include "b2/tma.h"

namespace b2 {
namespace {

constexpr int kPairThreads = 192;
constexpr int kPairABytes = 128 * 64 * 2;       // 16 KB: this CTA's 128 rows of X for one k-block
// BN = UMMA N of the pair (256 or 128); each CTA stages BN / 2 rows of W per k-block.
template <int BN>
struct PairCfg {
  static constexpr int kBBytes = (BN / 2) * 64 * 2;
  static constexpr int kStageBytes = kPairABytes + kBBytes;
  static constexpr int kStages = (192 * 1024) / kStageBytes;          // 6 (BN 256) or 8 (BN 128)
  static constexpr int kRing = kStages * kStageBytes;
  static constexpr int kBars = 2 * kStages + 4;                        // full, empty, tmem_full[2], tmem_empty[2]
  static constexpr int kSmem = kRing + 8 * kBars + 16 + 1024;
  static constexpr int kTmemCols = 2 * BN;                             // two accumulators
};

struct PairParams {
  __nv_bfloat16* y;
  int64_t ldy;
  int M, N, num_kb;
  int m_tiles, n_tiles;   // 256-row and 256-column tiles
  int swiglu;             // 1: W rows alternate 16 gate / 16 up rows; y[M, N / 2] = silu(gate) * up
};

// Tile order: groups of 8 row tiles, column tiles varying slowest inside a group, so that the pairs running at the
// same time share W tiles (8 pairs each) and X tiles through L2.
__device__ __forceinline__ void pair_tile(const PairParams& p, int t, int& mt, int& nt) {
  const int group_size = 8 * p.n_tiles;
  const int group = t / group_size;
  const int first = group * 8;
  const int gm = min(p.m_tiles - first, 8);
  const int r = t - group * group_size;
  mt = first + r % gm;
  nt = r / gm;
}

template <int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w, PairParams p,
                      Status* status) {
  using Cfg = PairCfg<BN>;
  constexpr int kPairBN = BN;
  constexpr int kPairStages = Cfg::kStages;
  constexpr int kPairStageBytes = Cfg::kStageBytes;
  constexpr int kPairRing = Cfg::kRing;
  constexpr int kPairBars = Cfg::kBars;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - ptx::smem_u32(smem_raw));
  const uint32_t bar_base = base + kPairRing;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kPairStages + s); };
  auto tmem_full = [&](int a) { return bar_base + 8u * (2 * kPairStages + a); };
  auto tmem_empty = [&](int a) { return bar_base + 8u * (2 * kPairStages + 2 + a); };
  uint32_t* holder = reinterpret_cast<uint32_t*>(smem + kPairRing + 8 * kPairBars);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();        // 0 = the CTA that issues the MMAs
  const int pair = static_cast<int>(blockIdx.x >> 1), num_pairs = static_cast<int>(gridDim.x >> 1);
  const int total = p.m_tiles * p.n_tiles;

  if (threadIdx.x == 0) {
    ptx::prefetch_tensormap(&tmap_x);
    ptx::prefetch_tensormap(&tmap_w);
    for (int s = 0; s < kPairStages; ++s) {
      ptx::mbar_init(full_bar(s), 1);     // used in the even CTA only
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(tmem_full(a), 1);
      ptx::mbar_init(tmem_empty(a), 8);   // used in the even CTA only: four epilogue warps of each CTA
    }
    ptx::fence_mbar_init();
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(ptx::smem_u32(holder), Cfg::kTmemCols);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();   // the peer's barriers are initialised before anything is signalled across the pair
  ptx::tc_fence_after();
  const uint32_t tmem_base = *holder;
  ptx::grid_dep_sync();   // the set-up above overlapped the previous kernel's tail; operands and outputs are global memory

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (ptx::elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      long issued = 0;
      bool ok = true;
      for (int t = pair; ok && t < total; t += num_pairs) {
        int mt, nt;
        pair_tile(p, t, mt, nt);
        const int row_x = mt * 256 + static_cast<int>(rank) * 128;
        const int row_w = nt * kPairBN + static_cast<int>(rank) * (kPairBN / 2);
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1u)) {
            status_record(status, kTimeout, kSiteGemmEmpty, t, kb);
            ok = false;
            break;
          }
          const uint32_t sp = base + stage * kPairStageBytes;
          const uint32_t leader_full = ptx::mapa(full_bar(stage), 0);
          if (rank == 0) ptx::mbar_arrive_expect_tx(full_bar(stage), 2 * kPairStageBytes);  // both CTAs' bytes
          ptx::tma_load_2d_pair(sp, &tmap_x, leader_full, kb * 64, row_x, ptx::kEvictNormal);
          ptx::tma_load_2d_pair(sp + kPairABytes, &tmap_w, leader_full, kb * 64, row_w, ptx::kEvictNormal);
          ++issued;
          if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
        }
      }
      // A copy of this CTA reports to the even CTA's barrier, so it cannot be waited for here: after a failed
      // wait give the copies in flight time to land before the pair meets at the closing cluster barrier.
      if (!ok && issued > 0) ptx::nanosleep(100000);
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (even CTA only)
    if (rank == 0 && ptx::elect_one()) {
      constexpr uint32_t idesc = ptx::make_idesc(1, 1, 256, kPairBN);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int t = pair; ok && t < total; t += num_pairs) {
        if (!ptx::mbar_wait(tmem_empty(acc), acc_phase ^ 1u)) {
          status_record(status, kTimeout, kSiteGemmTmemEmpty, t, acc);
          ok = false;
          break;
        }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kPairBN;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!ptx::mbar_wait(full_bar(stage), phase)) {
            status_record(status, kTimeout, kSiteGemmFull, t, kb);
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          const uint32_t sp = base + stage * kPairStageBytes;
          const uint64_t da = ptx::make_smem_desc_sw128(sp);
          const uint64_t db = ptx::make_smem_desc_sw128(sp + kPairABytes);
#pragma unroll
          for (int k = 0; k < 4; ++k) ptx::tc_mma_f16_pair(d_tmem, da + 2u * k, db + 2u * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          // the stage is free in both CTAs once these MMAs have read it
          ptx::tc_commit_pair(empty_bar(stage));
          ptx::tc_commit_pair(ptx::mapa(empty_bar(stage), 1));
          if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        ptx::tc_commit_pair(tmem_full(acc));
        ptx::tc_commit_pair(ptx::mapa(tmem_full(acc), 1));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue warps (both CTAs, 128 rows each)
    const int quarter = warp & 3;
    const int p_local = quarter * 32 + lane;
    const uint32_t leader_empty0 = ptx::mapa(tmem_empty(0), 0), leader_empty1 = ptx::mapa(tmem_empty(1), 0);
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = pair; t < total; t += num_pairs) {
      int mt, nt;
      pair_tile(p, t, mt, nt);
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(tmem_full(acc), acc_phase))) {
        if (lane == 0) status_record(status, kTimeout, kSiteGemmTmemFull, t, acc);
        break;
      }
      ptx::tc_fence_after();
      const uint32_t taddr = tmem_base + acc * kPairBN + (static_cast<uint32_t>(quarter * 32) << 16);
      const int m = mt * 256 + static_cast<int>(rank) * 128 + p_local;
#pragma unroll 1
      for (int c = 0; c < kPairBN / 32; ++c) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(taddr + c * 32, r);
        ptx::tc_wait_ld();
        const int n0 = nt * kPairBN + c * 32;
        if (p.swiglu) {
          // columns [n0, n0 + 16) are gate values, [n0 + 16, n0 + 32) the matching up values: 16 outputs
          if (m < p.M && n0 < p.N) {
            __nv_bfloat16* dst = p.y + static_cast<int64_t>(m) * p.ldy + (n0 >> 1);
#pragma unroll
            for (int g = 0; g < 2; ++g) {
              float o[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) o[i] = ptx::silu(__uint_as_float(r[g * 8 + i])) * __uint_as_float(r[16 + g * 8 + i]);
              uint4 pk;
              pk.x = ptx::pack_bf16x2(o[0], o[1]);
              pk.y = ptx::pack_bf16x2(o[2], o[3]);
              pk.z = ptx::pack_bf16x2(o[4], o[5]);
              pk.w = ptx::pack_bf16x2(o[6], o[7]);
              ptx::st_v4(dst + g * 8, pk);
            }
          }
        } else if (m < p.M) {
          __nv_bfloat16* dst = p.y + static_cast<int64_t>(m) * p.ldy + n0;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            if (n0 + g * 8 >= p.N) break;
            uint4 pk;
            pk.x = ptx::pack_bf16x2(__uint_as_float(r[g * 8 + 0]), __uint_as_float(r[g * 8 + 1]));
            pk.y = ptx::pack_bf16x2(__uint_as_float(r[g * 8 + 2]), __uint_as_float(r[g * 8 + 3]));
            pk.z = ptx::pack_bf16x2(__uint_as_float(r[g * 8 + 4]), __uint_as_float(r[g * 8 + 5]));
            pk.w = ptx::pack_bf16x2(__uint_as_float(r[g * 8 + 6]), __uint_as_float(r[g * 8 + 7]));
            ptx::st_v4(dst + g * 8, pk);
          }
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive_cluster(acc == 0 ? leader_empty0 : leader_empty1);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();   // neither CTA frees TMEM or leaves while the other may still read its shared memory / TMEM
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
  }
}

template <int BN>
int launch_pair(const void* x, const void* w, void* y, int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldy, int epilogue,
                Status* status, cudaStream_t stream) {
  using Cfg = PairCfg<BN>;
  CUtensorMap tx, tw;
  if (!make_tmap_2d(&tx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, M, K, ldx * 2, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B) ||
      !make_tmap_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w, N, K, ldw * 2, BN / 2, 64, CU_TENSOR_MAP_SWIZZLE_128B))
    return -kBadArgument;
  PairParams p{};
  p.y = static_cast<__nv_bfloat16*>(y);
  p.ldy = ldy;
  p.M = M;
  p.N = N;
  p.num_kb = (K + 63) / 64;
  p.m_tiles = (M + 255) / 256;
  p.n_tiles = (N + BN - 1) / BN;
  p.swiglu = epilogue == B2_EPI_SWIGLU ? 1 : 0;
  static DeviceOnce attr_once;
  if (const int rc = attr_once.run([&] {
        cudaError_t e = cudaFuncSetAttribute(gemm_bf16_pair_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem);
        return e;
      }))
    return rc;
  const int total = p.m_tiles * p.n_tiles;
  const int pairs = total < kNumSMs / 2 ? total : kNumSMs / 2;
  launch_pdl(gemm_bf16_pair_kernel<BN>, dim3(2 * pairs), dim3(kPairThreads), Cfg::kSmem, stream, tx, tw, p, status);
  return last_launch_rc();
}

}  // namespace
}  // namespace b2

using namespace b2;

// Y = X W^T on CTA pairs (epilogue B2_EPI_NONE, or B2_EPI_SWIGLU with the 16-row interleaved gate/up weight and
// y [M, N / 2]); tiles of 256 rows x `bn` columns, bn = 256 or 128. K a multiple of 8; N a multiple of 8; ldx, ldw,
// ldy multiples of 8 elements. Any M and N are accepted (edges are zero-filled on load and clipped on store).
extern "C" int b2_gemm_bf16_pair(const void* x, const void* w, void* y, int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldy,
                                 int epilogue, int bn, Status* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 != 0 || N % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0 || ldy % 8 != 0) return -kBadArgument;
  if (epilogue != B2_EPI_NONE && epilogue != B2_EPI_SWIGLU) return -kBadArgument;
  if (epilogue == B2_EPI_SWIGLU && N % 32 != 0) return -kBadArgument;
  if (bn == 128) return launch_pair<128>(x, w, y, M, N, K, ldx, ldw, ldy, epilogue, status, stream);
  if (bn == 0 || bn == 256) return launch_pair<256>(x, w, y, M, N, K, ldx, ldw, ldy, epilogue, status, stream);
  return -kBadArgument;
}
