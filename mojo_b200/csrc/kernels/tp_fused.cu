// Tensor-parallel GEMMs fused with their collective, over NVLink peer memory.
//
//   gemm_rs   Y_r = reduce_scatter(X[M, K/tp] * W^T)      row-parallel GEMM; the epilogue stores each finished
//             (or all-reduce, mode 1)                      tile straight into the staging buffer of the rank that
//                                                          owns those rows, then raises that rank's flag. After
//                                                          its own tiles, every CTA turns to the rows its rank
//                                                          owns: waits (bounded) for the tp contributions of a
//                                                          tile, sums them in f32 and writes the result locally
//                                                          (reduce-scatter) or into every rank's copy (all-reduce).
//   ag_gemm   Y = all_gather(X_r[M/tp, K]) * W[N/tp, K]^T  a few CTAs push this rank's rows into every peer's
//                                                          gathered buffer chunk by chunk and raise per-chunk
//                                                          flags; the GEMM CTAs start on the local rows and wait
//                                                          (bounded) per tile for the chunks of the peers' rows.
//
// All cross-GPU traffic is plain peer loads/stores and .sys-scoped release/acquire flags issued from inside
// the same kernel as the tcgen05 tiles; no NCCL call and no cluster-broadcast TMA anywhere. Symmetric buffers
// are double-buffered by launch parity: a rank can run at most one launch ahead of any peer, because every
// launch ends by waiting for something every peer produces during that launch.
//
// Flags carry the launch epoch (monotonic), so nothing is ever reset and a flag left over from an earlier
// shape is simply stale (< epoch). Every wait has a deadline; on expiry the kernel records TIMEOUT and exits.
#include <cstdint>
#include <cuda.h>
#include <cuda_bf16.h>
#include "b2/api.h"
#include "b2/launch.h"
#include "b2/gemm_tc.cuh"
#include "b2/ptx.cuh"
#include "b2/tma.h"
#include "b2/tp.h"
#include <cstdlib>
#include "b2/tp_ag.cuh"
#include "b2/tp_rs.cuh"
#include "b2/vec.cuh"

namespace b2 {
namespace {

using gemm::WorkUnit;
using namespace b2::tp;
// The reduction runs next to the GEMM in every CTA: two side warps claim finished units of this rank's rows and
// sum the ranks' contributions while warps 0-5 keep the tile pipeline going, so all SMs do tensor work.
constexpr int kRsThreads = gemm::kThreads + SideTeam::kThreads;
template <int BN, bool SWAP>
struct RsSideReduce {
  static constexpr int kWarps = SideTeam::kThreads / 32;
  RsParams p;
  Status* status;
  __device__ __forceinline__ void operator()(int, int) const { reduce_phase<BN, SWAP, SideTeam>(p, status); }
};

// SIDE = true: the side-warp scheme above (every CTA runs the GEMM). SIDE = false: CTAs [n_gemm, grid) only reduce
// from the start and the GEMM CTAs join the reduction after their last tile; kept as the fallback the launch
// uses unless B2_RS_SIDE=1.
template <int BN, int STAGES, bool SWAP, bool SIDE>
__global__ void __launch_bounds__(SIDE ? kRsThreads : gemm::kThreads, 1)
gemm_rs_kernel(const __grid_constant__ CUtensorMap tmap_p, const __grid_constant__ CUtensorMap tmap_q,
               const __grid_constant__ RsSched sched, RsParams prm_in, EpochCtl ectl, int n_gemm, Status* status) {
  ptx::grid_dep_sync();
  constexpr uint32_t idesc = ptx::make_idesc(1, 1, 128, BN);
  RsParams prm = prm_in;
  prm.epoch = epoch_begin(ectl);
  prm.status = status;
  const bool has_tiles = static_cast<int>(blockIdx.x) < n_gemm;
  if (has_tiles) {
    extern __shared__ uint8_t smem_dyn[];
    uint8_t* epi_buf = smem_dyn + gemm::SmemLayout<BN, STAGES>::kTotalBytes;
    epi_buf += (16 - (reinterpret_cast<uintptr_t>(epi_buf) & 15)) & 15;  // 16-byte vector accesses
    RsEpilogue<BN, SWAP> epi{prm, epi_buf};
    if constexpr (SIDE) {
      gemm::run<BN, STAGES, 2>(&tmap_p, &tmap_q, idesc, ptx::kEvictNormal, ptx::kEvictNormal, sched, gemm::NoGate{}, epi, status,
                               static_cast<int>(blockIdx.x), n_gemm, gemm::NoFill{}, RsSideReduce<BN, SWAP>{prm, status});
    } else {
      gemm::run<BN, STAGES, 2>(&tmap_p, &tmap_q, idesc, ptx::kEvictNormal, ptx::kEvictNormal, sched, gemm::NoGate{}, epi, status,
                               static_cast<int>(blockIdx.x), n_gemm);
    }
  }
  if (!SIDE || !has_tiles) reduce_phase<BN, SWAP, CtaTeam>(prm, status);
  rs_epoch_end(ectl, prm);
}

constexpr int stages_for(int bn) {
  const int stage = 128 * 64 * 2 + bn * 64 * 2;
  int s = (200 * 1024) / stage;
  return s > 10 ? 10 : s;
}
// the reduce-scatter kernel gives part of its shared memory to the staged epilogue
constexpr int rs_stages_for(int bn) {
  const int stage = 128 * 64 * 2 + bn * 64 * 2;
  int s = (176 * 1024) / stage;
  return s > 10 ? 10 : s;
}

template <int BN, bool SWAP>
int launch_rs(const void* x, const void* w, int M, int N, int K, int64_t ldx, int64_t ldw, RsParams prm, EpochCtl ectl,
              Status* status, cudaStream_t stream) {
  constexpr int STAGES = rs_stages_for(BN);
  constexpr int SMEM = gemm::SmemLayout<BN, STAGES>::kTotalBytes + rs_epi_bytes<BN, SWAP>() + 16;
  using L = gemm::SmemLayout<BN, STAGES>;
  const void* p_ptr = SWAP ? w : x;
  const void* q_ptr = SWAP ? x : w;
  const int rows_p = SWAP ? N : M, rows_q = SWAP ? M : N;
  const int64_t ldp = SWAP ? ldw : ldx, ldq = SWAP ? ldx : ldw;
  CUtensorMap tp, tq;
  if (!make_tmap_2d(&tp, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p_ptr, rows_p, K, ldp * 2, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B) ||
      !make_tmap_2d(&tq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, q_ptr, rows_q, K, ldq * 2, BN, 64, CU_TENSOR_MAP_SWIZZLE_128B))
    return -kBadArgument;
  RsSched sched{};
  sched.p_blocks = (rows_p + 127) / 128;
  sched.q_blocks = (rows_q + BN - 1) / BN;
  sched.num_kb = (K + 63) / 64;
  sched.bn = BN;
  sched.swap = SWAP;
  constexpr int TM = SWAP ? BN : 128;
  sched.m_tiles = SWAP ? sched.q_blocks : sched.p_blocks;
  if (!build_rs_order(sched, prm.tp, prm.rank, prm.R, TM)) return -kTooLarge;
  prm.p_blocks = sched.p_blocks;
  prm.q_blocks = sched.q_blocks;
  static const bool side = [] {
    const char* e = std::getenv("B2_RS_SIDE");
    return e != nullptr && e[0] == '1';
  }();
  static DeviceOnce attr_once;
  if (const int rc = attr_once.run([&] {
        cudaError_t e = cudaFuncSetAttribute(gemm_rs_kernel<BN, STAGES, SWAP, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_rs_kernel<BN, STAGES, SWAP, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        return e;
      }))
    return rc;
  const int total = sched.p_blocks * sched.q_blocks;
  if (side) {
    // Full persistent grid: every CTA that has tiles runs the GEMM with its reduction side warps; CTAs beyond the
    // tile count only reduce.
    const int n_gemm = total < kNumSMs ? total : kNumSMs;
    launch_pdl(gemm_rs_kernel<BN, STAGES, SWAP, true>, dim3(kNumSMs), dim3(kRsThreads), SMEM, stream, tp, tq, sched, prm, ectl, n_gemm, status);
  } else {
    // Twelve CTAs only reduce, from the start: the reduction of finished units then overlaps the rest of the GEMM
    // (measured: with none, the all-reduce of a 4096-token tile set is 15 % slower although the GEMM has more SMs).
    const int n_red = prm.tp > 1 ? 12 : 0;
    int n_gemm = kNumSMs - n_red;
    if (total < n_gemm) n_gemm = total;
    launch_pdl(gemm_rs_kernel<BN, STAGES, SWAP, false>, dim3(kNumSMs), dim3(gemm::kThreads), SMEM, stream, tp, tq, sched, prm, ectl, n_gemm, status);
  }
  return last_launch_rc();
}

// ------------------------------------------------------------------------------------------------
// all-gather -> GEMM
// ------------------------------------------------------------------------------------------------
struct PlainEpiParams {
  __nv_bfloat16* y;
  int64_t ldy;
  int M, N;
};

template <int BN, bool SWAP>
struct PlainEpilogue {
  static constexpr int CH = BN >= 32 ? 32 : 16;
  PlainEpiParams p;
  __device__ __forceinline__ void operator()(const WorkUnit& u, uint32_t taddr, int quarter, int lane, uint32_t*,
                                             Status*) const {
    const int p_local = quarter * 32 + lane;
#pragma unroll 1
    for (int c = 0; c < BN / CH; ++c) {
      uint32_t r[CH];
      if constexpr (CH == 32) ptx::tmem_ld_32x32(taddr + c * CH, r);
      else ptx::tmem_ld_32x16(taddr + c * CH, r);
      ptx::tc_wait_ld();
      if constexpr (!SWAP) {
        const int m = u.pb * 128 + p_local, n0 = u.qb * BN + c * CH;
        if (m >= p.M) continue;
        __nv_bfloat16* dst = p.y + static_cast<int64_t>(m) * p.ldy + n0;
#pragma unroll
        for (int g = 0; g < CH / 8; ++g) {
          if (n0 + g * 8 >= p.N) break;
          uint4 pk;
          pk.x = ptx::pack_bf16x2(__uint_as_float(r[g * 8 + 0]), __uint_as_float(r[g * 8 + 1]));
          pk.y = ptx::pack_bf16x2(__uint_as_float(r[g * 8 + 2]), __uint_as_float(r[g * 8 + 3]));
          pk.z = ptx::pack_bf16x2(__uint_as_float(r[g * 8 + 4]), __uint_as_float(r[g * 8 + 5]));
          pk.w = ptx::pack_bf16x2(__uint_as_float(r[g * 8 + 6]), __uint_as_float(r[g * 8 + 7]));
          ptx::st_v4(dst + g * 8, pk);
        }
      } else {
        const int n = u.pb * 128 + p_local, m0 = u.qb * BN + c * CH;
        if (n >= p.N) continue;
#pragma unroll
        for (int j = 0; j < CH; ++j) {
          if (m0 + j >= p.M) break;
          p.y[static_cast<int64_t>(m0 + j) * p.ldy + n] = __float2bfloat16(__uint_as_float(r[j]));
        }
      }
    }
  }
};

// SIDE = false: the last n_comm CTAs of the grid only move data (bulk async copies through shared memory), the
// others run the GEMM. SIDE = true: every CTA runs the GEMM and one side warp per CTA pushes its share of this
// rank's row chunks with plain 16-byte loads and stores at kernel start, so no SM is set aside for communication;
// selected with B2_AG_SIDE=1.
constexpr int kAgThreads = gemm::kThreads + 32;
template <int BN, int STAGES, bool SWAP, bool SIDE>
__global__ void __launch_bounds__(SIDE ? kAgThreads : gemm::kThreads, 1)
ag_gemm_kernel(const __grid_constant__ CUtensorMap tmap_p, const __grid_constant__ CUtensorMap tmap_q, AgSched sched,
               AgParams prm_in, PlainEpiParams ep, EpochCtl ectl, Status* status) {
  ptx::grid_dep_sync();
  AgParams prm = prm_in;
  prm.epoch = epoch_begin(ectl);
  constexpr uint32_t idesc = ptx::make_idesc(1, 1, 128, BN);
  PlainEpilogue<BN, SWAP> epi{ep};
  AgGate gate{prm, SWAP, BN};
  if constexpr (SIDE) {
    AgSidePush push{prm, static_cast<int>(blockIdx.x), static_cast<int>(gridDim.x)};
    gemm::run<BN, STAGES, 2>(&tmap_p, &tmap_q, idesc, ptx::kEvictNormal, ptx::kEvictNormal, sched, gate, epi, status,
                             static_cast<int>(blockIdx.x), static_cast<int>(gridDim.x), gemm::NoFill{}, push);
  } else {
    const int n_gemm = static_cast<int>(gridDim.x) - prm.n_comm;
    if (static_cast<int>(blockIdx.x) >= n_gemm) {
      extern __shared__ uint8_t smem_dyn[];
      uint8_t* win = smem_dyn + ((128 - (reinterpret_cast<uintptr_t>(smem_dyn) & 127)) & 127);
      ag_push(prm, static_cast<int>(blockIdx.x) - n_gemm, win, status);
      epoch_end(ectl, prm.epoch);
      return;
    }
    gemm::run<BN, STAGES, 2>(&tmap_p, &tmap_q, idesc, ptx::kEvictNormal, ptx::kEvictNormal, sched, gate, epi, status,
                             static_cast<int>(blockIdx.x), n_gemm);
  }
  epoch_end(ectl, prm.epoch);
}

// Standalone push all-gather (no GEMM): used where the gathered rows feed something other than a GEMM.
__global__ void __launch_bounds__(256) ag_push_kernel(AgParams prm_in, EpochCtl ectl, Status* status) {
  ptx::grid_dep_sync();
  AgParams prm = prm_in;
  prm.epoch = epoch_begin(ectl);
  extern __shared__ uint8_t smem_dyn[];
  uint8_t* win = smem_dyn + ((128 - (reinterpret_cast<uintptr_t>(smem_dyn) & 127)) & 127);
  ag_push(prm, static_cast<int>(blockIdx.x), win, status);
  __syncthreads();
  // wait for every peer's chunks so the gathered buffer is complete when the kernel ends
  if (blockIdx.x == 0) {
    const uint32_t* flags = reinterpret_cast<const uint32_t*>(prm.peer[prm.rank] + prm.off_flags);
    for (int i = threadIdx.x; i < prm.tp * prm.chunks_per_rank; i += blockDim.x) {
      const int src = i / prm.chunks_per_rank;
      if (src == prm.rank) continue;
      if (!ptx::wait_flag_ge_sys(flags + i, prm.epoch, prm.timeout_ns)) status_record(status, kTimeout, kSiteAgChunk, src, i);
    }
  }
  epoch_end(ectl, prm.epoch);
}

template <int BN, bool SWAP>
int launch_ag(const void* xall_local, const void* w, void* y, int M, int N, int K, int64_t ldw, int64_t ldy, AgParams prm,
              EpochCtl ectl, Status* status, cudaStream_t stream) {
  constexpr int STAGES = stages_for(BN);
  using L = gemm::SmemLayout<BN, STAGES>;
  const void* p_ptr = SWAP ? w : xall_local;
  const void* q_ptr = SWAP ? xall_local : w;
  const int rows_p = SWAP ? N : M, rows_q = SWAP ? M : N;
  const int64_t ldp = SWAP ? ldw : K, ldq = SWAP ? K : ldw;
  CUtensorMap tp, tq;
  if (!make_tmap_2d(&tp, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p_ptr, rows_p, K, ldp * 2, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B) ||
      !make_tmap_2d(&tq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, q_ptr, rows_q, K, ldq * 2, BN, 64, CU_TENSOR_MAP_SWIZZLE_128B))
    return -kBadArgument;
  AgSched sched;
  sched.p_blocks = (rows_p + 127) / 128;
  sched.q_blocks = (rows_q + BN - 1) / BN;
  sched.num_kb = (K + 63) / 64;
  sched.bn = BN;
  sched.swap = SWAP;
  constexpr int TM = SWAP ? BN : 128;
  sched.m_tiles = SWAP ? sched.q_blocks : sched.p_blocks;
  sched.first_tile = (prm.rank * prm.R / TM) % sched.m_tiles;
  PlainEpiParams ep{static_cast<__nv_bfloat16*>(y), ldy, M, N};
  static const bool side = [] {
    const char* e = std::getenv("B2_AG_SIDE");
    return e != nullptr && e[0] == '1';
  }();
  static DeviceOnce attr_once;
  if (const int rc = attr_once.run([&] {
        cudaError_t e = cudaFuncSetAttribute(ag_gemm_kernel<BN, STAGES, SWAP, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotalBytes);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(ag_gemm_kernel<BN, STAGES, SWAP, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotalBytes);
        return e;
      }))
    return rc;
  const int total = sched.p_blocks * sched.q_blocks;
  if (side) {
    const int grid = total < kNumSMs ? total : kNumSMs;
    launch_pdl(ag_gemm_kernel<BN, STAGES, SWAP, true>, dim3(grid), dim3(kAgThreads), L::kTotalBytes, stream, tp, tq, sched, prm, ep, ectl, status);
  } else {
    int n_gemm = kNumSMs - prm.n_comm;
    if (total < n_gemm) n_gemm = total;
    launch_pdl(ag_gemm_kernel<BN, STAGES, SWAP, false>, dim3(n_gemm + prm.n_comm), dim3(gemm::kThreads), L::kTotalBytes, stream, tp, tq, sched, prm, ep, ectl, status);
  }
  return last_launch_rc();
}

// Cross-GPU barrier: every rank raises its slot on every peer, then waits for all slots.
__global__ void symm_barrier_kernel(B2TpRegion reg, int64_t off_flags, EpochCtl ectl, uint64_t timeout_ns, Status* status) {
  ptx::grid_dep_sync();
  const int t = threadIdx.x;
  const uint32_t epoch = epoch_begin(ectl);
  if (t < reg.tp) {
    ptx::st_release_sys(reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(reg.peer[t]) + off_flags) + reg.rank, epoch);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(static_cast<uint8_t*>(reg.peer[reg.rank]) + off_flags) + t;
    if (!ptx::wait_flag_ge_sys(mine, epoch, timeout_ns)) status_record(status, kTimeout, kSiteGridBarrier, t, epoch);
  }
  epoch_end(ectl, epoch);
}

// Test hook for the timeout path: wait on a flag that nothing raises, with a short deadline.
__global__ void wait_flag_kernel(const uint32_t* flag, uint32_t want, uint64_t timeout_ns, Status* status) {
  ptx::grid_dep_sync();
  if (threadIdx.x == 0 && !ptx::wait_flag_ge_sys(flag, want, timeout_ns)) status_record(status, kTimeout, kSiteTest, want, 0);
}

int pick_bn_swap(int M) { return M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256; }

}  // namespace
}  // namespace b2

using namespace b2;

extern "C" int b2_tp_gemm_rs_bf16(const void* x, const void* w, const B2TpRegion* reg, const B2TpLayout* lay, void* out,
                                  const void* residual, int M, int N, int K, int64_t ldx, int64_t ldw, int mode,
                                  int slot, uint64_t timeout_ns, int config, b2::Status* status,
                                  cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (reg == nullptr || lay == nullptr || reg->tp < 1 || reg->tp > kMaxTp || K % 8 != 0 || N % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0)
    return -kBadArgument;
  const int tp = reg->tp;
  const int R = (M + tp - 1) / tp;
  if (mode == 0 && M % tp != 0) return -kBadArgument;
  RsParams prm{};
  prm.rank = reg->rank;
  prm.tp = tp;
  prm.M = M;
  prm.N = N;
  prm.R = R;
  prm.epoch = 0;  // read from device memory by the kernel
  prm.mode = mode;
  const int parity = slot & 1;
  for (int i = 0; i < tp; ++i) prm.peer[i] = static_cast<uint8_t*>(reg->peer[i]);
  EpochCtl ectl{reinterpret_cast<uint32_t*>(prm.peer[prm.rank] + lay->off_epoch_rs),
                reinterpret_cast<uint32_t*>(prm.peer[prm.rank] + lay->off_epoch_rs + 4)};
  const int64_t staging_bytes = static_cast<int64_t>(tp) * R * N * 2;
  const int64_t yall_bytes = static_cast<int64_t>(M) * N * 2;
  if (staging_bytes > lay->staging_half_bytes || (mode == 1 && yall_bytes > lay->yall_half_bytes)) return -kTooLarge;
  prm.off_staging = lay->off_staging + parity * lay->staging_half_bytes;
  prm.off_yall = lay->off_yall + parity * lay->yall_half_bytes;
  prm.off_flags = lay->off_rs_flags;
  prm.off_resflags = lay->off_res_flags;
  prm.off_done = lay->off_done;
  prm.residual = static_cast<const __nv_bfloat16*>(residual);
  prm.out = static_cast<__nv_bfloat16*>(out);
  prm.timeout_ns = timeout_ns;
  prm.region_bytes = lay->total_bytes;
  prm.mc_base = tp > 1 ? static_cast<uint8_t*>(reg->mc_base) : nullptr;   // non-null: reduce in the NVLink switch
  bool swap = M <= 128;
  int bn = swap ? pick_bn_swap(M) : 128;
  if (config != 0) {
    swap = (config >> 30) & 1;
    bn = config & 0xffff;
  }
  // 256-wide tiles are not built for this kernel: that instantiation raised an illegal memory access twice and the
  // cause was not found by reading, so no configuration word reaches it.
  if (bn > 128) return -kBadArgument;
  // flag capacity: units of the busiest owner
  const int tm = swap ? bn : 128;
  const int64_t units = static_cast<int64_t>((R + tm - 1) / tm + 1) * (swap ? (N + 127) / 128 : (N + bn - 1) / bn);
  if (units * tp * 4 > lay->rs_flags_bytes) return -kTooLarge;
#define B2_RS(BN_, SWAP_) return launch_rs<BN_, SWAP_>(x, w, M, N, K, ldx, ldw, prm, ectl, status, stream)
  if (swap) {
    switch (bn) {
      case 16: B2_RS(16, true);
      case 32: B2_RS(32, true);
      case 64: B2_RS(64, true);
      case 128: B2_RS(128, true);
      default: return -kBadArgument;
    }
  }
  switch (bn) {
    case 64: B2_RS(64, false);
    case 128: B2_RS(128, false);
    default: return -kBadArgument;
  }
#undef B2_RS
}

extern "C" int b2_tp_ag_gemm_bf16(const void* w, const B2TpRegion* reg, const B2TpLayout* lay, void* y, int M, int N, int K,
                                  int64_t ldw, int64_t ldy, int slot, uint64_t timeout_ns, int n_comm, int config,
                                  b2::Status* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (reg == nullptr || lay == nullptr || reg->tp < 1 || reg->tp > kMaxTp || K % 8 != 0 || N % 8 != 0 || ldw % 8 != 0 || ldy % 8 != 0 ||
      M % reg->tp != 0)
    return -kBadArgument;
  const int tp = reg->tp;
  AgParams prm{};
  prm.rank = reg->rank;
  prm.tp = tp;
  prm.M = M;
  prm.K = K;
  prm.R = M / tp;
  prm.chunk_rows = ag_chunk_rows(prm.R);
  prm.chunks_per_rank = (prm.R + prm.chunk_rows - 1) / prm.chunk_rows;
  prm.epoch = 0;
  const int parity = slot & 1;
  for (int i = 0; i < tp; ++i) prm.peer[i] = static_cast<uint8_t*>(reg->peer[i]);
  EpochCtl ectl{reinterpret_cast<uint32_t*>(prm.peer[prm.rank] + lay->off_epoch_ag),
                reinterpret_cast<uint32_t*>(prm.peer[prm.rank] + lay->off_epoch_ag + 4)};
  if (static_cast<int64_t>(M) * K * 2 > lay->xall_half_bytes) return -kTooLarge;
  if (static_cast<int64_t>(tp) * prm.chunks_per_rank * 4 > lay->ag_flags_bytes) return -kTooLarge;
  prm.off_xall = lay->off_xall + parity * lay->xall_half_bytes;
  prm.row_bytes = static_cast<int64_t>(K) * 2;
  prm.off_flags = lay->off_ag_flags;
  prm.n_comm = tp > 1 ? (n_comm > 0 ? n_comm : 8) : 0;
  if (prm.n_comm > prm.chunks_per_rank && tp > 1) prm.n_comm = prm.chunks_per_rank;
  prm.timeout_ns = timeout_ns;
  const void* xall_local = prm.peer[prm.rank] + prm.off_xall;
  bool swap = M <= 128;
  int bn = swap ? pick_bn_swap(M) : ((M + 127) / 128 * ((N + 255) / 256) >= 132 ? 256 : 128);
  if (config != 0) {
    swap = (config >> 30) & 1;
    bn = config & 0xffff;
  }
#define B2_AG(BN_, SWAP_) return launch_ag<BN_, SWAP_>(xall_local, w, y, M, N, K, ldw, ldy, prm, ectl, status, stream)
  if (swap) {
    switch (bn) {
      case 16: B2_AG(16, true);
      case 32: B2_AG(32, true);
      case 64: B2_AG(64, true);
      case 128: B2_AG(128, true);
      case 256: B2_AG(256, true);
      default: return -kBadArgument;
    }
  }
  switch (bn) {
    case 64: B2_AG(64, false);
    case 128: B2_AG(128, false);
    case 256: B2_AG(256, false);
    default: return -kBadArgument;
  }
#undef B2_AG
}

extern "C" int b2_tp_all_gather(const B2TpRegion* reg, const B2TpLayout* lay, int M, int K, int slot,
                                uint64_t timeout_ns, b2::Status* status, cudaStream_t stream) {
  if (reg == nullptr || lay == nullptr || reg->tp < 1 || reg->tp > kMaxTp || K % 8 != 0 || M % reg->tp != 0) return -kBadArgument;
  if (reg->tp == 1 || M == 0) return 0;
  AgParams prm{};
  prm.rank = reg->rank;
  prm.tp = reg->tp;
  prm.M = M;
  prm.K = K;
  prm.R = M / reg->tp;
  prm.chunk_rows = ag_chunk_rows(prm.R);
  prm.chunks_per_rank = (prm.R + prm.chunk_rows - 1) / prm.chunk_rows;
  prm.epoch = 0;
  const int parity = slot & 1;
  for (int i = 0; i < reg->tp; ++i) prm.peer[i] = static_cast<uint8_t*>(reg->peer[i]);
  EpochCtl ectl{reinterpret_cast<uint32_t*>(prm.peer[prm.rank] + lay->off_epoch_ag),
                reinterpret_cast<uint32_t*>(prm.peer[prm.rank] + lay->off_epoch_ag + 4)};
  if (static_cast<int64_t>(M) * K * 2 > lay->xall_half_bytes) return -kTooLarge;
  if (static_cast<int64_t>(reg->tp) * prm.chunks_per_rank * 4 > lay->ag_flags_bytes) return -kTooLarge;
  prm.off_xall = lay->off_xall + parity * lay->xall_half_bytes;
  prm.row_bytes = static_cast<int64_t>(K) * 2;
  prm.off_flags = lay->off_ag_flags;
  prm.n_comm = prm.chunks_per_rank < 32 ? prm.chunks_per_rank : 32;
  prm.timeout_ns = timeout_ns;
  constexpr int kPushSmem = kAgRingBytes + 64 + 128;
  static DeviceOnce attr_once;
  if (const int rc = attr_once.run([&] {
        cudaError_t e = cudaFuncSetAttribute(ag_push_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPushSmem);
        return e;
      }))
    return rc;
  launch_pdl(ag_push_kernel, dim3(prm.n_comm), dim3(256), kPushSmem, stream, prm, ectl, status);
  return last_launch_rc();
}

extern "C" int b2_symm_barrier(const B2TpRegion* reg, const B2TpLayout* lay, uint64_t timeout_ns, b2::Status* status,
                               cudaStream_t stream) {
  if (reg == nullptr || lay == nullptr || reg->tp < 1 || reg->tp > kMaxTp) return -kBadArgument;
  uint8_t* self = static_cast<uint8_t*>(reg->peer[reg->rank]);
  EpochCtl ectl{reinterpret_cast<uint32_t*>(self + lay->off_epoch_bar), reinterpret_cast<uint32_t*>(self + lay->off_epoch_bar + 4)};
  launch_pdl(symm_barrier_kernel, dim3(1), dim3(32), 0, stream, *reg, lay->off_barrier, ectl, timeout_ns, status);
  return last_launch_rc();
}

extern "C" int b2_wait_flag(const uint32_t* flag, uint32_t want, uint64_t timeout_ns, b2::Status* status,
                            cudaStream_t stream) {
  launch_pdl(wait_flag_kernel, dim3(1), dim3(32), 0, stream, flag, want, timeout_ns, status);
  return last_launch_rc();
}
