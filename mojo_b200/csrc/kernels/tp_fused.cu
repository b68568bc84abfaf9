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
#include "b2/gemm_tc.cuh"
#include "b2/ptx.cuh"
#include "b2/tma.h"
#include "b2/tp.h"
#include "b2/tp_rs.cuh"
#include "b2/vec.cuh"

namespace b2 {
namespace {

using gemm::WorkUnit;
using namespace b2::tp;
template <int BN, int STAGES, bool SWAP>
__global__ void __launch_bounds__(gemm::kThreads, 1)
gemm_rs_kernel(const __grid_constant__ CUtensorMap tmap_p, const __grid_constant__ CUtensorMap tmap_q,
               const __grid_constant__ RsSched sched, RsParams prm_in, EpochCtl ectl, int n_gemm, Status* status) {
  constexpr uint32_t idesc = ptx::make_idesc(1, 1, 128, BN);
  RsParams prm = prm_in;
  prm.epoch = epoch_begin(ectl);
  if (static_cast<int>(blockIdx.x) < n_gemm) {
    extern __shared__ uint8_t smem_dyn[];
    uint8_t* epi_buf = smem_dyn + gemm::SmemLayout<BN, STAGES>::kTotalBytes;
    epi_buf += (16 - (reinterpret_cast<uintptr_t>(epi_buf) & 15)) & 15;  // 16-byte vector accesses
    RsEpilogue<BN, SWAP> epi{prm, epi_buf};
    gemm::run<BN, STAGES, 2>(&tmap_p, &tmap_q, idesc, ptx::kEvictNormal, ptx::kEvictNormal, sched, gemm::NoGate{}, epi, status,
                             static_cast<int>(blockIdx.x), n_gemm);
  }
  reduce_phase<BN, SWAP>(prm, status);
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
  auto kern = gemm_rs_kernel<BN, STAGES, SWAP>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) return -kBadArgument;
    attr_set = true;
  }
  // Full persistent grid: the last CTAs only reduce from the start, the others join once their tiles are done.
  // large M is GEMM-bound and the reduction of the last units is a short tail: give the GEMM more CTAs
  const int n_red = prm.tp > 1 ? (M >= 2048 ? 4 : 12) : 0;
  const int total = sched.p_blocks * sched.q_blocks;
  int n_gemm = kNumSMs - n_red;
  if (total < n_gemm) n_gemm = total;
  kern<<<kNumSMs, gemm::kThreads, SMEM, stream>>>(tp, tq, sched, prm, ectl, n_gemm, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -kBadArgument;
}

// ------------------------------------------------------------------------------------------------
// all-gather -> GEMM
// ------------------------------------------------------------------------------------------------
struct AgParams {
  int rank, tp;
  int M, K;           // gathered rows, columns of X
  int R;              // rows per rank (M = R * tp)
  int chunk_rows;     // rows per flag chunk
  int chunks_per_rank;
  uint32_t epoch;
  uint8_t* peer[kMaxTp];
  int64_t off_xall;   // bf16 [M][K] of the current parity
  int64_t off_flags;  // u32 [tp][chunks_per_rank]
  int n_comm;         // CTAs that only move data
  uint64_t timeout_ns;
};

// Producer gate: before the first load of a tile, wait until every chunk of X rows it covers has arrived.
struct AgGate {
  AgParams p;
  bool swap;
  int bn;
  __device__ __forceinline__ bool operator()(const WorkUnit& u, Status* status) const {
    const int m_lo = swap ? u.qb * bn : u.pb * 128;
    const int m_hi = min(p.M, m_lo + (swap ? bn : 128)) - 1;
    if (m_hi < m_lo) return true;
    const uint32_t* flags = reinterpret_cast<const uint32_t*>(p.peer[p.rank] + p.off_flags);
    bool waited = false;
    for (int m = m_lo; m <= m_hi;) {
      const int src = m / p.R;
      const int c = (m - src * p.R) / p.chunk_rows;
      if (src != p.rank) {
        if (!ptx::wait_flag_ge_sys(flags + src * p.chunks_per_rank + c, p.epoch, p.timeout_ns)) {
          status_record(status, kTimeout, kSiteAgChunk, src, c);
          return false;
        }
        waited = true;
      }
      m = src * p.R + (c + 1) * p.chunk_rows;  // first row of the next chunk
    }
    // the rows were written by peers' ordinary stores; the loads that follow go through the async proxy
    if (waited) ptx::fence_proxy_async_all();
    return true;
  }
};

// Row-tile order: own rows first, then the peers' in ring order (rank + 1, rank + 2, ...).
struct AgSched {
  int p_blocks, q_blocks, num_kb, bn;
  int m_tiles, first_tile;
  bool swap;
  __device__ __forceinline__ int total() const { return p_blocks * q_blocks; }
  __device__ __forceinline__ WorkUnit get(int w) const {
    WorkUnit u;
    const int n_tiles = swap ? p_blocks : q_blocks;
    const int mt = (first_tile + w / n_tiles) % m_tiles;
    const int nt = w % n_tiles;
    u.pb = swap ? nt : mt;
    u.qb = swap ? mt : nt;
    u.split = 0;
    u.tile = u.pb * q_blocks + u.qb;
    u.kb0 = 0;
    u.kb1 = num_kb;
    u.p_coord = u.pb * 128;
    u.q_coord = u.qb * bn;
    return u;
  }
};

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

// Data-movement CTAs: copy this rank's rows into every peer's gathered buffer, one flag per chunk per peer.
// A chunk of rows is one contiguous byte range, so one thread drives it with bulk async copies: local memory ->
// shared memory (mbarrier completion) -> every peer (bulk store), 32 KB pieces through a 4-deep ring with the
// loads issued two pieces ahead. `smem` is a 128-byte aligned shared-memory window of kAgRingBytes + 64.
constexpr int kAgPiece = 32 * 1024;
constexpr int kAgStages = 4;
constexpr int kAgRingBytes = kAgPiece * kAgStages;

__device__ void ag_push(const AgParams& p, int comm_cta, uint8_t* smem, Status* status) {
  if (threadIdx.x != 0) return;
  const uint32_t ring = ptx::smem_u32(smem);
  const uint32_t bars = ring + kAgRingBytes;
  for (int s = 0; s < kAgStages; ++s) ptx::mbar_init(bars + 8 * s, 1);
  ptx::fence_mbar_init();
  const int row0 = p.rank * p.R;
  const uint8_t* src = p.peer[p.rank] + p.off_xall;
  const int64_t row_bytes = static_cast<int64_t>(p.K) * 2;
  long issued = 0, consumed = 0;  // pieces over the whole kernel (ring positions / phases)
  for (int c = comm_cta; c < p.chunks_per_rank; c += p.n_comm) {
    const int r_lo = row0 + c * p.chunk_rows;
    const int r_hi = min(min(p.M, row0 + p.R), r_lo + p.chunk_rows);
    const int64_t base = static_cast<int64_t>(r_lo) * row_bytes;
    const int64_t total = static_cast<int64_t>(max(0, r_hi - r_lo)) * row_bytes;
    const int n_pieces = static_cast<int>((total + kAgPiece - 1) / kAgPiece);
    int next_load = 0;
    bool ok = true;
    for (int i = 0; i < n_pieces && ok; ++i) {
      // keep two loads in flight; a ring slot is reusable once the stores that read it have finished reading
      while (next_load < n_pieces && next_load < i + 2) {
        if (issued >= kAgStages) ptx::tma_store_wait_read<kAgStages - 2>();
        const int s = static_cast<int>(issued % kAgStages);
        const int64_t off = static_cast<int64_t>(next_load) * kAgPiece;
        const uint32_t bytes = static_cast<uint32_t>((total - off < kAgPiece ? total - off : static_cast<int64_t>(kAgPiece)));
        ptx::mbar_arrive_expect_tx(bars + 8 * s, bytes);
        ptx::bulk_load(ring + s * kAgPiece, src + base + off, bytes, bars + 8 * s);
        ++issued;
        ++next_load;
      }
      const int s = static_cast<int>(consumed % kAgStages);
      if (!ptx::mbar_wait(bars + 8 * s, static_cast<uint32_t>((consumed / kAgStages) & 1))) {
        status_record(status, kTimeout, kSiteAgChunk, c, i);
        ok = false;
        break;
      }
      const int64_t off = static_cast<int64_t>(i) * kAgPiece;
      const uint32_t bytes = static_cast<uint32_t>((total - off < kAgPiece ? total - off : static_cast<int64_t>(kAgPiece)));
      for (int d = 1; d < p.tp; ++d) {
        const int peer = (p.rank + d) % p.tp;
        ptx::bulk_store(p.peer[peer] + p.off_xall + base + off, ring + s * kAgPiece, bytes);
      }
      ptx::tma_store_commit();
      ++consumed;
    }
    // the chunk is complete on every peer before its flag goes up
    ptx::tma_store_wait<0>();
    ptx::fence_proxy_async_all();
    __threadfence_system();
    if (ok)
      for (int d = 1; d < p.tp; ++d) {
        const int peer = (p.rank + d) % p.tp;
        ptx::st_release_sys(reinterpret_cast<uint32_t*>(p.peer[peer] + p.off_flags) + p.rank * p.chunks_per_rank + c, p.epoch);
      }
    if (!ok) {
      // let loads that were issued but not consumed land before the shared memory is released
      while (consumed < issued) {
        ptx::mbar_wait(bars + 8 * static_cast<int>(consumed % kAgStages), static_cast<uint32_t>((consumed / kAgStages) & 1), 200000000ull);
        ++consumed;
      }
      return;
    }
  }
}

template <int BN, int STAGES, bool SWAP>
__global__ void __launch_bounds__(gemm::kThreads, 1)
ag_gemm_kernel(const __grid_constant__ CUtensorMap tmap_p, const __grid_constant__ CUtensorMap tmap_q, AgSched sched,
               AgParams prm_in, PlainEpiParams ep, EpochCtl ectl, Status* status) {
  AgParams prm = prm_in;
  prm.epoch = epoch_begin(ectl);
  const int n_gemm = static_cast<int>(gridDim.x) - prm.n_comm;
  if (static_cast<int>(blockIdx.x) >= n_gemm) {
    extern __shared__ uint8_t smem_dyn[];
    uint8_t* win = smem_dyn + ((128 - (reinterpret_cast<uintptr_t>(smem_dyn) & 127)) & 127);
    ag_push(prm, static_cast<int>(blockIdx.x) - n_gemm, win, status);
    epoch_end(ectl, prm.epoch);
    return;
  }
  constexpr uint32_t idesc = ptx::make_idesc(1, 1, 128, BN);
  PlainEpilogue<BN, SWAP> epi{ep};
  AgGate gate{prm, SWAP, BN};
  gemm::run<BN, STAGES, 2>(&tmap_p, &tmap_q, idesc, ptx::kEvictNormal, ptx::kEvictNormal, sched, gate, epi, status,
                           static_cast<int>(blockIdx.x), n_gemm);
  epoch_end(ectl, prm.epoch);
}

// Standalone push all-gather (no GEMM): used where the gathered rows feed something other than a GEMM.
__global__ void __launch_bounds__(256) ag_push_kernel(AgParams prm_in, EpochCtl ectl, Status* status) {
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
  auto kern = ag_gemm_kernel<BN, STAGES, SWAP>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotalBytes) != cudaSuccess) return -kBadArgument;
    attr_set = true;
  }
  const int total = sched.p_blocks * sched.q_blocks;
  int n_gemm = kNumSMs - prm.n_comm;
  if (total < n_gemm) n_gemm = total;
  kern<<<n_gemm + prm.n_comm, gemm::kThreads, L::kTotalBytes, stream>>>(tp, tq, sched, prm, ep, ectl, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -kBadArgument;
}

// Cross-GPU barrier: every rank raises its slot on every peer, then waits for all slots.
__global__ void symm_barrier_kernel(B2TpRegion reg, int64_t off_flags, EpochCtl ectl, uint64_t timeout_ns, Status* status) {
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
  if (threadIdx.x == 0 && !ptx::wait_flag_ge_sys(flag, want, timeout_ns)) status_record(status, kTimeout, kSiteTest, want, 0);
}

// rows per all-gather flag chunk: about 16 chunks per rank, at most 128 rows each
int ag_chunk_rows(int R) {
  int c = (R + 15) / 16;
  if (c > 128) c = 128;
  if (c < 1) c = 1;
  return c;
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
  bool swap = M <= 128;
  int bn = swap ? pick_bn_swap(M) : (M >= 2048 ? 256 : 128);
  if (config != 0) {
    swap = (config >> 30) & 1;
    bn = config & 0xffff;
  }
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
      case 256: B2_RS(256, true);
      default: return -kBadArgument;
    }
  }
  switch (bn) {
    case 64: B2_RS(64, false);
    case 128: B2_RS(128, false);
    case 256: B2_RS(256, false);
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
  prm.off_flags = lay->off_ag_flags;
  prm.n_comm = prm.chunks_per_rank < 32 ? prm.chunks_per_rank : 32;
  prm.timeout_ns = timeout_ns;
  constexpr int kPushSmem = kAgRingBytes + 64 + 128;
  static bool push_attr = false;
  if (!push_attr) {
    if (cudaFuncSetAttribute(ag_push_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPushSmem) != cudaSuccess) return -kBadArgument;
    push_attr = true;
  }
  ag_push_kernel<<<prm.n_comm, 256, kPushSmem, stream>>>(prm, ectl, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -kBadArgument;
}

extern "C" int b2_symm_barrier(const B2TpRegion* reg, const B2TpLayout* lay, uint64_t timeout_ns, b2::Status* status,
                               cudaStream_t stream) {
  if (reg == nullptr || lay == nullptr || reg->tp < 1 || reg->tp > kMaxTp) return -kBadArgument;
  uint8_t* self = static_cast<uint8_t*>(reg->peer[reg->rank]);
  EpochCtl ectl{reinterpret_cast<uint32_t*>(self + lay->off_epoch_bar), reinterpret_cast<uint32_t*>(self + lay->off_epoch_bar + 4)};
  symm_barrier_kernel<<<1, 32, 0, stream>>>(*reg, lay->off_barrier, ectl, timeout_ns, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -kBadArgument;
}

extern "C" int b2_wait_flag(const uint32_t* flag, uint32_t want, uint64_t timeout_ns, b2::Status* status,
                            cudaStream_t stream) {
  wait_flag_kernel<<<1, 32, 0, stream>>>(flag, want, timeout_ns, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -kBadArgument;
}
