// Shared pieces of the fused row-parallel GEMM -> reduce-scatter / all-reduce kernels (bf16 and fp8 mainloops):
// launch-epoch control, parameters, the staged peer-write epilogue, the reduce phase and the row-tile visiting
// order. See csrc/kernels/tp_fused.cu for the protocol description.
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_bf16.h>
#include "b2/gemm_tc.cuh"
#include "b2/ptx.cuh"
#include "b2/status.h"
#include "b2/vec.cuh"

namespace b2 {
namespace tp {

using gemm::WorkUnit;
constexpr int kMaxTp = 8;

// Launch epochs live in device memory so that a CUDA graph replay sees a fresh value: every CTA reads
// `*epoch_ptr + 1` when it starts, and the CTA that finishes last (all others have therefore started and read)
// stores the new value. All ranks issue the same sequence of fused launches, so their epochs agree.
struct EpochCtl {
  uint32_t* epoch_ptr;
  uint32_t* cta_done;
};
__device__ __forceinline__ uint32_t epoch_begin(const EpochCtl& c) {
  return *reinterpret_cast<volatile uint32_t*>(c.epoch_ptr) + 1u;
}
__device__ __forceinline__ void epoch_end(const EpochCtl& c, uint32_t epoch) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(c.cta_done, 1u) == gridDim.x - 1) {
      *c.cta_done = 0;
      *reinterpret_cast<volatile uint32_t*>(c.epoch_ptr) = epoch;
      __threadfence();
    }
  }
}

struct RsParams {
  int rank, tp;
  int M, N;
  int R;              // rows owned per rank (ceil(M / tp))
  uint32_t epoch;
  int mode;           // 0 reduce-scatter, 1 all-reduce
  int p_blocks, q_blocks;
  uint8_t* peer[kMaxTp];   // base of every rank's symmetric region
  int64_t off_staging;     // bf16 [tp][R][N] of the current parity
  int64_t off_flags;       // u32 [units][tp]
  int64_t off_yall;        // bf16 [M][N] of the current parity (all-reduce result)
  int64_t off_resflags;    // u32 [tp]
  int64_t off_done;        // u32 local counter
  const __nv_bfloat16* residual;  // reduce-scatter: [R, N] local rows; all-reduce: [M, N]
  __nv_bfloat16* out;             // reduce-scatter result [R, N]
  uint64_t timeout_ns;
  int64_t region_bytes;    // size of every rank's symmetric region: accesses into it are checked against this bound
  Status* status;          // where a failed bounds check is recorded (the access is skipped)
  // In-switch reduction (NVLS): with a multicast mapping of the region, a rank keeps its partial tiles in its OWN staging
  // half, laid out like the result ([M][N] bf16), and only raises the owner's flag; the owner then reads each 16-byte
  // vector of its rows once with multimem.ld_reduce, which returns the sum over all ranks (added in f32 inside the
  // switch). NVLink carries each partial byte once, pulled, and the owner issues one load where the peer-store form
  // issues tp. All-reduce mode stores the result with one multimem.st instead of tp peer stores. Null: peer-store form.
  uint8_t* mc_base;
};

// Bounds check of a 16-byte access at byte offset `off` of a symmetric region; `what` names the access in the record.
__device__ __forceinline__ bool rs_in_region(const RsParams& p, int64_t off, int what) {
  return B2_ASSERT(p.status, p.region_bytes == 0 || (off >= 0 && off + 16 <= p.region_bytes), kSiteRsTile, what, off);
}

// Index of tile (pb, qb) among the units of `owner` (tiles that overlap the owner's rows).
template <bool SWAP, int BN>
__device__ __forceinline__ int unit_index(const RsParams& p, int owner, int pb, int qb) {
  if (!SWAP) return (pb - (owner * p.R) / 128) * p.q_blocks + qb;
  return (qb - (owner * p.R) / BN) * p.p_blocks + pb;
}

// Bytes of shared memory the reduce-scatter epilogue needs behind the GEMM core's own layout.
constexpr int kRsRowPad = 16;
template <int BN, bool SWAP>
constexpr int rs_epi_bytes() {
  // normal: two buffers of [128 rows][64 cols] bf16; swapped: two buffers of [32 tokens][128 cols] bf16
  return SWAP ? 2 * 32 * (256 + kRsRowPad) : 2 * 128 * (128 + kRsRowPad);
}

// Epilogue of the reduce-scatter GEMM. NVLink moves small scattered writes badly, so the accumulator is first
// transposed through shared memory and then leaves the SM as 128-byte (normal) or 256-byte (swapped) row
// segments of consecutive 16-byte stores, straight into the owner rank's staging buffer.
template <int BN, bool SWAP>
struct RsEpilogue {
  static constexpr int CH = BN >= 32 ? 32 : 16;
  RsParams p;
  uint8_t* epi_smem;

  __device__ __forceinline__ __nv_bfloat16* staging_row(int m) const {
    if (p.mc_base != nullptr)   // in-switch form: the partial stays here, at its place in the [M][N] result
      return reinterpret_cast<__nv_bfloat16*>(p.peer[p.rank] + p.off_staging) + static_cast<int64_t>(m) * p.N;
    const int owner = m / p.R;
    return reinterpret_cast<__nv_bfloat16*>(p.peer[owner] + p.off_staging) +
           (static_cast<int64_t>(p.rank) * p.R + (m - owner * p.R)) * p.N;
  }

  // byte offset inside the (owner's, or with in-switch reduction this rank's) region of column n of row m as written by this rank
  __device__ __forceinline__ int64_t staging_off(int m, int n) const {
    if (p.mc_base != nullptr) return p.off_staging + (static_cast<int64_t>(m) * p.N + n) * 2;
    const int owner = m / p.R;
    return p.off_staging + ((static_cast<int64_t>(p.rank) * p.R + (m - owner * p.R)) * p.N + n) * 2;
  }

  // TMEM-backed epilogue (bf16 GEMM core)
  __device__ __forceinline__ void operator()(const WorkUnit& u, uint32_t taddr, int quarter, int lane, uint32_t* flag,
                                             Status* status) const {
    (void)flag; (void)status;
    write_tile(u, quarter, lane, [&](int col0, uint32_t (&r)[CH]) {
      if constexpr (CH == 32) ptx::tmem_ld_32x32(taddr + col0, r);
      else ptx::tmem_ld_32x16(taddr + col0, r);
      ptx::tc_wait_ld();
    });
  }

  // `load(col0, r)` fills r with the CH accumulator columns [col0, col0 + CH) of this thread's row (f32 bit patterns).
  // The loops are fully unrolled so a register-resident accumulator can be indexed with constants.
  template <class Load>
  __device__ __forceinline__ void write_tile(const WorkUnit& u, int quarter, int lane, Load load) const {
    const int p_local = quarter * 32 + lane;
    const int t = static_cast<int>(threadIdx.x) - 64;  // 0..127 among the epilogue threads
    if constexpr (!SWAP) {
      constexpr int ROW = 128 + kRsRowPad;               // bytes per staged row (64 bf16 + pad)
      static_assert(BN % 64 == 0, "normal layout stages 64 columns at a time");
#pragma unroll
      for (int cg = 0; cg < BN / 64; ++cg) {
        uint8_t* buf = epi_smem + (cg & 1) * 128 * ROW;
#pragma unroll
        for (int c2 = 0; c2 < 2; ++c2) {
          uint32_t r[32];
          load(cg * 64 + c2 * 32, r);
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 pk;
            pk.x = ptx::pack_bf16x2(__uint_as_float(r[g * 8 + 0]), __uint_as_float(r[g * 8 + 1]));
            pk.y = ptx::pack_bf16x2(__uint_as_float(r[g * 8 + 2]), __uint_as_float(r[g * 8 + 3]));
            pk.z = ptx::pack_bf16x2(__uint_as_float(r[g * 8 + 4]), __uint_as_float(r[g * 8 + 5]));
            pk.w = ptx::pack_bf16x2(__uint_as_float(r[g * 8 + 6]), __uint_as_float(r[g * 8 + 7]));
            *reinterpret_cast<uint4*>(buf + p_local * ROW + c2 * 64 + g * 16) = pk;
          }
        }
        ptx::named_barrier_sync(1, gemm::kEpiThreads);
        const int n0 = u.qb * BN + cg * 64;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int v = t + 128 * i;
          const int row = v >> 3, cv = v & 7;
          const int m = u.pb * 128 + row;
          if (m < p.M && n0 + cv * 8 < p.N && rs_in_region(p, staging_off(m, n0 + cv * 8), 1))
            ptx::st_v4(staging_row(m) + n0 + cv * 8, *reinterpret_cast<const uint4*>(buf + row * ROW + cv * 16));
        }
      }
    } else {
      constexpr int ROW = 256 + kRsRowPad;               // bytes per staged token row (128 bf16 + pad)
#pragma unroll
      for (int c = 0; c < BN / CH; ++c) {
        uint8_t* buf = epi_smem + (c & 1) * 32 * ROW;
        uint32_t r[CH];
        load(c * CH, r);
#pragma unroll
        for (int j = 0; j < CH; ++j)
          *reinterpret_cast<__nv_bfloat16*>(buf + j * ROW + p_local * 2) = __float2bfloat16(__uint_as_float(r[j]));
        ptx::named_barrier_sync(1, gemm::kEpiThreads);
        const int m0 = u.qb * BN + c * CH;
#pragma unroll
        for (int i = 0; i < CH / 8; ++i) {
          const int v = t + 128 * i;
          const int j = v >> 4, cv = v & 15;
          const int m = m0 + j, n = u.pb * 128 + cv * 8;
          if (m < p.M && n < p.N && rs_in_region(p, staging_off(m, n), 2))
            ptx::st_v4(staging_row(m) + n, *reinterpret_cast<const uint4*>(buf + j * ROW + cv * 16));
        }
      }
    }
    // publish: the barrier orders every epilogue thread's stores before the signalling threads (CTA scope); each of
    // those then fences at system scope and releases one flag per owner this tile touched. One fence per flag
    // instead of one per thread: the per-thread form showed up as the top stall of this epilogue.
    ptx::named_barrier_sync(1, gemm::kEpiThreads);
    const int m_lo = SWAP ? u.qb * BN : u.pb * 128;
    const int m_hi = min(p.M, m_lo + (SWAP ? BN : 128)) - 1;
    const int o_lo = m_lo / p.R, o_hi = m_hi / p.R;
    if (t <= o_hi - o_lo) {
      __threadfence_system();
      const int owner = o_lo + t;
      const int unit = unit_index<SWAP, BN>(p, owner, u.pb, u.qb);
      uint32_t* f = reinterpret_cast<uint32_t*>(p.peer[owner] + p.off_flags) + static_cast<int64_t>(unit) * p.tp + p.rank;
      if (rs_in_region(p, p.off_flags + (static_cast<int64_t>(unit) * p.tp + p.rank) * 4 - 12, 6)) ptx::st_release_sys(f, p.epoch);
    }
  }
};

// Reduce phase. Units (output tiles of the rows this rank owns) are claimed from a counter in this rank's
// memory, in the order in which their contributions are produced, by the dedicated reduce CTAs from the start
// and by the GEMM CTAs once they run out of tiles. Returns false when a wait ran out.
// `Team` says which threads of the CTA do the reducing: the whole CTA, or the two side warps of a GEMM CTA.
struct CtaTeam {
  static __device__ __forceinline__ int tid() { return static_cast<int>(threadIdx.x); }
  static __device__ __forceinline__ int size() { return static_cast<int>(blockDim.x); }
  static __device__ __forceinline__ void sync() { __syncthreads(); }
};
struct SideTeam {  // warps 6..7 of a CTA whose warps 0..5 run the GEMM roles (8 warps keep 255 registers per thread)
  static constexpr int kThreads = 64;
  static __device__ __forceinline__ int tid() { return static_cast<int>(threadIdx.x) - gemm::kThreads; }
  static __device__ __forceinline__ int size() { return kThreads; }
  static __device__ __forceinline__ void sync() { ptx::named_barrier_sync(4, kThreads); }
};

template <int BN, bool SWAP, class Team = CtaTeam>
__device__ inline bool reduce_phase(const RsParams& p, Status* status) {
  __shared__ uint32_t sh_ok;
  __shared__ uint32_t sh_last;
  __shared__ int sh_unit;
  const int row0 = p.rank * p.R;
  const int rows = max(0, min(p.R, p.M - row0));
  uint8_t* self = p.peer[p.rank];
  const uint32_t* flags = reinterpret_cast<const uint32_t*>(self + p.off_flags);
  const __nv_bfloat16* staging = reinterpret_cast<const __nv_bfloat16*>(self + p.off_staging);
  uint32_t* next_unit = reinterpret_cast<uint32_t*>(self + p.off_done);
  uint32_t* done = next_unit + 1;
  constexpr int TM = SWAP ? BN : 128;
  constexpr int TN = SWAP ? 128 : BN;
  const int tm0 = row0 / TM;
  const int tm1 = rows > 0 ? (row0 + rows - 1) / TM + 1 : tm0;
  const int n_tiles_n = SWAP ? p.p_blocks : p.q_blocks;
  const int n_units = (tm1 - tm0) * n_tiles_n;
  bool ok = true;
  while (true) {
    Team::sync();
    if (Team::tid() == 0) {
      sh_unit = static_cast<int>(atomicAdd(next_unit, 1u));
      sh_ok = 1;
    }
    Team::sync();
    const int un = sh_unit;
    if (un >= n_units) break;
    // same enumeration as unit_index(): (tile along m) major, (tile along n) minor
    const int tm = tm0 + un / n_tiles_n, tn = un % n_tiles_n;
    if (Team::tid() < p.tp) {
      if (!rs_in_region(p, p.off_flags + (static_cast<int64_t>(un) * p.tp + Team::tid()) * 4 - 12, 5)) {
        sh_ok = 0;
      } else if (!ptx::wait_flag_ge_sys(flags + static_cast<int64_t>(un) * p.tp + Team::tid(), p.epoch, p.timeout_ns)) {
        status_record(status, kTimeout, kSiteRsTile, un, Team::tid());
        sh_ok = 0;
      }
    }
    Team::sync();
    if (sh_ok == 0) { ok = false; break; }
    const int r_lo = max(row0, tm * TM), r_hi = min(row0 + rows, tm * TM + TM);
    const int c_lo = tn * TN, c_hi = min(p.N, tn * TN + TN);
    const int vec_per_row = (c_hi - c_lo) >> 3;
    const int n_vec = (r_hi - r_lo) * vec_per_row;
    if (p.mc_base != nullptr) {
      // in-switch form: one multimem.ld_reduce per 16-byte vector returns the sum of all ranks' partials
      constexpr int UN = 8;
      for (int i0 = Team::tid(); i0 < n_vec; i0 += Team::size() * UN) {
        uint4 sum[UN];
        int64_t el[UN];   // element offset of the vector in the [M][N] result
#pragma unroll
        for (int u = 0; u < UN; ++u) {
          const int i = i0 + u * Team::size();
          const int m = r_lo + (i < n_vec ? i / vec_per_row : 0);
          const int col = c_lo + (i < n_vec ? (i % vec_per_row) * 8 : 0);
          el[u] = static_cast<int64_t>(m) * p.N + col;
          if (i < n_vec && rs_in_region(p, p.off_staging + el[u] * 2, 3)) sum[u] = ptx::multimem_ld_reduce_bf16x8(p.mc_base + p.off_staging + el[u] * 2);
          else sum[u] = make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < UN; ++u) {
          const int i = i0 + u * Team::size();
          if (i >= n_vec) continue;
          uint4 pk = sum[u];
          const int m = static_cast<int>(el[u] / p.N);
          const int col = static_cast<int>(el[u] - static_cast<int64_t>(m) * p.N);
          if (p.residual != nullptr) {
            float acc[8], v[8];
            bf16x8_to_f32(pk, acc);
            const int64_t rrow = p.mode == 0 ? m - row0 : m;
            bf16x8_to_f32(ptx::ld_v4(p.residual + rrow * p.N + col), v);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += v[j];
            pk = f32_to_bf16x8(acc);
          }
          if (p.mode == 0) {
            ptx::st_v4(p.out + static_cast<int64_t>(m - row0) * p.N + col, pk);
          } else if (rs_in_region(p, p.off_yall + el[u] * 2, 4)) {
            ptx::multimem_st_v4(p.mc_base + p.off_yall + el[u] * 2, pk);   // the switch writes every rank's copy
          }
        }
      }
    } else {
    constexpr int U = 4;  // independent 16-byte vectors per thread per pass: keeps tp * U loads in flight
    for (int i0 = Team::tid(); i0 < n_vec; i0 += Team::size() * U) {
      uint4 raw[U][kMaxTp];
      int64_t off[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = i0 + u * Team::size();
        const int m = r_lo + (i < n_vec ? i / vec_per_row : 0);
        const int col = c_lo + (i < n_vec ? (i % vec_per_row) * 8 : 0);
        off[u] = static_cast<int64_t>(m - row0) * p.N + col;
#pragma unroll
        for (int s2 = 0; s2 < kMaxTp; ++s2)
          if (s2 < p.tp && i < n_vec && rs_in_region(p, p.off_staging + (static_cast<int64_t>(s2) * p.R * p.N + off[u]) * 2, 3))
            raw[u][s2] = ptx::ld_relaxed_sys_v4(staging + static_cast<int64_t>(s2) * p.R * p.N + off[u]);
          else if (s2 < p.tp)
            raw[u][s2] = make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = i0 + u * Team::size();
        if (i >= n_vec) continue;
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
        for (int s2 = 0; s2 < kMaxTp; ++s2) {
          if (s2 < p.tp) {
            float v[8];
            bf16x8_to_f32(raw[u][s2], v);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += v[j];
          }
        }
        const int row_local = static_cast<int>(off[u] / p.N);
        const int col = static_cast<int>(off[u] - static_cast<int64_t>(row_local) * p.N);
        const int m = row0 + row_local;
        if (p.residual != nullptr) {
          float v[8];
          const int64_t rrow = p.mode == 0 ? row_local : m;
          bf16x8_to_f32(ptx::ld_v4(p.residual + rrow * p.N + col), v);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += v[j];
        }
        const uint4 pk = f32_to_bf16x8(acc);
        if (p.mode == 0) {
          ptx::st_v4(p.out + off[u], pk);
        } else {
#pragma unroll 1
          for (int d = 0; d < p.tp; ++d) {
            const int peer = (p.rank + d) % p.tp;  // local copy first, then around the ring
            if (!rs_in_region(p, p.off_yall + (static_cast<int64_t>(m) * p.N + col) * 2, 4)) continue;
            ptx::st_v4(reinterpret_cast<__nv_bfloat16*>(p.peer[peer] + p.off_yall) + static_cast<int64_t>(m) * p.N + col, pk);
          }
        }
      }
    }
    }
    if (p.mode == 1) {
      __threadfence_system();
      Team::sync();
      if (Team::tid() == 0) {
        const uint32_t old = atomicAdd(done, 1u);
        sh_last = (old == static_cast<uint32_t>(n_units - 1)) ? 1u : 0u;
        if (sh_last) *done = 0;
      }
      Team::sync();
      if (sh_last && Team::tid() < p.tp)
        ptx::st_release_sys(reinterpret_cast<uint32_t*>(p.peer[Team::tid()] + p.off_resflags) + p.rank, p.epoch);
    }
  }
  if (p.mode == 1) {
    // a rank that owns no rows still announces that it has entered this launch
    if (n_units == 0 && blockIdx.x == 0 && Team::tid() < p.tp)
      ptx::st_release_sys(reinterpret_cast<uint32_t*>(p.peer[Team::tid()] + p.off_resflags) + p.rank, p.epoch);
    // the launch is complete when every rank's rows have landed in this rank's copy
    Team::sync();
    if (Team::tid() == 0) sh_ok = ok ? 1u : 0u;
    Team::sync();
    if (ok && Team::tid() < p.tp) {
      const uint32_t* rf = reinterpret_cast<const uint32_t*>(self + p.off_resflags) + Team::tid();
      if (!ptx::wait_flag_ge_sys(rf, p.epoch, p.timeout_ns)) {
        status_record(status, kTimeout, kSitePeerSignal, Team::tid(), p.epoch);
        sh_ok = 0;
      }
    }
    Team::sync();
    ok = sh_ok != 0;
  }
  return ok;
}

// Row-tile visiting order of the reduce-scatter GEMM (built on the host): round-robin over the owners starting
// with rank + 1, one row-tile of each per round. At any moment the ranks are sending to different owners, and
// every owner's tiles complete at a steady rate, so its reduction overlaps the remaining GEMM work.
constexpr int kMaxRowTiles = 512;
struct RsSched {
  int p_blocks, q_blocks, num_kb, bn;
  int m_tiles;
  bool swap;
  int16_t order[kMaxRowTiles];
  __device__ __forceinline__ int total() const { return p_blocks * q_blocks; }
  __device__ __forceinline__ WorkUnit get(int w) const {
    WorkUnit u;
    const int n_tiles = swap ? p_blocks : q_blocks;
    const int mt = order[w / n_tiles];
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


// Host side: fill the row-tile visiting order of `sched` for this rank.
inline bool build_rs_order(RsSched& sched, int tp, int rank, int R, int tile_rows) {
  if (sched.m_tiles > kMaxRowTiles) return false;
  int next_of[kMaxTp], end_of[kMaxTp];
  for (int o = 0; o < tp; ++o) {
    next_of[o] = (o * R + tile_rows - 1) / tile_rows;
    end_of[o] = ((o + 1) * R + tile_rows - 1) / tile_rows;
    if (next_of[o] > sched.m_tiles) next_of[o] = sched.m_tiles;
    if (end_of[o] > sched.m_tiles) end_of[o] = sched.m_tiles;
  }
  next_of[0] = 0;
  end_of[tp - 1] = sched.m_tiles;
  int n = 0;
  while (n < sched.m_tiles) {
    for (int d = 1; d <= tp && n < sched.m_tiles; ++d) {
      const int o = (rank + d) % tp;
      if (next_of[o] < end_of[o]) sched.order[n++] = static_cast<int16_t>(next_of[o]++);
    }
  }
  return true;
}

// Last CTA out of a reduce-scatter kernel: every CTA has made its final (failed) unit claim, so the claim counter
// goes back to zero and the new epoch is published.
__device__ __forceinline__ void rs_epoch_end(const EpochCtl& ectl, const RsParams& prm) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(ectl.cta_done, 1u) == gridDim.x - 1) {
      *ectl.cta_done = 0;
      *reinterpret_cast<uint32_t*>(prm.peer[prm.rank] + prm.off_done) = 0;
      *reinterpret_cast<volatile uint32_t*>(ectl.epoch_ptr) = prm.epoch;
      __threadfence();
    }
  }
}

}  // namespace tp
}  // namespace b2
