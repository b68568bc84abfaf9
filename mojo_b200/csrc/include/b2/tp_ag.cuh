// Shared pieces of the fused all-gather -> column-parallel GEMM kernels (bf16 and fp8 mainloops): parameters,
// the producer gate that waits for a tile's rows, the row-tile visiting order and the data-movement loop of the
// communication CTAs. See csrc/kernels/tp_fused.cu for the protocol description.
#pragma once
#include <cstdint>
#include <cuda.h>
#include "b2/gemm_tc.cuh"
#include "b2/ptx.cuh"
#include "b2/status.h"
#include "b2/tp_rs.cuh"

namespace b2 {
namespace tp {

struct AgParams {
  int rank, tp;
  int M, K;           // gathered rows, columns of X
  int R;              // rows per rank (M = R * tp)
  int chunk_rows;     // rows per flag chunk
  int chunks_per_rank;
  uint32_t epoch;
  uint8_t* peer[kMaxTp];
  int64_t off_xall;   // gathered rows [M][row_bytes] of the current parity
  int64_t row_bytes;  // bytes per gathered row (bf16: K * 2, e4m3: K)
  int64_t off_aux;    // second gathered array [M][aux_row_bytes] (fp8: the f32 scales), moved with the same flags
  int64_t aux_row_bytes;  // 0 = none
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

// Data-movement CTAs: copy this rank's rows into every peer's gathered buffer, one flag per chunk per peer.
// A chunk of rows is one contiguous byte range, so one thread drives it with bulk async copies: local memory ->
// shared memory (mbarrier completion) -> every peer (bulk store), 32 KB pieces through a 4-deep ring with the
// loads issued two pieces ahead. `smem` is a 128-byte aligned shared-memory window of kAgRingBytes + 64.
constexpr int kAgPiece = 32 * 1024;
constexpr int kAgStages = 4;
constexpr int kAgRingBytes = kAgPiece * kAgStages;

__device__ inline void ag_push(const AgParams& p, int comm_cta, uint8_t* smem, Status* status) {
  if (threadIdx.x != 0) return;
  const uint32_t ring = ptx::smem_u32(smem);
  const uint32_t bars = ring + kAgRingBytes;
  for (int s = 0; s < kAgStages; ++s) ptx::mbar_init(bars + 8 * s, 1);
  ptx::fence_mbar_init();
  const int row0 = p.rank * p.R;
  long issued = 0, consumed = 0;  // pieces over the whole kernel (ring positions / phases)
  for (int c = comm_cta; c < p.chunks_per_rank; c += p.n_comm) {
    const int r_lo = row0 + c * p.chunk_rows;
    const int r_hi = min(min(p.M, row0 + p.R), r_lo + p.chunk_rows);
    bool ok = true;
    // the chunk's rows of the main array, then (fp8) its rows of the scale array
    for (int part = 0; part < (p.aux_row_bytes > 0 ? 2 : 1) && ok; ++part) {
    const int64_t row_bytes = part == 0 ? p.row_bytes : p.aux_row_bytes;
    const int64_t off_arr = part == 0 ? p.off_xall : p.off_aux;
    const uint8_t* src = p.peer[p.rank] + off_arr;
    const int64_t base = static_cast<int64_t>(r_lo) * row_bytes;
    const int64_t total = static_cast<int64_t>(max(0, r_hi - r_lo)) * row_bytes;
    const int n_pieces = static_cast<int>((total + kAgPiece - 1) / kAgPiece);
    int next_load = 0;
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
        ptx::bulk_store(p.peer[peer] + off_arr + base + off, ring + s * kAgPiece, bytes);
      }
      ptx::tma_store_commit();
      ++consumed;
    }
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


// Side-warp variant of the push (gemm::run's Side policy): one warp per GEMM CTA moves whole chunks of this rank's
// rows with 16-byte loads and stores, four per lane in flight, then raises the chunk's flag on every peer.
struct AgSidePush {
  static constexpr int kWarps = 1;
  AgParams p;
  int cta, num_ctas;
  __device__ __forceinline__ void operator()(int, int lane) const {
    if (p.tp == 1) return;
    const int row0 = p.rank * p.R;
    for (int c = cta; c < p.chunks_per_rank; c += num_ctas) {
      const int r_lo = row0 + c * p.chunk_rows;
      const int r_hi = min(min(p.M, row0 + p.R), r_lo + p.chunk_rows);
      for (int part = 0; part < (p.aux_row_bytes > 0 ? 2 : 1); ++part) {
        const int64_t row_bytes = part == 0 ? p.row_bytes : p.aux_row_bytes;
        const int64_t off_arr = (part == 0 ? p.off_xall : p.off_aux) + static_cast<int64_t>(r_lo) * row_bytes;
        const int64_t n_vec = static_cast<int64_t>(max(0, r_hi - r_lo)) * row_bytes / 16;
        const uint8_t* src = p.peer[p.rank] + off_arr;
        for (int64_t i0 = lane; i0 < n_vec; i0 += 128) {
          uint4 v[4];
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (i0 + 32 * u < n_vec) v[u] = ptx::ld_v4(src + (i0 + 32 * u) * 16);
          for (int d = 1; d < p.tp; ++d) {
            uint8_t* dst = p.peer[(p.rank + d) % p.tp] + off_arr;
#pragma unroll
            for (int u = 0; u < 4; ++u)
              if (i0 + 32 * u < n_vec) ptx::st_v4(dst + (i0 + 32 * u) * 16, v[u]);
          }
        }
      }
      // the chunk is complete on every peer before its flag goes up
      __threadfence_system();
      __syncwarp();
      if (lane >= 1 && lane < p.tp) {
        const int peer = (p.rank + lane) % p.tp;
        ptx::st_release_sys(reinterpret_cast<uint32_t*>(p.peer[peer] + p.off_flags) + p.rank * p.chunks_per_rank + c, p.epoch);
      }
      __syncwarp();
    }
  }
};

// rows per all-gather flag chunk: about 16 chunks per rank, at most 128 rows each
inline int ag_chunk_rows(int R) {
  int c = (R + 15) / 16;
  if (c > 128) c = 128;
  if (c < 1) c = 1;
  return c;
}

}  // namespace tp
}  // namespace b2
