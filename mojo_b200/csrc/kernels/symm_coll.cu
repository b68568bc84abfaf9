// Standalone collectives over symmetric memory (NVLink peer loads / stores, optional in-switch reduction).
//
// Protocol shared by all kernels. Every launch has an epoch e (kept in device memory, so a CUDA graph replay
// advances it). Flags only grow. A rank raises flag A[e] on every peer when its kernel starts: by stream order
// its input is complete and everything that consumed results of earlier launches has finished. Nobody reads a
// peer's input or writes into a peer's result half before it has seen that peer's A[e]. Kernels that write into
// peers raise B[e] once all their CTAs have fenced their stores, and every rank leaves only after it has seen all
// B[e]. Inputs and results are double-buffered by launch parity: a half is reused two launches later, and a rank
// can only get there after every peer has started the launch in between, hence finished the one before.
// Every wait is bounded; on expiry the kernel records a TIMEOUT status, skips its data phase, still raises the
// flags it owes (so that peers do not wait for it in turn) and returns.
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "b2/coll.h"
#include "b2/launch.h"
#include "b2/config.h"
#include "b2/ptx.cuh"
#include "b2/status.h"
#include "b2/tp_rs.cuh"
#include "b2/vec.cuh"

namespace b2 {
namespace {

using tp::EpochCtl;
constexpr int kCollThreads = 256;

struct CollParams {
  uint8_t* peer[tp::kMaxTp];
  int rank, tp;
  int64_t off_buf, off_out, off_flags_a, off_flags_b, off_counts, off_done;
  uint64_t timeout_ns;
};

// Raise flag `off` (CTA 0 only when `signal`) and wait for every peer's. Returns false when a wait ran out.
__device__ __forceinline__ bool arrive_and_wait(const CollParams& p, int64_t off, uint32_t epoch, bool signal, Status* status) {
  __shared__ uint32_t sh_ok;
  if (threadIdx.x == 0) sh_ok = 1;
  __syncthreads();
  if (threadIdx.x < p.tp) {
    const int t = threadIdx.x;
    if (signal) ptx::st_release_sys(reinterpret_cast<uint32_t*>(p.peer[t] + off) + p.rank, epoch);
    if (!ptx::wait_flag_ge_sys(reinterpret_cast<const uint32_t*>(p.peer[p.rank] + off) + t, epoch, p.timeout_ns)) {
      status_record(status, kTimeout, kSitePeerSignal, t, epoch);
      sh_ok = 0;
    }
  }
  __syncthreads();
  return sh_ok != 0;
}

// After this CTA's peer stores: fence them, count the CTA, and let the last one raise B on every peer.
__device__ __forceinline__ void publish_writes(const CollParams& p, uint32_t epoch) {
  __shared__ uint32_t sh_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t* done = reinterpret_cast<uint32_t*>(p.peer[p.rank] + p.off_done);
    const uint32_t old = atomicAdd(done, 1u);
    sh_last = old == gridDim.x - 1 ? 1u : 0u;
    if (sh_last) *done = 0;
  }
  __syncthreads();
  if (sh_last && threadIdx.x < p.tp)
    ptx::st_release_sys(reinterpret_cast<uint32_t*>(p.peer[threadIdx.x] + p.off_flags_b) + p.rank, epoch);
}

__device__ __forceinline__ uint4 sum_peers(const CollParams& p, int64_t byte_off) {
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
  // fixed rank order: every rank computes bit-identical sums
  for (int r = 0; r < p.tp; ++r) {
    const uint4 v = ptx::ld_relaxed_sys_v4(p.peer[r] + p.off_buf + byte_off);
    float f[8];
    bf16x8_to_f32(v, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] += f[j];
  }
  return f32_to_bf16x8(acc);
}

// ALGO 0: one-shot. ALGO 1: two-shot with peer stores. ALGO 2: two-shot through the multicast mapping.
template <int ALGO>
__global__ void __launch_bounds__(kCollThreads) all_reduce_kernel(CollParams p, EpochCtl ectl, uint8_t* mc_base, uint4* out, int64_t n_vec,
                                                                  Status* status) {
  ptx::grid_dep_sync();
  const uint32_t epoch = tp::epoch_begin(ectl);
  const bool ok = arrive_and_wait(p, p.off_flags_a, epoch, blockIdx.x == 0, status);
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  if (ALGO == 0) {
    if (ok)
      for (int64_t i = tid; i < n_vec; i += nthreads) out[i] = sum_peers(p, i * 16);
  } else {
    const int64_t per = (n_vec + p.tp - 1) / p.tp;
    const int64_t lo = per * p.rank, hi = lo + per < n_vec ? lo + per : n_vec;
    if (ok) {
      for (int64_t i = lo + tid; i < hi; i += nthreads) {
        if (ALGO == 2) {
          const uint4 v = ptx::multimem_ld_reduce_bf16x8(mc_base + p.off_buf + i * 16);
          ptx::multimem_st_v4(mc_base + p.off_out + i * 16, v);
        } else {
          const uint4 v = sum_peers(p, i * 16);
          for (int d = 0; d < p.tp; ++d) ptx::st_v4(p.peer[(p.rank + d) % p.tp] + p.off_out + i * 16, v);
        }
      }
    }
    publish_writes(p, epoch);
    arrive_and_wait(p, p.off_flags_b, epoch, false, status);
  }
  tp::epoch_end(ectl, epoch);
}

// One-shot all-reduce fused with the residual add and the RMSNorm that follow it in a transformer layer:
//   h = bf16(sum over ranks of the partial rows);  residual += h (stored in bf16);  out = rmsnorm(residual) * weight
// One CTA per row at a time; the row stays in registers between the reduction and the scaling (VPT 16-byte
// vectors per thread). Numerics match `all_reduce` followed by the rmsnorm kernel with a residual.
template <int VPT>
__global__ void __launch_bounds__(kCollThreads) all_reduce_rmsnorm_kernel(CollParams p, EpochCtl ectl, uint4* __restrict__ residual,
                                                                          const uint4* __restrict__ weight, uint4* __restrict__ out, int rows,
                                                                          int hidden, float eps, Status* status) {
  ptx::grid_dep_sync();
  __shared__ float scratch[33];
  const uint32_t epoch = tp::epoch_begin(ectl);
  const bool ok = arrive_and_wait(p, p.off_flags_a, epoch, blockIdx.x == 0, status);
  const int nvec = hidden >> 3;
  if (ok) {
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
      const int64_t base = static_cast<int64_t>(row) * nvec;
      float v[VPT][8];
      float ss = 0.0f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + i * kCollThreads;
        if (c < nvec) {
          bf16x8_to_f32(sum_peers(p, (base + c) * 16), v[i]);   // rounded to bf16 like the stand-alone all-reduce
          if (residual != nullptr) {
            float r[8];
            bf16x8_to_f32(residual[base + c], r);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[i][j] += r[j];
            const uint4 packed = f32_to_bf16x8(v[i]);
            residual[base + c] = packed;                        // the stream is stored in bf16: normalise what is stored
            bf16x8_to_f32(packed, v[i]);
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] = 0.0f;
        }
      }
      ss = block_sum(ss, scratch);
      const float rstd = ptx::rsqrt(ss / static_cast<float>(hidden) + eps);
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + i * kCollThreads;
        if (c < nvec) {
          float w[8];
          bf16x8_to_f32(weight[c], w);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] = v[i][j] * rstd * w[j];
          out[base + c] = f32_to_bf16x8(v[i]);
        }
      }
    }
  }
  tp::epoch_end(ectl, epoch);
}

// The same operation through the NVLink switch (NVLS), for messages where the one-shot form's traffic (every rank reads
// every peer's partials: tp - 1 times the message in per rank) is the cost. Rank r owns rows [r * rows_per, ...):
//   * `multimem.ld_reduce` on the multicast address returns the sum over all ranks' partials (added in f32 inside the
//     switch, rounded to bf16), so each partial byte crosses NVLink once and only 1 / tp of the message comes in;
//   * the owner adds the residual rows, normalises, and stores the new residual rows and the normalised rows with
//     `multimem.st`, which the switch replicates into every rank's result half.
// Results therefore live in the symmetric result half: [rows, hidden] normalised, then [rows, hidden] residual.
// Every rank gets bit-identical rows (one rank computed them). Flags A before (all partials are in place), B after.
template <int VPT>
__global__ void __launch_bounds__(kCollThreads) all_reduce_rmsnorm_nvls_kernel(CollParams p, EpochCtl ectl, uint8_t* mc_base,
                                                                               const uint4* __restrict__ residual, const uint4* __restrict__ weight,
                                                                               int rows, int hidden, float eps, int64_t off_res_out, Status* status) {
  ptx::grid_dep_sync();
  __shared__ float scratch[33];
  const uint32_t epoch = tp::epoch_begin(ectl);
  const bool ok = arrive_and_wait(p, p.off_flags_a, epoch, blockIdx.x == 0, status);
  const int nvec = hidden >> 3;
  const int rows_per = (rows + p.tp - 1) / p.tp;
  const int row_lo = rows_per * p.rank, row_hi = min(rows, row_lo + rows_per);
  if (ok) {
    for (int row = row_lo + blockIdx.x; row < row_hi; row += gridDim.x) {
      const int64_t base = static_cast<int64_t>(row) * nvec;
      float v[VPT][8];
      float ss = 0.0f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + i * kCollThreads;
        if (c < nvec) {
          bf16x8_to_f32(ptx::multimem_ld_reduce_bf16x8(mc_base + p.off_buf + (base + c) * 16), v[i]);
          if (residual != nullptr) {
            float r[8];
            bf16x8_to_f32(residual[base + c], r);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[i][j] += r[j];
          }
          const uint4 packed = f32_to_bf16x8(v[i]);
          ptx::multimem_st_v4(mc_base + off_res_out + (base + c) * 16, packed);
          bf16x8_to_f32(packed, v[i]);                            // the stream is stored in bf16: normalise what is stored
#pragma unroll
          for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] = 0.0f;
        }
      }
      ss = block_sum(ss, scratch);
      const float rstd = ptx::rsqrt(ss / static_cast<float>(hidden) + eps);
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + i * kCollThreads;
        if (c < nvec) {
          float w[8];
          bf16x8_to_f32(weight[c], w);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] = v[i][j] * rstd * w[j];
          ptx::multimem_st_v4(mc_base + p.off_out + (base + c) * 16, f32_to_bf16x8(v[i]));
        }
      }
    }
  }
  publish_writes(p, epoch);
  arrive_and_wait(p, p.off_flags_b, epoch, false, status);
  tp::epoch_end(ectl, epoch);
}

__global__ void __launch_bounds__(kCollThreads) reduce_scatter_kernel(CollParams p, EpochCtl ectl, uint4* out, int64_t n_vec_per_rank,
                                                                      Status* status) {
  ptx::grid_dep_sync();
  const uint32_t epoch = tp::epoch_begin(ectl);
  const bool ok = arrive_and_wait(p, p.off_flags_a, epoch, blockIdx.x == 0, status);
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  if (ok)
    for (int64_t i = tid; i < n_vec_per_rank; i += nthreads) out[i] = sum_peers(p, (p.rank * n_vec_per_rank + i) * 16);
  tp::epoch_end(ectl, epoch);
}

__global__ void __launch_bounds__(kCollThreads) all_gather_kernel(CollParams p, EpochCtl ectl, const uint4* in, int64_t n_vec, Status* status) {
  ptx::grid_dep_sync();
  const uint32_t epoch = tp::epoch_begin(ectl);
  const bool ok = arrive_and_wait(p, p.off_flags_a, epoch, blockIdx.x == 0, status);
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  if (ok) {
    for (int64_t i = tid; i < n_vec; i += nthreads) {
      const uint4 v = in[i];
      for (int d = 0; d < p.tp; ++d) ptx::st_v4(p.peer[(p.rank + d) % p.tp] + p.off_out + (p.rank * n_vec + i) * 16, v);
    }
  }
  publish_writes(p, epoch);
  arrive_and_wait(p, p.off_flags_b, epoch, false, status);
  tp::epoch_end(ectl, epoch);
}

// Link probe: every rank whose bit is set in `senders` moves `n_vec` 16-byte vectors to (push: plain stores into the
// peer's result half, block [rank]) or from (pull: loads from the peer's input half into the local result half, block
// [peer]) each of the peers rank + 1 ... rank + n_peers (mod tp), eight vectors in flight per thread. Flags A before and
// B after, so the timed launch covers the delivery of every byte. This is how the NVLink figure used in the rooflines
// of the fused kernels is measured: with the library's own peer loads and stores, not with a driver copy.
__global__ void __launch_bounds__(kCollThreads) p2p_probe_kernel(CollParams p, EpochCtl ectl, int n_peers, uint32_t senders, int pull,
                                                                 int64_t n_vec, int64_t block_vec, Status* status) {
  ptx::grid_dep_sync();
  const uint32_t epoch = tp::epoch_begin(ectl);
  const bool ok = arrive_and_wait(p, p.off_flags_a, epoch, blockIdx.x == 0, status);
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  if (ok && ((senders >> p.rank) & 1u)) {
    constexpr int U = 8;
    for (int d = 1; d <= n_peers; ++d) {
      const int peer = (p.rank + d) % p.tp;
      const uint4* src = reinterpret_cast<const uint4*>((pull ? p.peer[peer] : p.peer[p.rank]) + p.off_buf);
      uint4* dst = reinterpret_cast<uint4*>((pull ? p.peer[p.rank] : p.peer[peer]) + p.off_out) + (pull ? peer : p.rank) * block_vec;
      for (int64_t i0 = tid; i0 < n_vec; i0 += nthreads * U) {
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int64_t i = i0 + u * nthreads;
          if (i < n_vec) v[u] = pull ? ptx::ld_relaxed_sys_v4(src + i) : src[i];
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int64_t i = i0 + u * nthreads;
          if (i < n_vec) ptx::st_v4(dst + i, v[u]);
        }
      }
    }
  }
  publish_writes(p, epoch);
  arrive_and_wait(p, p.off_flags_b, epoch, false, status);
  tp::epoch_end(ectl, epoch);
}

struct A2ACounts {
  int n[tp::kMaxTp];
};

__global__ void __launch_bounds__(kCollThreads) all_to_all_kernel(CollParams p, EpochCtl ectl, const uint4* in, A2ACounts counts, int max_rows,
                                                                  int64_t row_vec, int parity, Status* status) {
  ptx::grid_dep_sync();
  const uint32_t epoch = tp::epoch_begin(ectl);
  const bool ok = arrive_and_wait(p, p.off_flags_a, epoch, blockIdx.x == 0, status);
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  if (ok) {
    const int64_t block_vec = static_cast<int64_t>(max_rows) * row_vec;
    for (int d = 0; d < p.tp; ++d) {
      const int dst = (p.rank + d) % p.tp;
      const int64_t n = static_cast<int64_t>(counts.n[dst]) * row_vec;
      uint8_t* base = p.peer[dst] + p.off_out + p.rank * block_vec * 16;
      for (int64_t i = tid; i < n; i += nthreads) ptx::st_v4(base + i * 16, in[dst * block_vec + i]);
    }
    if (blockIdx.x == 0 && threadIdx.x < p.tp)
      ptx::st_relaxed_sys(reinterpret_cast<uint32_t*>(p.peer[threadIdx.x] + p.off_counts) + parity * tp::kMaxTp + p.rank,
                          static_cast<uint32_t>(counts.n[threadIdx.x]));
  }
  publish_writes(p, epoch);
  arrive_and_wait(p, p.off_flags_b, epoch, false, status);
  tp::epoch_end(ectl, epoch);
}

// Monotone map from float to unsigned: a > b  <=>  key(a) > key(b).
__device__ __forceinline__ uint32_t orderable(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__global__ void __launch_bounds__(kCollThreads) vocab_argmax_kernel(CollParams p, EpochCtl ectl, const __nv_bfloat16* logits, int64_t ld,
                                                                    const int64_t* local_idx, int64_t* tokens, int S, int v_local, int v_stride, Status* status) {
  ptx::grid_dep_sync();
  const uint32_t epoch = tp::epoch_begin(ectl);
  const bool ok = arrive_and_wait(p, p.off_flags_a, epoch, true, status);
  if (ok) {
    for (int s = threadIdx.x; s < S; s += blockDim.x) {
      int idx = static_cast<int>(local_idx[s]);
      idx = idx < 0 ? 0 : idx >= v_local ? v_local - 1 : idx;
      const float v = __bfloat162float(logits[static_cast<int64_t>(s) * ld + idx]);
      const uint32_t gidx = static_cast<uint32_t>(p.rank) * static_cast<uint32_t>(v_stride) + static_cast<uint32_t>(idx);
      const unsigned long long key = (static_cast<unsigned long long>(orderable(v)) << 32) | (0xFFFFFFFFu - gidx);
      for (int d = 0; d < p.tp; ++d) {
        unsigned long long* dst = reinterpret_cast<unsigned long long*>(p.peer[(p.rank + d) % p.tp] + p.off_out) + static_cast<int64_t>(p.rank) * S + s;
        ptx::st_relaxed_sys_u64(dst, key);
      }
    }
  }
  publish_writes(p, epoch);
  const bool ok2 = arrive_and_wait(p, p.off_flags_b, epoch, false, status);
  if (ok && ok2) {
    const unsigned long long* keys = reinterpret_cast<const unsigned long long*>(p.peer[p.rank] + p.off_out);
    for (int s = threadIdx.x; s < S; s += blockDim.x) {
      unsigned long long best = 0;
      for (int r = 0; r < p.tp; ++r) {
        const unsigned long long k = ptx::ld_relaxed_sys_u64(keys + static_cast<int64_t>(r) * S + s);
        best = k > best ? k : best;
      }
      tokens[s] = static_cast<int64_t>(0xFFFFFFFFu - static_cast<uint32_t>(best & 0xFFFFFFFFull));
    }
  }
  tp::epoch_end(ectl, epoch);
}

bool fill(CollParams& p, EpochCtl& ectl, const B2TpRegion* reg, const B2CollLayout* lay, int slot, uint64_t timeout_ns) {
  if (reg == nullptr || lay == nullptr || reg->tp < 1 || reg->tp > tp::kMaxTp) return false;
  p.rank = reg->rank;
  p.tp = reg->tp;
  for (int i = 0; i < reg->tp; ++i) p.peer[i] = static_cast<uint8_t*>(reg->peer[i]);
  const int parity = slot & 1;
  p.off_buf = lay->off_buf + parity * lay->buf_half_bytes;
  p.off_out = lay->off_out + parity * lay->out_half_bytes;
  p.off_flags_a = lay->off_flags_a;
  p.off_flags_b = lay->off_flags_b;
  p.off_counts = lay->off_counts;
  p.off_done = lay->off_done;
  p.timeout_ns = timeout_ns;
  ectl.epoch_ptr = reinterpret_cast<uint32_t*>(p.peer[p.rank] + lay->off_epoch);
  ectl.cta_done = ectl.epoch_ptr + 1;
  return true;
}

int grid_for(int64_t n_vec) {
  int64_t g = (n_vec + kCollThreads * 4 - 1) / (kCollThreads * 4);
  if (g < 1) g = 1;
  return static_cast<int>(g > kNumSMs ? kNumSMs : g);
}

int launched() { return last_launch_rc(); }

}  // namespace
}  // namespace b2

using namespace b2;

extern "C" int b2_coll_all_reduce_bf16(const B2TpRegion* reg, const B2CollLayout* lay, void* mc_base, void* out, int64_t n, int algo,
                                       int slot, uint64_t timeout_ns, Status* status, cudaStream_t stream) {
  CollParams p{};
  EpochCtl ectl{};
  if (!fill(p, ectl, reg, lay, slot, timeout_ns) || n <= 0 || n % 8 != 0 || algo < 0 || algo > 2) return -kBadArgument;
  if (n * 2 > lay->buf_half_bytes || (algo != 0 && n * 2 > lay->out_half_bytes)) return -kTooLarge;
  if ((algo == 0 && out == nullptr) || (algo == 2 && mc_base == nullptr)) return -kBadArgument;
  const int64_t n_vec = n / 8;
  const int grid = grid_for(algo == 0 ? n_vec : (n_vec + p.tp - 1) / p.tp);
  if (algo == 0) launch_pdl(all_reduce_kernel<0>, dim3(grid), dim3(kCollThreads), 0, stream, p, ectl, nullptr, static_cast<uint4*>(out), n_vec, status);
  else if (algo == 1) launch_pdl(all_reduce_kernel<1>, dim3(grid), dim3(kCollThreads), 0, stream, p, ectl, nullptr, nullptr, n_vec, status);
  else launch_pdl(all_reduce_kernel<2>, dim3(grid), dim3(kCollThreads), 0, stream, p, ectl, static_cast<uint8_t*>(mc_base), nullptr, n_vec, status);
  return launched();
}

extern "C" int b2_coll_all_reduce_rmsnorm_bf16(const B2TpRegion* reg, const B2CollLayout* lay, void* residual, const void* weight,
                                               void* out, int rows, int hidden, float eps, int slot, uint64_t timeout_ns,
                                               Status* status, cudaStream_t stream) {
  CollParams p{};
  EpochCtl ectl{};
  if (!fill(p, ectl, reg, lay, slot, timeout_ns) || rows <= 0 || hidden <= 0 || hidden % 8 != 0 || hidden > 8 * kCollThreads * 8 ||
      weight == nullptr || out == nullptr)
    return -kBadArgument;
  if (static_cast<int64_t>(rows) * hidden * 2 > lay->buf_half_bytes) return -kTooLarge;
  const int nvec = hidden / 8;
  const int vpt = (nvec + kCollThreads - 1) / kCollThreads;
  const int grid = rows < 4 * kNumSMs ? rows : 4 * kNumSMs;
  uint4* res = static_cast<uint4*>(residual);
  const uint4* w = static_cast<const uint4*>(weight);
  uint4* o = static_cast<uint4*>(out);
  if (vpt <= 1) launch_pdl(all_reduce_rmsnorm_kernel<1>, dim3(grid), dim3(kCollThreads), 0, stream, p, ectl, res, w, o, rows, hidden, eps, status);
  else if (vpt <= 2) launch_pdl(all_reduce_rmsnorm_kernel<2>, dim3(grid), dim3(kCollThreads), 0, stream, p, ectl, res, w, o, rows, hidden, eps, status);
  else if (vpt <= 4) launch_pdl(all_reduce_rmsnorm_kernel<4>, dim3(grid), dim3(kCollThreads), 0, stream, p, ectl, res, w, o, rows, hidden, eps, status);
  else launch_pdl(all_reduce_rmsnorm_kernel<8>, dim3(grid), dim3(kCollThreads), 0, stream, p, ectl, res, w, o, rows, hidden, eps, status);
  return launched();
}

extern "C" int b2_coll_all_reduce_rmsnorm_nvls_bf16(const B2TpRegion* reg, const B2CollLayout* lay, void* mc_base, const void* residual,
                                                    const void* weight, int rows, int hidden, float eps, int slot, uint64_t timeout_ns,
                                                    Status* status, cudaStream_t stream) {
  CollParams p{};
  EpochCtl ectl{};
  if (!fill(p, ectl, reg, lay, slot, timeout_ns) || rows <= 0 || hidden <= 0 || hidden % 8 != 0 || hidden > 8 * kCollThreads * 8 ||
      weight == nullptr || mc_base == nullptr)
    return -kBadArgument;
  const int64_t bytes = static_cast<int64_t>(rows) * hidden * 2;
  if (bytes > lay->buf_half_bytes || 2 * bytes > lay->out_half_bytes) return -kTooLarge;
  const int nvec = hidden / 8;
  const int vpt = (nvec + kCollThreads - 1) / kCollThreads;
  const int rows_per = (rows + p.tp - 1) / p.tp;
  const int grid = rows_per < 2 * kNumSMs ? rows_per : 2 * kNumSMs;
  const uint4* res = static_cast<const uint4*>(residual);
  const uint4* w = static_cast<const uint4*>(weight);
  uint8_t* mc = static_cast<uint8_t*>(mc_base);
  const int64_t off_res = p.off_out + bytes;
#define B2_NVLS_NORM(V) launch_pdl(all_reduce_rmsnorm_nvls_kernel<V>, dim3(grid), dim3(kCollThreads), 0, stream, p, ectl, mc, res, w, rows, hidden, eps, off_res, status)
  if (vpt <= 1) B2_NVLS_NORM(1);
  else if (vpt <= 2) B2_NVLS_NORM(2);
  else if (vpt <= 4) B2_NVLS_NORM(4);
  else B2_NVLS_NORM(8);
#undef B2_NVLS_NORM
  return launched();
}

extern "C" int b2_coll_reduce_scatter_bf16(const B2TpRegion* reg, const B2CollLayout* lay, void* out, int64_t n, int slot,
                                           uint64_t timeout_ns, Status* status, cudaStream_t stream) {
  CollParams p{};
  EpochCtl ectl{};
  if (!fill(p, ectl, reg, lay, slot, timeout_ns) || n <= 0 || out == nullptr || n % (8 * reg->tp) != 0) return -kBadArgument;
  if (n * 2 > lay->buf_half_bytes) return -kTooLarge;
  const int64_t per = n / 8 / p.tp;
  launch_pdl(reduce_scatter_kernel, dim3(grid_for(per)), dim3(kCollThreads), 0, stream, p, ectl, static_cast<uint4*>(out), per, status);
  return launched();
}

extern "C" int b2_coll_all_gather(const B2TpRegion* reg, const B2CollLayout* lay, const void* in, int64_t bytes, int slot,
                                  uint64_t timeout_ns, Status* status, cudaStream_t stream) {
  CollParams p{};
  EpochCtl ectl{};
  if (!fill(p, ectl, reg, lay, slot, timeout_ns) || bytes <= 0 || bytes % 16 != 0 || in == nullptr ||
      (reinterpret_cast<uintptr_t>(in) & 15) != 0)
    return -kBadArgument;
  if (bytes * p.tp > lay->out_half_bytes) return -kTooLarge;
  launch_pdl(all_gather_kernel, dim3(grid_for(bytes / 16)), dim3(kCollThreads), 0, stream, p, ectl, static_cast<const uint4*>(in), bytes / 16, status);
  return launched();
}

extern "C" int b2_coll_all_to_all(const B2TpRegion* reg, const B2CollLayout* lay, const void* in, const int* send_counts, int max_rows,
                                  int64_t row_bytes, int slot, uint64_t timeout_ns, Status* status, cudaStream_t stream) {
  CollParams p{};
  EpochCtl ectl{};
  if (!fill(p, ectl, reg, lay, slot, timeout_ns) || in == nullptr || send_counts == nullptr || max_rows <= 0 || row_bytes <= 0 ||
      row_bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(in) & 15) != 0)
    return -kBadArgument;
  if (static_cast<int64_t>(p.tp) * max_rows * row_bytes > lay->out_half_bytes) return -kTooLarge;
  A2ACounts c{};
  int64_t most = 0;
  for (int i = 0; i < p.tp; ++i) {
    if (send_counts[i] < 0 || send_counts[i] > max_rows) return -kBadArgument;
    c.n[i] = send_counts[i];
    most = send_counts[i] > most ? send_counts[i] : most;
  }
  launch_pdl(all_to_all_kernel, dim3(grid_for(most * (row_bytes / 16))), dim3(kCollThreads), 0, stream, p, ectl, static_cast<const uint4*>(in), c, max_rows,
                                                                                   row_bytes / 16, slot & 1, status);
  return launched();
}

extern "C" int b2_coll_vocab_argmax(const B2TpRegion* reg, const B2CollLayout* lay, const void* logits, int64_t ld, const int64_t* local_idx,
                                    int64_t* tokens, int S, int v_local, int v_stride, int slot, uint64_t timeout_ns,
                                    Status* status, cudaStream_t stream) {
  CollParams p{};
  EpochCtl ectl{};
  if (S <= 0) return 0;
  if (!fill(p, ectl, reg, lay, slot, timeout_ns) || logits == nullptr || local_idx == nullptr || tokens == nullptr || v_local <= 0 || v_stride < v_local)
    return -kBadArgument;
  if (static_cast<int64_t>(S) * p.tp * 8 > lay->out_half_bytes) return -kTooLarge;
  launch_pdl(vocab_argmax_kernel, dim3(1), dim3(kCollThreads), 0, stream, p, ectl, static_cast<const __nv_bfloat16*>(logits), ld, local_idx, tokens, S, v_local,
                                                      v_stride, status);
  return launched();
}

extern "C" int b2_coll_p2p_probe(const B2TpRegion* reg, const B2CollLayout* lay, int64_t bytes, int n_peers, uint32_t senders, int pull,
                                 int ctas, int slot, uint64_t timeout_ns, Status* status, cudaStream_t stream) {
  CollParams p{};
  EpochCtl ectl{};
  if (!fill(p, ectl, reg, lay, slot, timeout_ns) || bytes <= 0 || bytes % 16 != 0 || n_peers < 1 || n_peers >= p.tp || ctas < 1 || ctas > 8 * kNumSMs)
    return -kBadArgument;
  if (bytes > lay->buf_half_bytes || bytes * p.tp > lay->out_half_bytes) return -kTooLarge;
  launch_pdl(p2p_probe_kernel, dim3(ctas), dim3(kCollThreads), 0, stream, p, ectl, n_peers, senders, pull ? 1 : 0, bytes / 16, bytes / 16, status);
  return launched();
}
