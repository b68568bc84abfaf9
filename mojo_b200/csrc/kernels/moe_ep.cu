// Mixture-of-experts with expert parallelism: dispatch, grouped expert GEMM, combine.
//
//   ep_dispatch   per token: softmax over the router logits, top-k, and for every selected expert a copy of the
//                 token's activation row straight into the owning rank's receive buffer (slot claimed with a
//                 system-scope atomic on that rank's per-expert counter, rows packed densely per expert).
//                 The last CTA raises this rank's "dispatched" flag on every peer and waits (bounded) for theirs,
//                 so when the kernel ends the receive buffer and counts are final.
//   grouped GEMM  the tcgen05 core over work units (local expert, token tile, weight-row tile); weights are
//                 the UMMA M side (128 rows), tokens the N side, counts come from device memory.
//                 Epilogues: SwiGLU on 16-row-interleaved gate/up weights, or plain store.
//   ep_combine    every expert-output row goes back to the rank and (token, k) slot it came from; after a
//                 bounded wait for all ranks, each token's k rows are summed with the router weights (+ the
//                 shared-expert output).
// All cross-GPU traffic is peer stores / atomics / flags from inside these kernels. With one rank the same
// kernels run against the local buffer.
#include <cstdint>
#include <cuda.h>
#include <cuda_bf16.h>
#include "b2/api.h"
#include "b2/launch.h"
#include "b2/ep.h"
#include "b2/gemm_tc.cuh"
#include "b2/ptx.cuh"
#include "b2/tma.h"
#include "b2/vec.cuh"

namespace b2 {
namespace {

constexpr int kMaxRanks = 8;

struct EpDev {
  int rank, n_ranks;
  uint8_t* peer[kMaxRanks];
  B2EpLayout lay;
  uint64_t timeout_ns;
};

__device__ __forceinline__ uint32_t epoch_begin(uint32_t* p) { return *reinterpret_cast<volatile uint32_t*>(p) + 1u; }
__device__ __forceinline__ bool last_cta(uint32_t* counter) {
  __shared__ uint32_t sh_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const uint32_t old = atomicAdd(counter, 1u);
    sh_last = (old == gridDim.x - 1) ? 1u : 0u;
    if (sh_last) *counter = 0;
  }
  __syncthreads();
  return sh_last != 0;
}

// ------------------------------------------------------------------------------------------------
// dispatch
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) ep_dispatch_kernel(
    EpDev d, const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ logits, float* __restrict__ w_out,
    int32_t* __restrict__ id_out, int T, int E, int top_k, int norm_topk, float route_scale, int slot, Status* status) {
  uint8_t* self = d.peer[d.rank];
  uint32_t* ectl = reinterpret_cast<uint32_t*>(self + d.lay.off_epoch);
  const uint32_t epoch = epoch_begin(ectl);
  const int e_local = d.lay.e_local, cap = d.lay.cap, H = d.lay.hidden;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int n_warps = (gridDim.x * blockDim.x) >> 5;
  // the counters of the other parity belong to the next launch: clear them now (see header comment of ep.h)
  if (blockIdx.x == 0 && threadIdx.x < e_local)
    reinterpret_cast<uint32_t*>(self + d.lay.off_recv_count)[(slot ^ 1) * e_local + threadIdx.x] = 0;

  for (int t = warp; t < T; t += n_warps) {
    // ---- router: softmax over E experts, top-k (lowest index wins ties) ----
    float v[8];  // E <= 256
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = lane + 32 * i;
      v[i] = e < E ? __bfloat162float(logits[static_cast<int64_t>(t) * E + e]) : -INFINITY;
      mx = fmaxf(mx, v[i]);
    }
    mx = warp_max(mx);
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      v[i] = (lane + 32 * i) < E ? ptx::ex2((v[i] - mx) * ptx::kLog2e) : -1.0f;
      if (v[i] > 0.0f) sum += v[i];
    }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    float sel_w = 0.0f;   // lane kk keeps the kk-th selection
    int sel_e = 0;
    float wsum = 0.0f;
    for (int kk = 0; kk < top_k; ++kk) {
      float best = -2.0f;
      int best_e = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (v[i] > best) { best = v[i]; best_e = lane + 32 * i; }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
        if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
      }
      if ((best_e & 31) == lane) v[best_e >> 5] = -1.0f;  // remove from the pool
      if (lane == kk) { sel_w = best * inv; sel_e = best_e; }
      wsum += best * inv;
    }
    if (norm_topk) sel_w /= wsum;
    sel_w *= route_scale;
    if (lane < top_k) {
      w_out[static_cast<int64_t>(t) * top_k + lane] = sel_w;
      id_out[static_cast<int64_t>(t) * top_k + lane] = sel_e;
    }
    // ---- permute + all-to-all: one row copy per selected expert ----
    // Lane kk claims the slot of the kk-th selection, so the top_k system-scope atomics (a link round trip each when the
    // expert lives on a peer) are in flight together instead of one after the other.
    uint32_t my_pos = 0;
    if (lane < top_k) {
      const int dst = sel_e / e_local, el = sel_e - dst * e_local;
      uint8_t* base = d.peer[dst];
      my_pos = ptx::atom_add_acqrel_sys(reinterpret_cast<uint32_t*>(base + d.lay.off_recv_count) + slot * e_local + el, 1u);
      if (my_pos >= static_cast<uint32_t>(cap))
        status_record(status, kTooLarge, kSiteEpCount, sel_e, my_pos);
      else
        reinterpret_cast<int32_t*>(base + d.lay.off_recv_meta)[static_cast<int64_t>(el) * cap + my_pos] = (d.rank << 24) | (t * top_k + lane);
    }
    // The token's row is read once (four 16-byte vectors per lane at a time) and stored to every destination.
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<int64_t>(t) * H);
    const int hv = H >> 3;
    for (int c0 = 0; c0 < hv; c0 += 128) {   // warp-uniform trip count: the shuffles below need every lane
      uint4 row[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (c0 + u * 32 + lane < hv) row[u] = ptx::ld_nc_v4(src + c0 + u * 32 + lane);
      for (int kk = 0; kk < top_k; ++kk) {
        const int e = __shfl_sync(0xffffffffu, sel_e, kk);
        const uint32_t pos = __shfl_sync(0xffffffffu, my_pos, kk);
        if (pos >= static_cast<uint32_t>(cap)) continue;   // recorded above; the row is dropped
        const int dst = e / e_local, el = e - dst * e_local;
        uint4* dstp = reinterpret_cast<uint4*>(d.peer[dst] + d.lay.off_recv_x) + (static_cast<int64_t>(el) * cap + pos) * hv;
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (c0 + u * 32 + lane < hv) dstp[c0 + u * 32 + lane] = row[u];
      }
    }
  }
  // ---- all rows of this rank are on their way: tell every destination, then wait for every source ----
  if (last_cta(ectl + 1)) {
    if (threadIdx.x < d.n_ranks) {
      ptx::st_release_sys(reinterpret_cast<uint32_t*>(d.peer[threadIdx.x] + d.lay.off_disp_done) + d.rank, epoch);
      if (!ptx::wait_flag_ge_sys(reinterpret_cast<const uint32_t*>(self + d.lay.off_disp_done) + threadIdx.x, epoch, d.timeout_ns))
        status_record(status, kTimeout, kSiteEpCount, threadIdx.x, epoch);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      *reinterpret_cast<volatile uint32_t*>(ectl) = epoch;
      __threadfence();
    }
  }
}

// ------------------------------------------------------------------------------------------------
// grouped GEMM (weights on the UMMA M side, tokens on the N side)
// ------------------------------------------------------------------------------------------------
constexpr int kMaxLocalExperts = 64;

struct GroupedSched {
  const uint32_t* counts;  // [e_local] tokens per local expert (device memory, final before launch)
  int e_local, cap, n_rows;  // n_rows = output rows of one expert's weight (N)
  int num_kb, bn;
  int p_blocks;            // n_rows / 128
  int prefix[kMaxLocalExperts + 1];  // filled by init(): work-unit prefix sums
  __device__ __forceinline__ void init() {
    int acc = 0;
    for (int e = 0; e < e_local; ++e) {
      prefix[e] = acc;
      const int c = min(static_cast<int>(counts[e]), cap);
      acc += ((c + bn - 1) / bn) * p_blocks;
    }
    prefix[e_local] = acc;
  }
  __device__ __forceinline__ int total() const { return prefix[e_local]; }
  __device__ __forceinline__ gemm::WorkUnit get(int w) const {
    int e = 0;
    while (e + 1 < e_local && w >= prefix[e + 1]) ++e;
    const int r = w - prefix[e];
    gemm::WorkUnit u;
    // Consecutive units share the token tile. The other order (consecutive units share the weight tile) was measured on
    // one DeepSeek-V2-Lite layer of 4096 tokens and lost: 951 us against 891 us for the whole layer.
    u.pb = r % p_blocks;          // weight-row tile
    u.qb = r / p_blocks;          // token tile inside the expert
    u.split = e;                  // carries the expert index to the epilogue
    u.tile = w;
    u.kb0 = 0;
    u.kb1 = num_kb;
    u.p_coord = e * n_rows + u.pb * 128;
    u.q_coord = e * cap + u.qb * bn;
    return u;
  }
};

struct GroupedEpiParams {
  __nv_bfloat16* y;       // [e_local][cap][ldy]
  int64_t ldy;
  const uint32_t* counts;
  int cap, n_rows;
  int swiglu;
};

template <int BN>
struct GroupedEpilogue {
  static constexpr int CH = BN >= 32 ? 32 : 16;
  GroupedEpiParams p;
  __device__ __forceinline__ void operator()(const gemm::WorkUnit& u, uint32_t taddr, int quarter, int lane, uint32_t*,
                                             Status*) const {
    const int e = u.split;
    const int cnt = min(static_cast<int>(p.counts[e]), p.cap);
    const int p_local = quarter * 32 + lane;
    const int n = u.pb * 128 + p_local;
    __nv_bfloat16* base = p.y + static_cast<int64_t>(e) * p.cap * p.ldy;
#pragma unroll 1
    for (int c = 0; c < BN / CH; ++c) {
      uint32_t r[CH];
      if constexpr (CH == 32) ptx::tmem_ld_32x32(taddr + c * CH, r);
      else ptx::tmem_ld_32x16(taddr + c * CH, r);
      ptx::tc_wait_ld();
      const int m0 = u.qb * BN + c * CH;
      if (p.swiglu) {
        const int out_col = (u.pb * 128 + (p_local & ~31)) / 2 + (lane & 15);
#pragma unroll
        for (int j = 0; j < CH; ++j) {
          const float v = __uint_as_float(r[j]);
          const float other = __shfl_xor_sync(0xffffffffu, v, 16);
          if (lane < 16 && n < p.n_rows && m0 + j < cnt)
            base[static_cast<int64_t>(m0 + j) * p.ldy + out_col] = __float2bfloat16(ptx::silu(v) * other);
        }
      } else if (n < p.n_rows) {
#pragma unroll
        for (int j = 0; j < CH; ++j) {
          if (m0 + j >= cnt) break;
          base[static_cast<int64_t>(m0 + j) * p.ldy + n] = __float2bfloat16(__uint_as_float(r[j]));
        }
      }
    }
  }
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(gemm::kThreads, 1)
moe_grouped_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, GroupedSched sched_in,
                   GroupedEpiParams ep, Status* status) {
  constexpr uint32_t idesc = ptx::make_idesc(1, 1, 128, BN);
  GroupedSched sched = sched_in;
  sched.init();
  GroupedEpilogue<BN> epi{ep};
  gemm::run<BN, STAGES, 2>(&tmap_w, &tmap_x, idesc, ptx::kEvictFirst, ptx::kEvictLast, sched, gemm::NoGate{}, epi, status,
                           static_cast<int>(blockIdx.x), static_cast<int>(gridDim.x));
}

constexpr int stages_for(int bn) {
  const int stage = 128 * 64 * 2 + bn * 64 * 2;
  int s = (200 * 1024) / stage;
  return s > 10 ? 10 : s;
}

template <int BN>
int launch_grouped(const void* x, const void* w, const uint32_t* counts, void* y, int e_local, int cap, int N, int K,
                   int64_t ldy, int swiglu, Status* status, cudaStream_t stream) {
  constexpr int STAGES = stages_for(BN);
  using L = gemm::SmemLayout<BN, STAGES>;
  CUtensorMap tw, tx;
  if (!make_tmap_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w, static_cast<uint64_t>(e_local) * N, K, static_cast<uint64_t>(K) * 2, 128, 64,
                    CU_TENSOR_MAP_SWIZZLE_128B) ||
      !make_tmap_2d(&tx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, static_cast<uint64_t>(e_local) * cap, K, static_cast<uint64_t>(K) * 2, BN, 64,
                    CU_TENSOR_MAP_SWIZZLE_128B))
    return -kBadArgument;
  GroupedSched sched{};
  sched.counts = counts;
  sched.e_local = e_local;
  sched.cap = cap;
  sched.n_rows = N;
  sched.num_kb = (K + 63) / 64;
  sched.bn = BN;
  sched.p_blocks = (N + 127) / 128;
  GroupedEpiParams ep{static_cast<__nv_bfloat16*>(y), ldy, counts, cap, N, swiglu};
  auto kern = moe_grouped_kernel<BN, STAGES>;
  static DeviceOnce attr_once;
  if (const int rc = attr_once.run([&] {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotalBytes);
        return e;
      }))
    return rc;
  kern<<<kNumSMs, gemm::kThreads, L::kTotalBytes, stream>>>(tw, tx, sched, ep, status);
  return last_launch_rc();
}

// ------------------------------------------------------------------------------------------------
// combine
// ------------------------------------------------------------------------------------------------
constexpr int kCombineThreads = 512;   // one CTA per SM (its waits need the whole grid resident): sixteen warps of loads in flight
__global__ void __launch_bounds__(kCombineThreads) ep_combine_kernel(EpDev d, const __nv_bfloat16* __restrict__ y_local,
                                                         const float* __restrict__ weights, const __nv_bfloat16* __restrict__ shared,
                                                         __nv_bfloat16* __restrict__ out, int T, int top_k, int slot, Status* status) {
  __shared__ uint32_t sh_ok;
  uint8_t* self = d.peer[d.rank];
  uint32_t* ectl = reinterpret_cast<uint32_t*>(self + d.lay.off_epoch) + 2;
  const uint32_t epoch = epoch_begin(ectl);
  const int e_local = d.lay.e_local, cap = d.lay.cap, H = d.lay.hidden, hv = H >> 3;
  const uint32_t* counts = reinterpret_cast<const uint32_t*>(self + d.lay.off_recv_count) + slot * e_local;
  const int32_t* meta = reinterpret_cast<const int32_t*>(self + d.lay.off_recv_meta);
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int n_warps = (gridDim.x * blockDim.x) >> 5;
  // ---- phase A: return every expert-output row to its source ----
  for (int el = 0; el < e_local; ++el) {
    const int cnt = min(static_cast<int>(counts[el]), cap);
    for (int r = warp; r < cnt; r += n_warps) {
      const int mt = meta[static_cast<int64_t>(el) * cap + r];
      const int src = (mt >> 24) & 0xff, idx = mt & 0xffffff;
      const uint4* from = reinterpret_cast<const uint4*>(y_local) + (static_cast<int64_t>(el) * cap + r) * hv;
      uint4* to = reinterpret_cast<uint4*>(d.peer[src] + d.lay.off_ret_y) + static_cast<int64_t>(idx) * hv;
      // four 16-byte vectors in flight per lane: the copy is bound by round trips, not by bytes
      for (int c0 = lane; c0 < hv; c0 += 128) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (c0 + u * 32 < hv) v[u] = ptx::ld_nc_v4(from + c0 + u * 32);
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (c0 + u * 32 < hv) to[c0 + u * 32] = v[u];
      }
    }
  }
  if (last_cta(ectl + 1)) {
    if (threadIdx.x < d.n_ranks)
      ptx::st_release_sys(reinterpret_cast<uint32_t*>(d.peer[threadIdx.x] + d.lay.off_comb_done) + d.rank, epoch);
  }
  // ---- phase B: wait for every rank's rows, then the weighted sum per token ----
  if (threadIdx.x == 0) sh_ok = 1;
  __syncthreads();
  if (threadIdx.x < d.n_ranks) {
    if (!ptx::wait_flag_ge_sys(reinterpret_cast<const uint32_t*>(self + d.lay.off_comb_done) + threadIdx.x, epoch, d.timeout_ns)) {
      status_record(status, kTimeout, kSiteEpCount, 100 + threadIdx.x, epoch);
      sh_ok = 0;
    }
  }
  __syncthreads();
  if (sh_ok != 0) {
    const uint4* ret = reinterpret_cast<const uint4*>(self + d.lay.off_ret_y);
    for (int t = warp; t < T; t += n_warps) {
      for (int c = lane; c < hv; c += 32) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (shared != nullptr) bf16x8_to_f32(reinterpret_cast<const uint4*>(shared)[static_cast<int64_t>(t) * hv + c], acc);
        // the returned rows of up to four experts are requested before the first is used
        for (int k0 = 0; k0 < top_k; k0 += 4) {
          uint4 raw[4];
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (k0 + u < top_k) raw[u] = ptx::ld_relaxed_sys_v4(ret + (static_cast<int64_t>(t) * top_k + k0 + u) * hv + c);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            if (k0 + u < top_k) {
              float v[8];
              bf16x8_to_f32(raw[u], v);
              const float w = weights[static_cast<int64_t>(t) * top_k + k0 + u];
#pragma unroll
              for (int j = 0; j < 8; ++j) acc[j] = fmaf(w, v[j], acc[j]);
            }
          }
        }
        reinterpret_cast<uint4*>(out)[static_cast<int64_t>(t) * hv + c] = f32_to_bf16x8(acc);
      }
    }
  }
  // the CTA that finishes phase B last publishes the new epoch (own counter word, separate from phase A's)
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    uint32_t* fin = ectl + 2;
    if (atomicAdd(fin, 1u) == gridDim.x - 1) {
      *fin = 0;
      *reinterpret_cast<volatile uint32_t*>(ectl) = epoch;
      __threadfence();
    }
  }
}

EpDev make_dev(const B2TpRegion* reg, const B2EpLayout* lay, uint64_t timeout_ns) {
  EpDev d{};
  d.rank = reg->rank;
  d.n_ranks = reg->tp;
  for (int i = 0; i < reg->tp; ++i) d.peer[i] = static_cast<uint8_t*>(reg->peer[i]);
  d.lay = *lay;
  d.timeout_ns = timeout_ns;
  return d;
}

}  // namespace
}  // namespace b2

using namespace b2;

extern "C" int b2_ep_dispatch(const void* x, const void* logits, float* weights_out, int32_t* ids_out, const B2TpRegion* reg,
                              const B2EpLayout* lay, int T, int E, int top_k, int norm_topk, float route_scale, int slot,
                              uint64_t timeout_ns, b2::Status* status, cudaStream_t stream) {
  if (reg == nullptr || lay == nullptr || reg->tp < 1 || reg->tp > kMaxRanks || E > 256 || E != lay->e_local * reg->tp || top_k < 1 ||
      top_k > 32 || lay->hidden % 8 != 0 || T < 0 || T > lay->t_cap || lay->e_local > kMaxLocalExperts || T * top_k >= (1 << 24))
    return -kBadArgument;
  const EpDev d = make_dev(reg, lay, timeout_ns);
  int blocks = (T + 7) / 8;
  if (blocks < 1) blocks = 1;
  if (blocks > 2 * kNumSMs) blocks = 2 * kNumSMs;
  ep_dispatch_kernel<<<blocks, 256, 0, stream>>>(d, static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(logits),
                                                 weights_out, ids_out, T, E, top_k, norm_topk, route_scale, slot & 1, status);
  return last_launch_rc();
}

extern "C" int b2_moe_grouped_gemm(const void* x, const void* w, const uint32_t* counts, void* y, int e_local, int cap, int N,
                                   int K, int64_t ldy, int swiglu, int bn, b2::Status* status, cudaStream_t stream) {
  if (e_local < 1 || e_local > kMaxLocalExperts || cap < 1 || K % 8 != 0 || N % 8 != 0 || (swiglu && N % 32 != 0)) return -kBadArgument;
  switch (bn) {
    case 16: return launch_grouped<16>(x, w, counts, y, e_local, cap, N, K, ldy, swiglu, status, stream);
    case 32: return launch_grouped<32>(x, w, counts, y, e_local, cap, N, K, ldy, swiglu, status, stream);
    case 64: return launch_grouped<64>(x, w, counts, y, e_local, cap, N, K, ldy, swiglu, status, stream);
    case 128: return launch_grouped<128>(x, w, counts, y, e_local, cap, N, K, ldy, swiglu, status, stream);
    case 256: return launch_grouped<256>(x, w, counts, y, e_local, cap, N, K, ldy, swiglu, status, stream);
    default: return -kBadArgument;
  }
}

extern "C" int b2_ep_combine(const void* y_local, const float* weights, const void* shared, void* out, const B2TpRegion* reg,
                             const B2EpLayout* lay, int T, int top_k, int slot, uint64_t timeout_ns, b2::Status* status,
                             cudaStream_t stream) {
  if (reg == nullptr || lay == nullptr || reg->tp < 1 || reg->tp > kMaxRanks || T < 0 || T > lay->t_cap) return -kBadArgument;
  const EpDev d = make_dev(reg, lay, timeout_ns);
  ep_combine_kernel<<<kNumSMs, kCombineThreads, 0, stream>>>(d, static_cast<const __nv_bfloat16*>(y_local), weights,
                                                 static_cast<const __nv_bfloat16*>(shared), static_cast<__nv_bfloat16*>(out), T, top_k,
                                                 slot & 1, status);
  return last_launch_rc();
}
