// bf16 GEMM on tcgen05/TMEM: Y[M, N] = X[M, K] * W[N, K]^T, f32 accumulate, bf16 out.
//
// Two operand assignments of the same core (b2/gemm_tc.cuh):
//   normal  P = X, Q = W   D[m, n]: each epilogue thread owns one output row and writes 64-byte row segments.
//                          Used for prefill-sized M.
//   swapped P = W, Q = X   D[n, m]: the 128-row UMMA M dimension is filled by weight rows, the token count
//                          becomes the UMMA N (16..256). Every byte staged in shared memory is weight data, so
//                          decode-sized M streams the weights once at HBM rate; K can be split across CTAs
//                          (f32 partials in a workspace, last CTA of a tile reduces) to fill all 148 SMs.
// Epilogues: plain store, + residual, SwiGLU on 16-row-interleaved gate/up weights.
#include <cstdint>
#include <cuda.h>
#include <cuda_bf16.h>
#include "b2/api.h"
#include "b2/launch.h"
#include "b2/gemm_tc.cuh"
#include "b2/ptx.cuh"
#include "b2/tma.h"

namespace b2 {
namespace {

using gemm::WorkUnit;

struct EpiParams {
  __nv_bfloat16* y;
  const __nv_bfloat16* residual;
  int64_t ldy;
  int64_t ldr;
  int M, N;          // logical output shape before any SwiGLU halving
  int splits;        // slots per tile in the workspace (split-K: the split count; stream-K: the most contributors a tile can have)
  float* workspace;  // [tiles][splits][BN][128] f32 partials
  uint32_t* counters;  // [tiles], zero on entry and on exit
  int mode;          // B2Epilogue
};

// Shared by both layouts: either pull a 32-column chunk out of TMEM or, for the reducing CTA of a split-K
// tile, sum the f32 partials of all splits.
template <int BN, int CH>
struct AccSource {
  bool from_ws;
  uint32_t taddr;
  const float* ws_tile;  // partials of this tile: [splits][BN][128]
  int splits;
  int p_local;
  __device__ __forceinline__ void load(int c, float (&v)[CH]) const {
    if (!from_ws) {
      uint32_t r[CH];
      if constexpr (CH == 32) ptx::tmem_ld_32x32(taddr + c * CH, r);
      else ptx::tmem_ld_32x16(taddr + c * CH, r);
      ptx::tc_wait_ld();
#pragma unroll
      for (int j = 0; j < CH; ++j) v[j] = __uint_as_float(r[j]);
    } else {
#pragma unroll
      for (int j = 0; j < CH; ++j) v[j] = 0.0f;
      for (int s = 0; s < splits; ++s) {
        const float* base = ws_tile + (static_cast<size_t>(s) * BN + c * CH) * 128 + p_local;
#pragma unroll
        for (int j = 0; j < CH; ++j) v[j] += __ldcg(base + j * 128);
      }
    }
  }
};

template <int BN, bool SWAP>
struct Epilogue {
  static constexpr int CH = BN >= 32 ? 32 : 16;
  EpiParams p;

  __device__ __forceinline__ void store_chunk(const WorkUnit& u, int c, int p_local, int lane, float (&v)[CH]) const {
    if constexpr (!SWAP) {
      // thread = output row m; chunk = CH consecutive output columns
      const int m = u.pb * 128 + p_local;
      const int n0 = u.qb * BN + c * CH;
      if (m >= p.M) return;
      if (p.mode == B2_EPI_SWIGLU) {
        // columns [0, CH/2) of the chunk are gate, [CH/2, CH) are up for the same CH/2 ffn indices
        constexpr int HALF = CH / 2;
        if (n0 >= p.N) return;
        float o[HALF];
#pragma unroll
        for (int j = 0; j < HALF; ++j) o[j] = ptx::silu(v[j]) * v[HALF + j];
        __nv_bfloat16* dst = p.y + static_cast<int64_t>(m) * p.ldy + n0 / 2;
#pragma unroll
        for (int g = 0; g < HALF / 8; ++g) {
          uint4 pk;
          pk.x = ptx::pack_bf16x2(o[g * 8 + 0], o[g * 8 + 1]);
          pk.y = ptx::pack_bf16x2(o[g * 8 + 2], o[g * 8 + 3]);
          pk.z = ptx::pack_bf16x2(o[g * 8 + 4], o[g * 8 + 5]);
          pk.w = ptx::pack_bf16x2(o[g * 8 + 6], o[g * 8 + 7]);
          ptx::st_v4(dst + g * 8, pk);
        }
        return;
      }
      __nv_bfloat16* dst = p.y + static_cast<int64_t>(m) * p.ldy + n0;
      const __nv_bfloat16* res = p.mode == B2_EPI_ADD_RESIDUAL ? p.residual + static_cast<int64_t>(m) * p.ldr + n0 : nullptr;
#pragma unroll
      for (int g = 0; g < CH / 8; ++g) {
        if (n0 + g * 8 >= p.N) break;
        float a[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] = v[g * 8 + j];
        if (res != nullptr) {
          const uint4 rv = ptx::ld_v4(res + g * 8);
          a[0] += ptx::bf16_lo(rv.x); a[1] += ptx::bf16_hi(rv.x);
          a[2] += ptx::bf16_lo(rv.y); a[3] += ptx::bf16_hi(rv.y);
          a[4] += ptx::bf16_lo(rv.z); a[5] += ptx::bf16_hi(rv.z);
          a[6] += ptx::bf16_lo(rv.w); a[7] += ptx::bf16_hi(rv.w);
        }
        uint4 pk;
        pk.x = ptx::pack_bf16x2(a[0], a[1]);
        pk.y = ptx::pack_bf16x2(a[2], a[3]);
        pk.z = ptx::pack_bf16x2(a[4], a[5]);
        pk.w = ptx::pack_bf16x2(a[6], a[7]);
        ptx::st_v4(dst + g * 8, pk);
      }
    } else {
      // thread = output column n; chunk = CH consecutive output rows (tokens)
      const int n = u.pb * 128 + p_local;
      const int m0 = u.qb * BN + c * CH;
      if (p.mode == B2_EPI_SWIGLU) {
        // lanes 0-15 hold gate rows, lanes 16-31 the matching up rows (16-row interleave of W)
        const int out_col = (u.pb * 128 + (p_local & ~31)) / 2 + (lane & 15);
#pragma unroll
        for (int j = 0; j < CH; ++j) {
          const float other = __shfl_xor_sync(0xffffffffu, v[j], 16);
          if (lane < 16 && n < p.N && m0 + j < p.M)
            p.y[static_cast<int64_t>(m0 + j) * p.ldy + out_col] = __float2bfloat16(ptx::silu(v[j]) * other);
        }
        return;
      }
      if (n >= p.N) return;
#pragma unroll
      for (int j = 0; j < CH; ++j) {
        if (m0 + j >= p.M) break;
        float a = v[j];
        if (p.mode == B2_EPI_ADD_RESIDUAL) a += __bfloat162float(p.residual[static_cast<int64_t>(m0 + j) * p.ldr + n]);
        p.y[static_cast<int64_t>(m0 + j) * p.ldy + n] = __float2bfloat16(a);
      }
    }
  }

  __device__ __forceinline__ void operator()(const WorkUnit& u, uint32_t taddr, int quarter, int lane,
                                             uint32_t* flag, Status* status) const {
    const int p_local = quarter * 32 + lane;
    AccSource<BN, CH> src{false, taddr, nullptr, u.nsplit, p_local};
    if (u.nsplit > 1) {
      // 1. publish this CTA's partial
      float* ws_tile = p.workspace + static_cast<size_t>(u.tile) * p.splits * BN * 128;
      float* mine = ws_tile + static_cast<size_t>(u.split) * BN * 128 + p_local;
#pragma unroll 1
      for (int c = 0; c < BN / CH; ++c) {
        float v[CH];
        src.load(c, v);
#pragma unroll
        for (int j = 0; j < CH; ++j) __stcg(mine + (c * CH + j) * 128, v[j]);
      }
      __threadfence();
      ptx::named_barrier_sync(1, gemm::kEpiThreads);
      if (threadIdx.x == 64) {  // first epilogue thread
        const uint32_t old = atomicAdd(p.counters + u.tile, 1u);
        const bool last = old == static_cast<uint32_t>(u.nsplit - 1);
        if (last) p.counters[u.tile] = 0;  // leave the counter ready for the next launch
        __threadfence();
        *flag = last ? 1u : 0u;
      }
      ptx::named_barrier_sync(1, gemm::kEpiThreads);
      const bool last = *flag != 0;
      ptx::named_barrier_sync(1, gemm::kEpiThreads);  // flag may be rewritten by the next work unit
      if (!last) return;
      src.from_ws = true;
      src.ws_tile = ws_tile;
    }
#pragma unroll 1
    for (int c = 0; c < BN / CH; ++c) {
      float v[CH];
      src.load(c, v);
      store_chunk(u, c, p_local, lane, v);
    }
  }
};

template <int BN, int STAGES, bool SWAP>
__global__ void __launch_bounds__(gemm::kThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_p, const __grid_constant__ CUtensorMap tmap_q,
                 gemm::TileSched sched, EpiParams ep, uint64_t policy_p, uint64_t policy_q, Status* status) {
  constexpr uint32_t idesc = ptx::make_idesc(1, 1, 128, BN);
  Epilogue<BN, SWAP> epi{ep};
  gemm::run<BN, STAGES, 2>(&tmap_p, &tmap_q, idesc, policy_p, policy_q, sched, gemm::NoGate{}, epi, status,
                           static_cast<int>(blockIdx.x), static_cast<int>(gridDim.x));
}

constexpr int stages_for(int bn) {
  const int stage = 128 * 64 * 2 + bn * 64 * 2;
  int s = (200 * 1024) / stage;
  return s > 10 ? 10 : s;
}

struct Config {
  bool swap;
  int bn;
  int splits;
  bool stream_k;   // cut the ragged last wave along K instead (splits == 1)
};

// Stream-K geometry for `tiles` output tiles of `num_kb` k-blocks on a grid of kNumSMs CTAs.
struct StreamK {
  int sk_tiles, per, units, max_nsplit;
};
StreamK stream_k_plan(long tiles, int num_kb) {
  StreamK s{};
  int rem = static_cast<int>(tiles % kNumSMs);
  if (tiles >= 2 * kNumSMs && rem > 0 && rem * 2 < kNumSMs) rem += kNumSMs;  // short runs cost more fix-up than they balance
  s.sk_tiles = rem;
  if (rem == 0) return s;
  const long iters = static_cast<long>(rem) * num_kb;
  s.per = static_cast<int>((iters + kNumSMs - 1) / kNumSMs);
  s.units = (s.per + num_kb - 1) / num_kb + 1;
  s.max_nsplit = (num_kb + s.per - 1) / s.per + 1;
  return s;
}

// Cost model behind the automatic configuration (cycles at SM clock; constants fitted to a sweep of the four
// Llama-8B layer GEMMs at M = 16 ... 1024 on a B200):
//   one work unit = k-blocks * max(tensor time, shared-memory fill time) + fixed epilogue cost
//   tensor time of a 128 x bn x 64 block  = 2 * bn / 0.75   (8192 dense bf16 FLOP/clk/SM nominal, ~75 % reachable)
//   fill time of the same block           = (128 + bn) * 128 B at ~128 B/clk from L2
//   a unit can go no faster than its share of the operand bytes at one SM's share of HBM bandwidth (decode shapes)
//   split-K adds a semaphore round trip and a pass over splits * bn * 128 f32 partials
//   the kernel is persistent over 148 SMs, so the total is waves * unit + launch/prologue cost,
//   and never less than streaming every operand once from HBM.
double model_cycles(int M, int N, int K, bool swap, int bn, int splits, bool stream_k = false) {
  const int num_kb = (K + 63) / 64;
  const int rows_p = swap ? N : M, rows_q = swap ? M : N;
  const long units = static_cast<long>((rows_p + 127) / 128) * ((rows_q + bn - 1) / bn) * splits;
  const double kb = (num_kb + splits - 1) / splits;
  const double mma = kb * 2.0 * bn / 0.75;
  const double fill = kb * (128.0 + bn);
  // each unit's share of the bytes that must come from HBM, at one SM's share of the HBM bandwidth
  const double dram = (static_cast<double>(N) * K + static_cast<double>(M) * K) * 2.0 / units / (3300.0 / kNumSMs);
  double unit = (mma > fill ? mma : fill);
  unit = (unit > dram ? unit : dram) + 600.0;
  if (splits > 1) unit += 2500.0 + splits * bn * 128.0 * 4.0 / 48.0;
  double waves = static_cast<double>((units + kNumSMs - 1) / kNumSMs);
  double extra = 0.0;
  if (stream_k) {
    // every CTA gets the same number of k-blocks; each pays the epilogue of the tiles it touches and one fix-up
    const StreamK sk = stream_k_plan(units, num_kb);
    waves = static_cast<double>(units) / kNumSMs;
    if (sk.sk_tiles > 0) extra = 600.0 * sk.units + 2500.0 + sk.max_nsplit * bn * 128.0 * 4.0 / 48.0;
  }
  const double total = waves * unit + extra + 7000.0;
  const double hbm = (static_cast<double>(N) * K + static_cast<double>(M) * K + static_cast<double>(M) * N) * 2.0 / 3300.0 + 5000.0;
  return total > hbm ? total : hbm;
}

Config choose_config(int M, int N, int K, int epilogue) {
  const int num_kb = (K + 63) / 64;
  Config best{};
  double best_t = 1e300;
  auto consider = [&](bool swap, int bn, int splits) {
    if (splits > num_kb || (splits > 1 && num_kb / splits < 4)) return;
    if (epilogue == B2_EPI_SWIGLU && !swap && bn < 32) return;
    const long rows_p = swap ? N : M, rows_q = swap ? M : N;
    const long tiles = ((rows_p + 127) / 128) * ((rows_q + bn - 1) / bn);
    if (splits > 1 && (tiles > 65536 || tiles * splits * bn * 128 * 4 > (64l << 20))) return;
    const double t = model_cycles(M, N, K, swap, bn, splits);
    if (t < best_t) {
      best_t = t;
      best = Config{swap, bn, splits, false};
    }
    // Stream-K staggers the CTAs along K, which breaks the lock-step in which CTAs that share an operand tile
    // fetch it (measured: up to 1.5x slower once operands are shared). It pays where nothing is shared: the
    // swapped layout with a single token tile, where every weight byte is read by exactly one CTA.
    if (splits == 1 && swap && M <= bn && num_kb >= 8 && tiles % kNumSMs != 0) {
      const double ts = model_cycles(M, N, K, swap, bn, 1, true);
      if (ts < best_t) {
        best_t = ts;
        best = Config{swap, bn, 1, true};
      }
    }
  };
  static const int kSplits[] = {1, 2, 4, 8};
  if (M <= 256) {
    static const int kBn[] = {16, 32, 64, 128, 256};
    for (int bn : kBn) {
      if (bn == 256 && M <= 128) continue;
      if (bn * 4 < M || (bn >= 2 * M && bn > 16)) continue;  // neither many token tiles nor mostly padding
      for (int sp : kSplits) consider(true, bn, sp);
    }
  }
  if (M > 64) {
    static const int kBn[] = {64, 96, 128, 160, 192, 224, 256};
    for (int bn : kBn) {
      if (N % 8 != 0) continue;
      for (int sp : kSplits) consider(false, bn, sp);
    }
  }
  if (best_t == 1e300) best = Config{true, 16, 1, false};
  return best;
}

template <int BN, bool SWAP>
int launch(const void* x, const void* w, int M, int N, int K, int64_t ldx, int64_t ldw, int splits, bool stream_k, EpiParams ep,
           Status* status, cudaStream_t stream) {
  constexpr int STAGES = stages_for(BN);
  using L = gemm::SmemLayout<BN, STAGES>;
  const void* p_ptr = SWAP ? w : x;
  const void* q_ptr = SWAP ? x : w;
  const int rows_p = SWAP ? N : M, rows_q = SWAP ? M : N;
  const int64_t ldp = SWAP ? ldw : ldx, ldq = SWAP ? ldx : ldw;
  CUtensorMap tp, tq;
  if (!make_tmap_2d(&tp, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p_ptr, rows_p, K, ldp * 2, 128, 64,
                    CU_TENSOR_MAP_SWIZZLE_128B) ||
      !make_tmap_2d(&tq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, q_ptr, rows_q, K, ldq * 2, BN, 64,
                    CU_TENSOR_MAP_SWIZZLE_128B))
    return -kBadArgument;
  gemm::TileSched sched{};
  sched.p_blocks = (rows_p + 127) / 128;
  sched.q_blocks = (rows_q + BN - 1) / BN;
  sched.splits = splits;
  sched.num_kb = (K + 63) / 64;
  sched.kb_per_split = (sched.num_kb + splits - 1) / splits;
  sched.bn = BN;
  ep.splits = splits;
  if (stream_k && splits == 1) {
    const StreamK sk = stream_k_plan(static_cast<long>(sched.p_blocks) * sched.q_blocks, sched.num_kb);
    if (sk.sk_tiles > 0) {
      sched.sk_tiles = sk.sk_tiles;
      sched.sk_per = sk.per;
      sched.sk_units = sk.units;
      sched.num_ctas = kNumSMs;
      ep.splits = sk.max_nsplit;
    }
  }
  auto kern = gemm_bf16_kernel<BN, STAGES, SWAP>;
  static DeviceOnce attr_once;
  if (const int rc = attr_once.run([&] {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotalBytes);
        return e;
      }))
    return rc;
  const int total = sched.p_blocks * sched.q_blocks * splits;
  const int grid = (total < kNumSMs && sched.sk_tiles == 0) ? total : kNumSMs;
  // Weights are read once per step: stream them; activations are re-read by every weight tile: keep them.
  const uint64_t pol_w = ptx::kEvictFirst, pol_x = ptx::kEvictLast;
  const uint64_t pol_p = SWAP ? pol_w : (M <= 1024 ? pol_x : ptx::kEvictNormal);
  const uint64_t pol_q = SWAP ? pol_x : (M <= 1024 ? pol_w : ptx::kEvictNormal);
  launch_pdl(kern, dim3(grid), dim3(gemm::kThreads), L::kTotalBytes, stream, tp, tq, sched, ep, pol_p, pol_q, status);
  return last_launch_rc();
}

}  // namespace
}  // namespace b2

using namespace b2;

extern "C" int64_t b2_gemm_workspace_bytes(int M, int N, int K) {
  // counters + the partials bound the automatic configuration respects (explicit configurations are checked
  // against the caller's actual workspace size at launch)
  (void)M; (void)N; (void)K;
  return 65536 * 4 + (64l << 20);
}

extern "C" int b2_gemm_bf16(const void* x, const void* w, void* y, const void* residual, int M, int N, int K,
                            int64_t ldx, int64_t ldw, int64_t ldy, int epilogue, int config, void* workspace,
                            int64_t workspace_bytes, Status* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0) return -kBadArgument;
  Config c = choose_config(M, N, K, epilogue);
  if (config != 0) {
    c.swap = (config >> 30) & 1;
    c.stream_k = (config >> 29) & 1;
    c.splits = (config >> 16) & 0xff;
    c.bn = config & 0xffff;
    if (c.splits < 1) c.splits = 1;
    if (c.stream_k) c.splits = 1;
  }
  const int num_kb = (K + 63) / 64;
  if (c.splits > num_kb) c.splits = num_kb;
  if (c.splits > 16) c.splits = 16;
  // every split must own at least one k-block
  while (c.splits > 1 && ((num_kb + c.splits - 1) / c.splits) * (c.splits - 1) >= num_kb) --c.splits;
  if (epilogue == B2_EPI_SWIGLU) {
    if (N % 32 != 0) return -kBadArgument;
    if (c.bn < 32 && !c.swap) return -kBadArgument;
  } else if (!c.swap && (N % 8 != 0 || ldy % 8 != 0)) {
    return -kBadArgument;
  }
  if (epilogue == B2_EPI_ADD_RESIDUAL && residual == nullptr) return -kBadArgument;
  EpiParams ep{};
  ep.y = static_cast<__nv_bfloat16*>(y);
  ep.residual = static_cast<const __nv_bfloat16*>(residual);
  ep.ldy = ldy;
  ep.ldr = ldy;
  ep.M = M;
  ep.N = N;
  ep.mode = epilogue;
  if (c.splits > 1) {
    const int64_t counters_bytes = 65536 * 4;
    // P is the 128-row operand: W rows when swapped, X rows otherwise
    const int rows_p = c.swap ? N : M, rows_q = c.swap ? M : N;
    const int64_t tiles = static_cast<int64_t>((rows_p + 127) / 128) * ((rows_q + c.bn - 1) / c.bn);
    const int64_t need = counters_bytes + tiles * c.splits * c.bn * 128 * 4;
    if (workspace == nullptr || workspace_bytes < need || tiles > 65536) return -kTooLarge;
    ep.counters = static_cast<uint32_t*>(workspace);
    ep.workspace = reinterpret_cast<float*>(static_cast<char*>(workspace) + counters_bytes);
  } else if (c.stream_k) {
    const int64_t counters_bytes = 65536 * 4;
    const int rows_p = c.swap ? N : M, rows_q = c.swap ? M : N;
    const int64_t tiles = static_cast<int64_t>((rows_p + 127) / 128) * ((rows_q + c.bn - 1) / c.bn);
    const StreamK sk = stream_k_plan(tiles, num_kb);
    const int64_t need = counters_bytes + static_cast<int64_t>(kNumSMs) * sk.max_nsplit * c.bn * 128 * 4;
    if (sk.sk_tiles == 0 || workspace == nullptr || workspace_bytes < need) {
      c.stream_k = false;  // nothing ragged to balance, or no room for the partials: plain tile loop
    } else {
      ep.counters = static_cast<uint32_t*>(workspace);
      ep.workspace = reinterpret_cast<float*>(static_cast<char*>(workspace) + counters_bytes);
    }
  }
#define B2_LAUNCH(BN_, SWAP_) \
  return launch<BN_, SWAP_>(x, w, M, N, K, ldx, ldw, c.splits, c.stream_k, ep, status, stream)
  if (c.swap) {
    switch (c.bn) {
      case 16: B2_LAUNCH(16, true);
      case 32: B2_LAUNCH(32, true);
      case 64: B2_LAUNCH(64, true);
      case 128: B2_LAUNCH(128, true);
      case 256: B2_LAUNCH(256, true);
      default: return -kBadArgument;
    }
  } else {
    switch (c.bn) {
      case 64: B2_LAUNCH(64, false);
      case 96: B2_LAUNCH(96, false);
      case 128: B2_LAUNCH(128, false);
      case 160: B2_LAUNCH(160, false);
      case 192: B2_LAUNCH(192, false);
      case 224: B2_LAUNCH(224, false);
      case 256: B2_LAUNCH(256, false);
      default: return -kBadArgument;
    }
  }
#undef B2_LAUNCH
}

// ------------------------------------------------------------------------------------------------------------
// Allocation-free variant (declared in b2/noalloc.h). The split-K scratch is this file-scope array: the first
// 256 KiB are the per-tile semaphores, the rest holds f32 partial tiles. In host code the name `g_noalloc_scratch`
// is only a handle for the runtime; the address a kernel can use comes from cudaGetSymbolAddress, looked up once
// per device with that device current.
// ------------------------------------------------------------------------------------------------------------
#include "b2/noalloc.h"

static __device__ __align__(256) unsigned char g_noalloc_scratch[B2_NOALLOC_SCRATCH_BYTES];
// Where a kernel launched through this entry point records a wait that ran out (it has no caller-supplied status).
static __device__ b2::Status g_noalloc_status;

#include <mutex>

namespace {
constexpr int kNoallocMaxDevices = 64;
constexpr int64_t kNoallocCounterBytes = 65536 * 4;
struct NoallocDevice {
  std::atomic<void*> scratch{nullptr};
  b2::Status* status = nullptr;
};
NoallocDevice g_noalloc_dev[kNoallocMaxDevices];
std::mutex g_noalloc_mutex;   // first use per device may come from several host threads at once

// Device addresses of the scratch and the status word for the current device. The first use on a device looks
// them up (the names above are host-side handles, not addresses a kernel could use) and clears the semaphore words
// and the status word.
int noalloc_device(NoallocDevice** out, cudaStream_t stream) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoallocMaxDevices) return -b2::kBadArgument;
  NoallocDevice& d = g_noalloc_dev[dev];
  if (d.scratch.load(std::memory_order_acquire) == nullptr) {
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (d.scratch.load(std::memory_order_relaxed) == nullptr) {
      void* p = nullptr;
      void* st = nullptr;
      cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
      if (e == cudaSuccess) e = cudaGetSymbolAddress(&st, g_noalloc_status);
      if (e == cudaSuccess && (p == nullptr || st == nullptr)) e = cudaErrorInvalidSymbol;
      if (e == cudaSuccess) e = cudaMemsetAsync(p, 0, kNoallocCounterBytes, stream);
      if (e == cudaSuccess) e = cudaMemsetAsync(st, 0, sizeof(b2::Status), stream);
      if (e != cudaSuccess) {
        cudaGetLastError();
        return b2::cuda_rc(e);
      }
      d.status = static_cast<b2::Status*>(st);
      d.scratch.store(p, std::memory_order_release);
    }
  }
  *out = &d;
  return 0;
}
}  // namespace

extern "C" int b2_gemm_bf16_noalloc(const void* x, const void* w, void* y, int M, int N, int K, int64_t ldx,
                                    int64_t ldw, int64_t ldy, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (x == nullptr || w == nullptr || y == nullptr || K <= 0 || K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0) return -kBadArgument;
  // Same configuration rule and the same clamps as the allocating entry point, then checked against the fixed capacity.
  Config c = choose_config(M, N, K, B2_EPI_NONE);
  const int num_kb = (K + 63) / 64;
  if (c.splits > num_kb) c.splits = num_kb;
  if (c.splits > 16) c.splits = 16;
  while (c.splits > 1 && ((num_kb + c.splits - 1) / c.splits) * (c.splits - 1) >= num_kb) --c.splits;
  if (!c.swap && (N % 8 != 0 || ldy % 8 != 0)) return -kBadArgument;
  const int rows_p = c.swap ? N : M, rows_q = c.swap ? M : N;
  const int64_t tiles = static_cast<int64_t>((rows_p + 127) / 128) * ((rows_q + c.bn - 1) / c.bn);
  if (c.splits > 1) {
    const int64_t need = kNoallocCounterBytes + tiles * c.splits * c.bn * 128 * 4;
    if (need > B2_NOALLOC_SCRATCH_BYTES || tiles > 65536) return -kTooLarge;
  }
  NoallocDevice* d = nullptr;
  const int rc = noalloc_device(&d, stream);
  if (rc != 0) return rc;
  void* scratch = d->scratch.load(std::memory_order_acquire);
  EpiParams ep{};
  ep.y = static_cast<__nv_bfloat16*>(y);
  ep.ldy = ldy;
  ep.ldr = ldy;
  ep.M = M;
  ep.N = N;
  ep.mode = B2_EPI_NONE;
  ep.counters = static_cast<uint32_t*>(scratch);
  ep.workspace = reinterpret_cast<float*>(static_cast<char*>(scratch) + kNoallocCounterBytes);
#define B2_LAUNCH_NA(BN_, SWAP_) return launch<BN_, SWAP_>(x, w, M, N, K, ldx, ldw, c.splits, false, ep, d->status, stream)
  if (c.swap) {
    switch (c.bn) {
      case 16: B2_LAUNCH_NA(16, true);
      case 32: B2_LAUNCH_NA(32, true);
      case 64: B2_LAUNCH_NA(64, true);
      case 128: B2_LAUNCH_NA(128, true);
      case 256: B2_LAUNCH_NA(256, true);
      default: return -kBadArgument;
    }
  }
  switch (c.bn) {
    case 64: B2_LAUNCH_NA(64, false);
    case 96: B2_LAUNCH_NA(96, false);
    case 128: B2_LAUNCH_NA(128, false);
    case 160: B2_LAUNCH_NA(160, false);
    case 192: B2_LAUNCH_NA(192, false);
    case 224: B2_LAUNCH_NA(224, false);
    case 256: B2_LAUNCH_NA(256, false);
    default: return -kBadArgument;
  }
#undef B2_LAUNCH_NA
}

extern "C" int b2_gemm_bf16_noalloc_status(cudaStream_t stream) {
  NoallocDevice* d = nullptr;
  const int rc = noalloc_device(&d, stream);
  if (rc != 0) return rc;
  b2::Status host{};
  cudaError_t e = cudaMemcpyAsync(&host, d->status, sizeof(host), cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return b2::cuda_rc(e);
  }
  if (host.code == kOk) return 0;
  // A kernel that gave up may have left semaphores mid-count: put both the semaphores and the record back to zero,
  // so the calls that follow count from a clean state.
  e = cudaMemsetAsync(d->scratch.load(std::memory_order_acquire), 0, kNoallocCounterBytes, stream);
  if (e == cudaSuccess) e = cudaMemsetAsync(d->status, 0, sizeof(b2::Status), stream);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return b2::cuda_rc(e);
  }
  return -host.code;
}

// The configuration the automatic rule picks for a shape, encoded like the `config` argument
// ((swap << 30) | (stream_k << 29) | (splits << 16) | bn): for tuning sweeps and tests. Host only, no launch.
extern "C" int b2_gemm_auto_config(int M, int N, int K, int epilogue) {
  const Config c = choose_config(M, N, K, epilogue);
  return (static_cast<int>(c.swap) << 30) | (static_cast<int>(c.stream_k) << 29) | (c.splits << 16) | c.bn;
}
