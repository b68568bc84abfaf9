// GGUF k-quant weights: standalone dequantisation and the dequant-fused GEMM
//   Y[M, N] = X[M, K] * dequant(Wq)[N, K]^T     Wq: Q4_K or Q6_K super-blocks, row-major [N][K / 256].
// The fused kernel is the tcgen05 GEMM core with the weights on the UMMA M side (decode-shaped: tokens are the UMMA
// N dimension) and a fourth role: four fill warps read the packed blocks, dequantise 64 weights per row per stage
// to bf16 and write them in the 128-byte-swizzled shared-memory layout the MMA descriptor reads. The packed
// weights (4.5 / 6.56 bits each) are the only weight bytes that cross HBM.
#include <cstdint>
#include <cuda.h>
#include <cuda_bf16.h>
#include "b2/api.h"
#include "b2/launch.h"
#include "b2/gemm_tc.cuh"
#include "b2/gguf.cuh"
#include "b2/ptx.cuh"
#include "b2/tma.h"

namespace b2 {
namespace {

// One thread per 64 weights, wide loads (tensor 16-byte aligned).
__global__ void dequant64_kernel(const uint8_t* __restrict__ wq, int ggml_type, __nv_bfloat16* __restrict__ out, int64_t n_pairs) {
  const int64_t pidx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (pidx >= n_pairs) return;
  const int64_t blk = pidx >> 2;
  const int g0 = static_cast<int>(pidx & 3) * 2;
  float v[64];
  if (ggml_type == gguf::kTypeQ4K) gguf::q4k_dequant64(wq + blk * gguf::kQ4KBytes, g0, v);
  else gguf::q6k_dequant64(wq + blk * gguf::kQ6KBytes, g0, v);
  uint4* dst = reinterpret_cast<uint4*>(out + pidx * 64);
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    uint4 pk;
    pk.x = ptx::pack_bf16x2(v[c * 8 + 0], v[c * 8 + 1]);
    pk.y = ptx::pack_bf16x2(v[c * 8 + 2], v[c * 8 + 3]);
    pk.z = ptx::pack_bf16x2(v[c * 8 + 4], v[c * 8 + 5]);
    pk.w = ptx::pack_bf16x2(v[c * 8 + 6], v[c * 8 + 7]);
    dst[c] = pk;
  }
}

__global__ void dequant_kernel(const uint8_t* __restrict__ wq, int ggml_type, __nv_bfloat16* __restrict__ out, int64_t n_groups) {
  // one thread per 32 weights
  const int64_t gidx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (gidx >= n_groups) return;
  const int64_t blk = gidx >> 3;
  const int g = static_cast<int>(gidx & 7);
  float v[32];
  if (ggml_type == gguf::kTypeQ4K) gguf::q4k_dequant32(wq + blk * gguf::kQ4KBytes, g, v);
  else gguf::q6k_dequant32(wq + blk * gguf::kQ6KBytes, g, v);
  uint4* dst = reinterpret_cast<uint4*>(out + gidx * 32);
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint4 pk;
    pk.x = ptx::pack_bf16x2(v[c * 8 + 0], v[c * 8 + 1]);
    pk.y = ptx::pack_bf16x2(v[c * 8 + 2], v[c * 8 + 3]);
    pk.z = ptx::pack_bf16x2(v[c * 8 + 4], v[c * 8 + 5]);
    pk.w = ptx::pack_bf16x2(v[c * 8 + 6], v[c * 8 + 7]);
    dst[c] = pk;
  }
}

// P-tile fill: thread (fill warp fw, lane) owns tile row fw * 32 + lane; a k-block is 64 weights = two 32-weight groups.
struct GgufFill {
  static constexpr bool kActive = true;
  const uint8_t* wq;
  int ggml_type, N, blocks_per_row;
  int wide;   // the packed tensor is 16-byte aligned: Q4_K blocks are read 16 bytes at a time, Q6_K blocks 2 bytes at a time
  __device__ __forceinline__ void operator()(const gemm::WorkUnit& u, int kb, uint8_t* stage, int fw, int lane) const {
    const int r = fw * 32 + lane;
    const int n = u.p_coord + r;
    float v[64];
    if (n < N) {
      const int sb = kb >> 2, g0 = (kb & 3) * 2;
      const uint8_t* blk = wq + (static_cast<int64_t>(n) * blocks_per_row + sb) * (ggml_type == gguf::kTypeQ4K ? gguf::kQ4KBytes : gguf::kQ6KBytes);
      if (ggml_type == gguf::kTypeQ4K) {
        if (wide) {
          gguf::q4k_dequant64(blk, g0, v);
        } else {
          gguf::q4k_dequant32(blk, g0, v);
          gguf::q4k_dequant32(blk, g0 + 1, v + 32);
        }
      } else if (wide) {
        gguf::q6k_dequant64(blk, g0, v);
      } else {
        gguf::q6k_dequant32(blk, g0, v);
        gguf::q6k_dequant32(blk, g0 + 1, v + 32);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 64; ++i) v[i] = 0.0f;
    }
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      uint4 pk;
      pk.x = ptx::pack_bf16x2(v[c * 8 + 0], v[c * 8 + 1]);
      pk.y = ptx::pack_bf16x2(v[c * 8 + 2], v[c * 8 + 3]);
      pk.z = ptx::pack_bf16x2(v[c * 8 + 4], v[c * 8 + 5]);
      pk.w = ptx::pack_bf16x2(v[c * 8 + 6], v[c * 8 + 7]);
      *reinterpret_cast<uint4*>(stage + gemm::sw128_offset(r, c)) = pk;
    }
  }
};

struct GgufEpiParams {
  __nv_bfloat16* y;
  int64_t ldy;
  int M, N;
};
template <int BN>
struct GgufEpilogue {
  static constexpr int CH = BN >= 32 ? 32 : 16;
  GgufEpiParams p;
  __device__ __forceinline__ void operator()(const gemm::WorkUnit& u, uint32_t taddr, int quarter, int lane, uint32_t*, Status*) const {
    const int n = u.pb * 128 + quarter * 32 + lane;
#pragma unroll 1
    for (int c = 0; c < BN / CH; ++c) {
      uint32_t r[CH];
      if constexpr (CH == 32) ptx::tmem_ld_32x32(taddr + c * CH, r);
      else ptx::tmem_ld_32x16(taddr + c * CH, r);
      ptx::tc_wait_ld();
      if (n >= p.N) continue;
      const int m0 = u.qb * BN + c * CH;
#pragma unroll
      for (int j = 0; j < CH; ++j) {
        if (m0 + j >= p.M) break;
        p.y[static_cast<int64_t>(m0 + j) * p.ldy + n] = __float2bfloat16(__uint_as_float(r[j]));
      }
    }
  }
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(gemm::kThreadsWithFill, 1)
gemm_gguf_kernel(const __grid_constant__ CUtensorMap tmap_x, gemm::TileSched sched, GgufFill fill, GgufEpiParams ep, Status* status) {
  constexpr uint32_t idesc = ptx::make_idesc(1, 1, 128, BN);
  GgufEpilogue<BN> epi{ep};
  gemm::run<BN, STAGES, 2>(&tmap_x, &tmap_x, idesc, ptx::kEvictNormal, ptx::kEvictLast, sched, gemm::NoGate{}, epi, status,
                           static_cast<int>(blockIdx.x), static_cast<int>(gridDim.x), fill);
}

template <int BN>
int launch_gguf(const void* x, const void* wq, int ggml_type, void* y, int M, int N, int K, Status* status, cudaStream_t stream) {
  constexpr int kStage = 128 * 64 * 2 + BN * 64 * 2;
  constexpr int STAGES = (160 * 1024 / kStage) > 8 ? 8 : (160 * 1024 / kStage);
  using L = gemm::SmemLayout<BN, STAGES>;
  CUtensorMap tx;
  if (!make_tmap_2d(&tx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, M, K, static_cast<uint64_t>(K) * 2, BN, 64, CU_TENSOR_MAP_SWIZZLE_128B))
    return -kBadArgument;
  gemm::TileSched sched{};
  sched.p_blocks = (N + 127) / 128;
  sched.q_blocks = (M + BN - 1) / BN;
  sched.splits = 1;
  sched.num_kb = K / 64;
  sched.kb_per_split = sched.num_kb;
  sched.bn = BN;
  GgufFill fill{static_cast<const uint8_t*>(wq), ggml_type, N, K / gguf::kQK, (reinterpret_cast<uintptr_t>(wq) & 15) == 0 ? 1 : 0};
  GgufEpiParams ep{static_cast<__nv_bfloat16*>(y), N, M, N};
  auto kern = gemm_gguf_kernel<BN, STAGES>;
  static DeviceOnce attr_once;
  if (const int rc = attr_once.run([&] {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotalBytes);
        return e;
      }))
    return rc;
  const int total = sched.p_blocks * sched.q_blocks;
  kern<<<total < kNumSMs ? total : kNumSMs, gemm::kThreadsWithFill, L::kTotalBytes, stream>>>(tx, sched, fill, ep, status);
  return last_launch_rc();
}

}  // namespace
}  // namespace b2

using namespace b2;

extern "C" int b2_dequant_gguf(const void* wq, int ggml_type, void* out_bf16, int64_t n_elems, cudaStream_t stream) {
  if (n_elems <= 0) return 0;
  if (n_elems % gguf::kQK != 0 || gguf::block_bytes(ggml_type) == 0) return -kBadArgument;
  if ((reinterpret_cast<uintptr_t>(wq) & 15) == 0 && (reinterpret_cast<uintptr_t>(out_bf16) & 15) == 0) {
    const int64_t pairs = n_elems / 64;
    dequant64_kernel<<<static_cast<unsigned>((pairs + 127) / 128), 128, 0, stream>>>(static_cast<const uint8_t*>(wq), ggml_type,
                                                                                    static_cast<__nv_bfloat16*>(out_bf16), pairs);
    return last_launch_rc();
  }
  const int64_t groups = n_elems / 32;
  dequant_kernel<<<static_cast<unsigned>((groups + 127) / 128), 128, 0, stream>>>(static_cast<const uint8_t*>(wq), ggml_type,
                                                                                  static_cast<__nv_bfloat16*>(out_bf16), groups);
  return last_launch_rc();
}

extern "C" int b2_gemm_gguf(const void* x, const void* wq, int ggml_type, void* y, int M, int N, int K, b2::Status* status,
                            cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K % gguf::kQK != 0 || gguf::block_bytes(ggml_type) == 0) return -kBadArgument;
  if (M <= 16) return launch_gguf<16>(x, wq, ggml_type, y, M, N, K, status, stream);
  if (M <= 32) return launch_gguf<32>(x, wq, ggml_type, y, M, N, K, status, stream);
  if (M <= 64) return launch_gguf<64>(x, wq, ggml_type, y, M, N, K, status, stream);
  return launch_gguf<128>(x, wq, ggml_type, y, M, N, K, status, stream);
}
