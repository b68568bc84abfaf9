// Token sampling: greedy argmax and temperature / top-k / top-p sampling over a [rows, vocab] logits matrix.
//
// Selection of the k-th largest logit is an MSB-first radix select on order-preserving integer keys: the
// GPU form of the quick-select `partition(span, k)` the reference offers on the CPU
// (stdlib/src/builtin/sort.mojo:373-506 - first k elements = k largest, unordered). Top-p reuses the same
// digit walk with probability mass instead of counts. The uniform draw is Philox4x32-10 keyed by
// (seed; step, row), replacing the reference's closed host RNG (stdlib/src/random/random.mojo:32-92).
// One CTA per row; the row stays in L2 across passes.
#include <cstdint>
#include <cuda_bf16.h>
#include "b2/api.h"
#include "b2/launch.h"
#include "b2/ptx.cuh"
#include "b2/vec.cuh"

namespace b2 {
namespace {

constexpr int kThreads = 1024;

template <bool BF16>
__device__ __forceinline__ float load_logit(const void* row, int i) {
  if (BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(row)[i]);
  return static_cast<const float*>(row)[i];
}
__device__ __forceinline__ uint32_t float_key(float x) {
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct Philox {
  uint32_t c[4];
  uint32_t k[2];
  __device__ __forceinline__ void round() {
    const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u;
    const uint32_t hi0 = __umulhi(M0, c[0]), lo0 = M0 * c[0];
    const uint32_t hi1 = __umulhi(M1, c[2]), lo1 = M1 * c[2];
    const uint32_t n0 = hi1 ^ c[1] ^ k[0], n1 = lo1, n2 = hi0 ^ c[3] ^ k[1], n3 = lo0;
    c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
  }
  __device__ __forceinline__ void run10() {
#pragma unroll
    for (int i = 0; i < 10; ++i) {
      round();
      if (i < 9) { k[0] += 0x9E3779B9u; k[1] += 0xBB67AE85u; }
    }
  }
};
__device__ __forceinline__ float philox_uniform(uint64_t seed, uint64_t step, uint32_t row) {
  Philox p;
  p.c[0] = static_cast<uint32_t>(step);
  p.c[1] = static_cast<uint32_t>(step >> 32);
  p.c[2] = row;
  p.c[3] = 0;
  p.k[0] = static_cast<uint32_t>(seed);
  p.k[1] = static_cast<uint32_t>(seed >> 32);
  p.run10();
  return static_cast<float>(p.c[0] >> 8) * (1.0f / 16777216.0f);
}

struct ArgMax {
  float v;
  int i;
};
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}
template <bool BF16>
__device__ ArgMax block_argmax(const void* row, int vocab, ArgMax* scratch) {
  ArgMax best{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float x = load_logit<BF16>(row, i);
    if (x > best.v || (x == best.v && i < best.i)) best = ArgMax{x, i};
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (lane == 0) scratch[warp] = best;
  __syncthreads();
  if (warp == 0) {
    ArgMax b = lane < nw ? scratch[lane] : ArgMax{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ArgMax other{__shfl_xor_sync(0xffffffffu, b.v, o), __shfl_xor_sync(0xffffffffu, b.i, o)};
      b = better(b, other);
    }
    if (lane == 0) scratch[32] = b;
  }
  __syncthreads();
  const ArgMax r = scratch[32];
  __syncthreads();
  if (r.i == 0x7fffffff) return ArgMax{r.v, 0};  // all -inf / NaN row
  return r;
}

template <bool BF16>
__global__ void __launch_bounds__(kThreads) argmax_kernel(const void* logits, int64_t* ids, float* max_out, int vocab,
                                                           int64_t row_stride) {
  ptx::grid_dep_sync();
  __shared__ ArgMax scratch[33];
  const int row = blockIdx.x;
  const void* base = static_cast<const char*>(logits) + static_cast<int64_t>(row) * row_stride * (BF16 ? 2 : 4);
  const ArgMax r = block_argmax<BF16>(base, vocab, scratch);
  if (threadIdx.x == 0) {
    ids[row] = r.i;
    if (max_out != nullptr) max_out[row] = r.v;
  }
}

// Visit every logit of a row with its index: 16-byte loads (8 bf16 / 4 f32 per load, consecutive threads on
// consecutive vectors) when the row is 16-byte aligned, scalar loads otherwise and for the tail.
template <bool BF16, class F>
__device__ __forceinline__ void for_each_logit(const void* row, int vocab, F&& f) {
  constexpr int V = BF16 ? 8 : 4;
  const bool aligned = (reinterpret_cast<uintptr_t>(row) & 15u) == 0;
  const int nvec = aligned ? vocab / V : 0;
  const uint4* rv = static_cast<const uint4*>(row);
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    const uint4 q = rv[v];
    if (BF16) {
      float x[8];
      bf16x8_to_f32(q, x);
#pragma unroll
      for (int j = 0; j < 8; ++j) f(x[j], v * 8 + j);
    } else {
      f(__uint_as_float(q.x), v * 4 + 0);
      f(__uint_as_float(q.y), v * 4 + 1);
      f(__uint_as_float(q.z), v * 4 + 2);
      f(__uint_as_float(q.w), v * 4 + 3);
    }
  }
  for (int i = nvec * V + threadIdx.x; i < vocab; i += blockDim.x) f(load_logit<BF16>(row, i), i);
}

constexpr int kWarps = kThreads / 32;

// MSB-first radix walk. MASS = false: find the key of the `want`-th largest element (counts).
// MASS = true: find the key at which the mass of strictly larger keys first reaches `want`.
// Only keys >= floor_key participate. Returns the selected key.
// Every warp accumulates into its own 256-bin histogram (logits crowd into a few exponent buckets: one shared
// histogram serialises all 1024 threads on the same two or three words), and the warps' histograms are added up
// afterwards. bf16 logits have 16 significant key bits, so their walk is two digits long instead of four.
template <bool BF16, bool MASS>
__device__ uint32_t radix_select(const void* row, int vocab, float want, uint32_t floor_key, float mx, float inv_t,
                                 float* hist /* [kWarps + 1][256] */, float* bcast) {
  uint32_t prefix = 0, mask = 0;
  const int warp = threadIdx.x >> 5;
  float* mine = hist + warp * 256;
  float* total = hist + kWarps * 256;
  constexpr int kLastPass = BF16 ? 2 : 0;
  for (int pass = 3; pass >= kLastPass; --pass) {
    for (int b = threadIdx.x; b < (kWarps + 1) * 256; b += blockDim.x) hist[b] = 0.0f;
    __syncthreads();
    const int shift = pass * 8;
    for_each_logit<BF16>(row, vocab, [&](float x, int) {
      const uint32_t key = float_key(x);
      if (key >= floor_key && (key & mask) == prefix) {
        const float w = MASS ? ptx::ex2((x - mx) * inv_t) : 1.0f;
        atomicAdd(&mine[(key >> shift) & 0xffu], w);
      }
    });
    __syncthreads();
    if (threadIdx.x < 256) {
      float acc = 0.0f;
#pragma unroll 4
      for (int w2 = 0; w2 < kWarps; ++w2) acc += hist[w2 * 256 + threadIdx.x];
      total[threadIdx.x] = acc;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float acc = 0.0f;
      int b = 255;
      for (; b > 0; --b) {
        if (acc + total[b] >= want) break;
        acc += total[b];
      }
      bcast[0] = acc;
      bcast[1] = __int_as_float(b);
    }
    __syncthreads();
    want -= bcast[0];
    const uint32_t b = static_cast<uint32_t>(__float_as_int(bcast[1]));
    prefix |= b << shift;
    mask |= 0xffu << shift;
    __syncthreads();
  }
  return prefix;
}

template <bool BF16>
__global__ void __launch_bounds__(kThreads) sample_kernel(const void* logits, int64_t* ids, const float* temperature,
                                                           const int32_t* top_k, const float* top_p,
                                                           const float* uniforms, uint64_t seed, uint64_t step,
                                                           int vocab, int64_t row_stride) {
  ptx::grid_dep_sync();
  __shared__ ArgMax scratch[33];
  __shared__ float fscratch[33];
  __shared__ float hist[(kWarps + 1) * 256];
  __shared__ float bcast[2];
  __shared__ float sums[kThreads];
  const int row = blockIdx.x;
  const void* base = static_cast<const char*>(logits) + static_cast<int64_t>(row) * row_stride * (BF16 ? 2 : 4);
  const float temp = temperature != nullptr ? temperature[row] : 1.0f;
  const ArgMax best = block_argmax<BF16>(base, vocab, scratch);
  if (temp <= 0.0f) {
    if (threadIdx.x == 0) ids[row] = best.i;
    return;
  }
  const float mx = best.v;
  const float inv_t = ptx::kLog2e / temp;  // exp((x - mx)/T) = 2^((x - mx) * log2e / T)
  const int k = top_k != nullptr ? top_k[row] : 0;
  const float pp = top_p != nullptr ? top_p[row] : 1.0f;

  uint32_t floor_key = 0;
  if (k > 0 && k < vocab)
    floor_key = radix_select<BF16, false>(base, vocab, static_cast<float>(k), 0u, mx, inv_t, hist, bcast);
  if (pp < 1.0f) {
    float z = 0.0f;
    for_each_logit<BF16>(base, vocab, [&](float x, int) {
      if (float_key(x) >= floor_key) z += ptx::ex2((x - mx) * inv_t);
    });
    z = block_sum(z, fscratch);
    const uint32_t pkey = radix_select<BF16, true>(base, vocab, pp * z, floor_key, mx, inv_t, hist, bcast);
    floor_key = max(floor_key, pkey);
  }
  // inverse-CDF draw in index order over the kept set
  const int chunk = (vocab + blockDim.x - 1) / blockDim.x;
  const int i0 = threadIdx.x * chunk, i1 = min(vocab, i0 + chunk);
  float local = 0.0f;
  for (int i = i0; i < i1; ++i) {
    const float x = load_logit<BF16>(base, i);
    if (float_key(x) >= floor_key) local += ptx::ex2((x - mx) * inv_t);
  }
  sums[threadIdx.x] = local;
  __syncthreads();
  // inclusive scan (Hillis-Steele over 1024 entries)
  for (int o = 1; o < kThreads; o <<= 1) {
    const float add = threadIdx.x >= o ? sums[threadIdx.x - o] : 0.0f;
    __syncthreads();
    sums[threadIdx.x] += add;
    __syncthreads();
  }
  const float total = sums[kThreads - 1];
  const float u = uniforms != nullptr ? uniforms[row] : philox_uniform(seed, step, static_cast<uint32_t>(row));
  const float target = u * total;
  const float before = threadIdx.x > 0 ? sums[threadIdx.x - 1] : 0.0f;
  const float after = sums[threadIdx.x];
  if (threadIdx.x == 0) bcast[0] = __int_as_float(-1);
  __syncthreads();
  if (local > 0.0f && before <= target && target < after) {
    float acc = before;
    int pick = -1;
    for (int i = i0; i < i1; ++i) {
      const float x = load_logit<BF16>(base, i);
      if (float_key(x) >= floor_key) {
        acc += ptx::ex2((x - mx) * inv_t);
        pick = i;
        if (acc > target) break;
      }
    }
    bcast[0] = __int_as_float(pick);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const int pick = __float_as_int(bcast[0]);
    ids[row] = pick >= 0 ? pick : best.i;  // rounding fell off the end: the mode is always in the kept set
  }
}

}  // namespace
}  // namespace b2

using namespace b2;

extern "C" int b2_argmax(const void* logits, int is_bf16, int64_t* ids, float* max_out, int rows, int vocab,
                         int64_t row_stride, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0) return -kBadArgument;
  if (is_bf16) launch_pdl(argmax_kernel<true>, dim3(rows), dim3(kThreads), 0, stream, logits, ids, max_out, vocab, row_stride);
  else launch_pdl(argmax_kernel<false>, dim3(rows), dim3(kThreads), 0, stream, logits, ids, max_out, vocab, row_stride);
  return last_launch_rc();
}

extern "C" int b2_sample(const void* logits, int is_bf16, int64_t* ids, const float* temperature, const int32_t* top_k,
                         const float* top_p, const float* uniforms, uint64_t seed, uint64_t step, int rows, int vocab,
                         int64_t row_stride, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0) return -kBadArgument;
  if (is_bf16)
    launch_pdl(sample_kernel<true>, dim3(rows), dim3(kThreads), 0, stream, logits, ids, temperature, top_k, top_p, uniforms, seed, step,
                                                       vocab, row_stride);
  else
    launch_pdl(sample_kernel<false>, dim3(rows), dim3(kThreads), 0, stream, logits, ids, temperature, top_k, top_p, uniforms, seed, step,
                                                        vocab, row_stride);
  return last_launch_rc();
}
