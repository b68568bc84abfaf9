// Small register-vector helpers for memory-bound kernels.
//
// The reference's `SIMD[type, size]` (stdlib/src/builtin/simd.mojo:233-251; cast :1721-1824, reductions
// :2437-2740) is a general value type; device code here only needs the 16-byte global access width
// (`simdwidthof` analogue: 16 / sizeof(T), stdlib/src/sys/info.mojo:561-785) and f32 math on the lanes.
#pragma once
#include <cstdint>
#include <cuda_bf16.h>
#include "b2/ptx.cuh"

namespace b2 {

template <typename T>
struct VecWidth {
  static constexpr int value = 16 / sizeof(T);
};

// 8 bf16 <-> 8 f32
__device__ __forceinline__ void bf16x8_to_f32(const uint4& v, float (&f)[8]) {
  f[0] = ptx::bf16_lo(v.x); f[1] = ptx::bf16_hi(v.x);
  f[2] = ptx::bf16_lo(v.y); f[3] = ptx::bf16_hi(v.y);
  f[4] = ptx::bf16_lo(v.z); f[5] = ptx::bf16_hi(v.z);
  f[6] = ptx::bf16_lo(v.w); f[7] = ptx::bf16_hi(v.w);
}
__device__ __forceinline__ uint4 f32_to_bf16x8(const float (&f)[8]) {
  uint4 v;
  v.x = ptx::pack_bf16x2(f[0], f[1]);
  v.y = ptx::pack_bf16x2(f[2], f[3]);
  v.z = ptx::pack_bf16x2(f[4], f[5]);
  v.w = ptx::pack_bf16x2(f[6], f[7]);
  return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide sum; `scratch` holds at least 33 floats. Every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.0f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  const float r = scratch[32];
  __syncthreads();
  return r;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  const float r = scratch[32];
  __syncthreads();
  return r;
}

}  // namespace b2
