// GGUF k-quant block formats (Q4_K, Q6_K) and their dequantisation, shared by the standalone dequant kernel and
// the dequant-fused GEMM. Super-blocks cover 256 weights along K and are 144 / 210 bytes long - not multiples
// of 16 - so everything here goes through byte / 16-bit loads; wider loads on such addresses are the unaligned
// access hazard the reference works around with byte-wise loads (stdlib/src/memory/unsafe_pointer.mojo:503-531).
#pragma once
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace b2 {
namespace gguf {

constexpr int kQK = 256;          // weights per super-block
constexpr int kQ4KBytes = 144;    // f16 d, f16 dmin, 12 B packed 6-bit scales/mins, 128 B nibbles
constexpr int kQ6KBytes = 210;    // 128 B ql, 64 B qh, 16 x i8 scales, f16 d
constexpr int kTypeQ4K = 12;      // ggml type ids
constexpr int kTypeQ6K = 14;

__host__ __device__ inline int block_bytes(int ggml_type) {
  return ggml_type == kTypeQ4K ? kQ4KBytes : ggml_type == kTypeQ6K ? kQ6KBytes : 0;
}

#if defined(__CUDACC__)
__device__ __forceinline__ float half_at(const uint8_t* p) {
  const uint16_t bits = static_cast<uint16_t>(p[0]) | (static_cast<uint16_t>(p[1]) << 8);
  return __half2float(__ushort_as_half(bits));
}

// 6-bit scale and min of sub-block j (0..7) of a Q4_K super-block; `sc` points at its 12 packed bytes.
__device__ __forceinline__ void q4k_scale_min(const uint8_t* sc, int j, int& scale, int& mn) {
  if (j < 4) {
    scale = sc[j] & 63;
    mn = sc[j + 4] & 63;
  } else {
    scale = (sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4);
    mn = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4);
  }
}

// Dequantise the 32 weights of sub-block `j` (0..7) of a Q4_K super-block into out[0..31].
__device__ __forceinline__ void q4k_dequant32(const uint8_t* blk, int j, float* out) {
  const float d = half_at(blk), dmin = half_at(blk + 2);
  int sc, mn;
  q4k_scale_min(blk + 4, j, sc, mn);
  const float a = d * sc, b = dmin * mn;
  const uint8_t* qs = blk + 16 + (j >> 1) * 32;  // two sub-blocks share 32 bytes: low nibbles, then high nibbles
  const int shift = (j & 1) * 4;
#pragma unroll
  for (int l = 0; l < 32; ++l) out[l] = a * ((qs[l] >> shift) & 0xF) - b;
}

// Dequantise 32 consecutive weights [32 g, 32 g + 32) (g = 0..7) of a Q6_K super-block.
__device__ __forceinline__ void q6k_dequant32(const uint8_t* blk, int g, float* out) {
  const float d = half_at(blk + 208);
  const int half = g >> 2;       // which 128-weight half
  const int quarter = g & 3;     // 32-weight group inside the half
  const uint8_t* ql = blk + half * 64 + (quarter & 1) * 32;
  const uint8_t* qh = blk + 128 + half * 32;
  const int8_t* sc = reinterpret_cast<const int8_t*>(blk + 192) + half * 8 + quarter * 2;
  const int ql_shift = (quarter >> 1) * 4;
  const int qh_shift = quarter * 2;
#pragma unroll
  for (int l = 0; l < 32; ++l) {
    const int q = (((ql[l] >> ql_shift) & 0xF) | (((qh[l] >> qh_shift) & 3) << 4)) - 32;
    out[l] = d * sc[l >> 4] * q;
  }
}
#endif

}  // namespace gguf
}  // namespace b2
