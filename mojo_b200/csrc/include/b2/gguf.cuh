// GGUF k-quant block formats (Q4_K, Q6_K) and their dequantisation, shared by the standalone dequant kernel and
// the dequant-fused GEMM. Super-blocks cover 256 weights along K and are 144 / 210 bytes long. A Q6_K block is not
// a multiple of 4 bytes, so wide loads on it are the unaligned-access hazard the reference works around with
// byte-wise loads (stdlib/src/memory/unsafe_pointer.mojo:503-531): the generic routines below read bytes, and the
// `*_dequant64` routines used on the hot paths read what the alignment allows, 16 bytes at a time for Q4_K
// (144 = 9 x 16, so every block of a 16-byte-aligned tensor is 16-byte aligned) and 2 bytes at a time for Q6_K.
// Measured on the 16 x 28672 x 4096 fused GEMM: byte loads put 65 L1 sectors behind every DRAM sector (753 us);
// the wide loads bring the kernel down to the dequantisation arithmetic.
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
// ---- 64 weights (two adjacent 32-weight groups g0, g0 + 1, g0 even) with the widest loads the format allows ----

// Byte i (0..11) of the 12 packed scale bytes held in three 32-bit words.
__device__ __forceinline__ int q4k_sc_byte(const uint32_t (&w)[3], int i) { return (w[i >> 2] >> ((i & 3) * 8)) & 0xFF; }

__device__ __forceinline__ void q4k_scale_min_w(const uint32_t (&w)[3], int j, int& scale, int& mn) {
  if (j < 4) {
    scale = q4k_sc_byte(w, j) & 63;
    mn = q4k_sc_byte(w, j + 4) & 63;
  } else {
    scale = (q4k_sc_byte(w, j + 4) & 0xF) | ((q4k_sc_byte(w, j - 4) >> 6) << 4);
    mn = (q4k_sc_byte(w, j + 4) >> 4) | ((q4k_sc_byte(w, j) >> 6) << 4);
  }
}

// Small non-negative integer -> float without a conversion instruction (2^23 + q has q in its low mantissa bits).
__device__ __forceinline__ float small_uint_to_float(uint32_t q) { return __uint_as_float(0x4B000000u | q) - 8388608.0f; }

// `blk` must be 16-byte aligned. out[0..31] = sub-block g0, out[32..63] = sub-block g0 + 1 (they share 32 quant bytes:
// low nibbles, then high nibbles). Three 16-byte loads.
__device__ __forceinline__ void q4k_dequant64(const uint8_t* blk, int g0, float* out) {
  const uint4 hdr = *reinterpret_cast<const uint4*>(blk);
  const float d = __half2float(__ushort_as_half(static_cast<uint16_t>(hdr.x & 0xFFFF)));
  const float dmin = __half2float(__ushort_as_half(static_cast<uint16_t>(hdr.x >> 16)));
  const uint32_t scw[3] = {hdr.y, hdr.z, hdr.w};
  int sc0, mn0, sc1, mn1;
  q4k_scale_min_w(scw, g0, sc0, mn0);
  q4k_scale_min_w(scw, g0 + 1, sc1, mn1);
  const float a0 = d * sc0, b0 = dmin * mn0, a1 = d * sc1, b1 = dmin * mn1;
  const uint4* qp = reinterpret_cast<const uint4*>(blk + 16 + (g0 >> 1) * 32);
  const uint4 qa = qp[0], qb = qp[1];
  const uint32_t q[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
  for (int w = 0; w < 8; ++w) {
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const uint32_t byte = (q[w] >> (8 * b)) & 0xFFu;
      out[w * 4 + b] = fmaf(a0, small_uint_to_float(byte & 0xFu), -b0);
      out[32 + w * 4 + b] = fmaf(a1, small_uint_to_float(byte >> 4), -b1);
    }
  }
}

// Q6_K blocks are only 2-byte aligned: 16-bit loads (51 of them for 64 weights instead of 136 byte loads).
__device__ __forceinline__ void q6k_dequant64(const uint8_t* blk, int g0, float* out) {
  const uint16_t* h = reinterpret_cast<const uint16_t*>(blk);
  const float d = __half2float(__ushort_as_half(h[104]));          // byte 208
  const int half = g0 >> 2, quarter = g0 & 3;                      // quarter is 0 or 2
  const uint16_t* ql = h + half * 32;                              // 64 bytes: quarter-even group, then quarter-odd group
  const uint16_t* qh = h + 64 + half * 16;                         // 32 bytes shared by the four groups of this half
  const uint16_t s01 = h[96 + half * 4 + quarter], s23 = h[96 + half * 4 + quarter + 1];   // four int8 scales
  const float sc[4] = {d * static_cast<int8_t>(s01 & 0xFF), d * static_cast<int8_t>(s01 >> 8), d * static_cast<int8_t>(s23 & 0xFF),
                       d * static_cast<int8_t>(s23 >> 8)};
  const int ql_shift = (quarter >> 1) * 4, qh_shift = quarter * 2;
#pragma unroll
  for (int l2 = 0; l2 < 16; ++l2) {
    const uint32_t lo0 = ql[l2], lo1 = ql[16 + l2], hi = qh[l2];
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      const int l = l2 * 2 + b;
      const uint32_t a = (lo0 >> (8 * b)) & 0xFFu, c = (lo1 >> (8 * b)) & 0xFFu, hb = (hi >> (8 * b)) & 0xFFu;
      const int q0 = static_cast<int>(((a >> ql_shift) & 0xFu) | (((hb >> qh_shift) & 3u) << 4)) - 32;
      const int q1 = static_cast<int>(((c >> ql_shift) & 0xFu) | (((hb >> (qh_shift + 2)) & 3u) << 4)) - 32;
      out[l] = sc[l >> 4] * static_cast<float>(q0);
      out[32 + l] = sc[2 + (l >> 4)] * static_cast<float>(q1);
    }
  }
}
#endif

}  // namespace gguf
}  // namespace b2
