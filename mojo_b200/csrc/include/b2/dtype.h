// Runtime dtype enum, sizes and host-side bit-exact conversions.
//
// Counterpart of the reference's `DType` (stdlib/src/builtin/dtype.mojo:30-147, predicates :394-506,
// sizeof :508-569, runtime dispatch :571-706), cut down to what an inference engine moves around.
// The software fp8/bf16 converts restate the numerics spec of stdlib/src/builtin/simd.mojo:3101-3158
// (e4m3/e5m2 -> f32 incl. subnormals/NaN) and :3230-3321 (f32 -> bf16 round-to-nearest-even with the
// 0x7FFF + lsb bias, NaN kept quiet); they are the CPU oracle for the device `cvt` instructions.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>

namespace b2 {

enum class DType : int32_t {
  kInvalid = 0,
  kBool,
  kU8,
  kI8,
  kI32,
  kI64,
  kF16,
  kBF16,
  kF32,
  kF64,
  kE4M3,   // float8 e4m3fn: no inf, NaN = S.1111.111, max 448
  kE5M2,   // float8 e5m2: IEEE-like, inf and NaN
  kUE8M0,  // power-of-two scale byte
};

constexpr int dtype_size(DType d) {
  switch (d) {
    case DType::kBool: case DType::kU8: case DType::kI8: case DType::kE4M3: case DType::kE5M2: case DType::kUE8M0: return 1;
    case DType::kF16: case DType::kBF16: return 2;
    case DType::kI32: case DType::kF32: return 4;
    case DType::kI64: case DType::kF64: return 8;
    default: return 0;
  }
}
constexpr bool dtype_is_float8(DType d) { return d == DType::kE4M3 || d == DType::kE5M2; }
constexpr bool dtype_is_half(DType d) { return d == DType::kF16 || d == DType::kBF16; }
constexpr bool dtype_is_floating(DType d) {
  return dtype_is_float8(d) || dtype_is_half(d) || d == DType::kF32 || d == DType::kF64;
}
// Half and fp8 types accumulate in f32 (the reference's get_accum_type rule,
// stdlib/src/utils/numerics.mojo:1031-1054).
constexpr DType dtype_accum(DType d) {
  return (dtype_is_float8(d) || dtype_is_half(d)) ? DType::kF32 : d;
}
inline const char* dtype_name(DType d) {
  switch (d) {
    case DType::kBool: return "bool"; case DType::kU8: return "uint8"; case DType::kI8: return "int8";
    case DType::kI32: return "int32"; case DType::kI64: return "int64"; case DType::kF16: return "float16";
    case DType::kBF16: return "bfloat16"; case DType::kF32: return "float32"; case DType::kF64: return "float64";
    case DType::kE4M3: return "float8_e4m3fn"; case DType::kE5M2: return "float8_e5m2"; case DType::kUE8M0: return "ue8m0";
    default: return "invalid";
  }
}

// ---- host-side bit-exact conversions (oracle) -------------------------------------------------
inline uint16_t f32_to_bf16_bits(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x0040u);  // quiet NaN, sign kept
  const uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return static_cast<uint16_t>(u >> 16);
}
inline float bf16_bits_to_f32(uint16_t h) {
  uint32_t u = static_cast<uint32_t>(h) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
inline float e4m3_bits_to_f32(uint8_t v) {
  const int sign = v >> 7, exp = (v >> 3) & 0xf, man = v & 0x7;
  float r;
  if (exp == 0xf && man == 0x7) r = std::nanf("");
  else if (exp == 0) r = std::ldexp(static_cast<float>(man), -9);  // subnormal: man * 2^-3 * 2^-6
  else r = std::ldexp(1.0f + man / 8.0f, exp - 7);
  return sign ? -r : r;
}
inline float e5m2_bits_to_f32(uint8_t v) {
  const int sign = v >> 7, exp = (v >> 2) & 0x1f, man = v & 0x3;
  float r;
  if (exp == 0x1f) r = man ? std::nanf("") : INFINITY;
  else if (exp == 0) r = std::ldexp(static_cast<float>(man), -16);
  else r = std::ldexp(1.0f + man / 4.0f, exp - 15);
  return sign ? -r : r;
}
// f32 -> e4m3fn, round to nearest even, saturating to +-448 (the `satfinite` convert).
inline uint8_t f32_to_e4m3_bits(float f) {
  if (std::isnan(f)) return 0x7f;
  const uint8_t sign = std::signbit(f) ? 0x80 : 0;
  float a = std::fabs(f);
  if (a >= 448.0f) return sign | 0x7e;
  if (a < std::ldexp(1.0f, -10)) return sign;  // below half of the smallest subnormal
  int e;
  std::frexp(a, &e);  // a = m * 2^e, m in [0.5, 1)
  int exp = e - 1;    // a = 1.x * 2^exp
  if (exp < -6) exp = -6;
  const float q = std::ldexp(a, 3 - exp);  // mantissa in units of 2^(exp-3)
  float r = std::nearbyint(q);              // RNE under the default rounding mode
  int ir = static_cast<int>(r);
  int biased = exp + 7;
  if (exp == -6 && ir < 8) return sign | static_cast<uint8_t>(ir);  // subnormal
  if (ir == 16) { ir = 8; biased += 1; }
  if (biased > 15 || (biased == 15 && (ir - 8) == 7)) return sign | 0x7e;
  return sign | static_cast<uint8_t>((biased << 3) | (ir - 8));
}

}  // namespace b2
