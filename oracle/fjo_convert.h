/*
 * f32 <-> f16 / bf16 conversions with the semantics of the `half` crate 2.7.1 that
 * crates/forja-cpu/src/lib.rs:1790-1847 (`decode` / `encode`) relies on: round to nearest, ties
 * to even; NaN stays NaN (quiet bit forced); overflow rounds to infinity; f16 subnormals are
 * produced exactly. Test infrastructure only (part of the CPU oracle).
 */
#ifndef FJO_CONVERT_H
#define FJO_CONVERT_H

#include <cstdint>
#include <cstring>

namespace fjo {

inline uint32_t f32_bits(float v) { uint32_t b; std::memcpy(&b, &v, 4); return b; }
inline float bits_f32(uint32_t b) { float v; std::memcpy(&v, &b, 4); return v; }

inline uint16_t f32_to_bf16(float value) {
  uint32_t x = f32_bits(value);
  if ((x & 0x7FFFFFFFu) > 0x7F800000u) return static_cast<uint16_t>((x >> 16) | 0x0040u);
  const uint32_t round_bit = 0x00008000u;
  if ((x & round_bit) != 0 && (x & (3 * round_bit - 1)) != 0) return static_cast<uint16_t>((x >> 16) + 1);
  return static_cast<uint16_t>(x >> 16);
}
inline float bf16_to_f32(uint16_t h) {
  if ((h & 0x7FFFu) > 0x7F80u) return bits_f32((static_cast<uint32_t>(h) | 0x0040u) << 16);
  return bits_f32(static_cast<uint32_t>(h) << 16);
}

inline uint16_t f32_to_f16(float value) {
  uint32_t x = f32_bits(value);
  uint32_t sign = x & 0x80000000u;
  uint32_t exp = x & 0x7F800000u;
  uint32_t man = x & 0x007FFFFFu;
  if (exp == 0x7F800000u) {
    uint32_t nan_bit = man == 0 ? 0 : 0x0200u;
    return static_cast<uint16_t>((sign >> 16) | 0x7C00u | nan_bit | (man >> 13));
  }
  uint32_t half_sign = sign >> 16;
  int32_t unbiased = static_cast<int32_t>(exp >> 23) - 127;
  int32_t half_exp = unbiased + 15;
  if (half_exp >= 0x1F) return static_cast<uint16_t>(half_sign | 0x7C00u);
  if (half_exp <= 0) {
    if (14 - half_exp > 24) return static_cast<uint16_t>(half_sign);
    uint32_t m = man | 0x00800000u;
    uint32_t half_man = m >> (14 - half_exp);
    uint32_t round_bit = 1u << (13 - half_exp);
    if ((m & round_bit) != 0 && (m & (3 * round_bit - 1)) != 0) half_man += 1;
    return static_cast<uint16_t>(half_sign | half_man);
  }
  uint32_t he = static_cast<uint32_t>(half_exp) << 10;
  uint32_t hm = man >> 13;
  const uint32_t round_bit = 0x00001000u;
  if ((man & round_bit) != 0 && (man & (3 * round_bit - 1)) != 0) return static_cast<uint16_t>((half_sign | he | hm) + 1);
  return static_cast<uint16_t>(half_sign | he | hm);
}
inline float f16_to_f32(uint16_t h) {
  if ((h & 0x7FFFu) == 0) return bits_f32(static_cast<uint32_t>(h) << 16);
  uint32_t sign = static_cast<uint32_t>(h & 0x8000u) << 16;
  uint32_t exp = h & 0x7C00u;
  uint32_t man = h & 0x03FFu;
  if (exp == 0x7C00u) {
    if (man == 0) return bits_f32(sign | 0x7F800000u);
    return bits_f32(sign | 0x7FC00000u | (man << 13));
  }
  if (exp == 0) {
    // subnormal: normalise
    int e = 0;
    while ((man & 0x0400u) == 0) { man <<= 1; ++e; }
    man &= 0x03FFu;
    uint32_t fexp = static_cast<uint32_t>(127 - 15 - e + 1) << 23;
    return bits_f32(sign | fexp | (man << 13));
  }
  uint32_t fexp = ((exp >> 10) + (127 - 15)) << 23;
  return bits_f32(sign | fexp | (man << 13));
}

}  // namespace fjo
#endif
