// Host-side fp16 / bf16 conversions (round to nearest even), used for scalar encoding and by the
// Float16 / BFloat16 holders.  Same contract as the reference's encoders (src/dvm.cc:64-186): fp16 NaN
// maps to 0x7e00, bf16 NaN to 0x7fc0.
#ifndef DVM_B200_NUMERIC_H_
#define DVM_B200_NUMERIC_H_

#include <cstdint>
#include <cstring>

namespace dvm {

inline uint32_t FloatBits(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  return u;
}
inline float BitsFloat(uint32_t u) {
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

inline uint16_t F32ToF16Bits(float f) {
  const uint32_t x = FloatBits(f);
  const uint16_t sign = static_cast<uint16_t>((x >> 16) & 0x8000u);
  const uint32_t mag = x & 0x7fffffffu;
  if (mag > 0x7f800000u) return sign | 0x7e00u;
  if (mag >= 0x47800000u) return sign | 0x7c00u;   // >= 65536 (or inf)
  const int32_t e = static_cast<int32_t>(mag >> 23) - 127 + 15;
  uint32_t m = mag & 0x7fffffu;
  if (e <= 0) {
    if (e < -10) return sign;
    m |= 0x800000u;
    const int shift = 14 - e;   // 14..24
    uint32_t h = m >> shift;
    const uint32_t rem = m & ((1u << shift) - 1u), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (h & 1u))) ++h;
    return sign | static_cast<uint16_t>(h);
  }
  uint32_t h = (static_cast<uint32_t>(e) << 10) | (m >> 13);
  const uint32_t rem = m & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) ++h;   // a carry may reach the exponent, up to inf
  return sign | static_cast<uint16_t>(h);
}

inline float F16BitsToF32(uint16_t h) {
  const uint32_t sign = static_cast<uint32_t>(h & 0x8000u) << 16;
  const uint32_t e = (h >> 10) & 0x1fu;
  uint32_t m = h & 0x3ffu;
  if (e == 0x1fu) return BitsFloat(sign | 0x7f800000u | (m << 13));
  if (e == 0) {
    if (m == 0) return BitsFloat(sign);
    int shift = 0;
    while (!(m & 0x400u)) {
      m <<= 1;
      ++shift;
    }
    m &= 0x3ffu;
    return BitsFloat(sign | (static_cast<uint32_t>(113 - shift) << 23) | (m << 13));
  }
  return BitsFloat(sign | ((e + 112u) << 23) | (m << 13));
}

inline uint16_t F32ToBF16Bits(float f) {
  uint32_t x = FloatBits(f);
  if ((x & 0x7fffffffu) > 0x7f800000u) return 0x7fc0u;
  x += 0x7fffu + ((x >> 16) & 1u);
  return static_cast<uint16_t>(x >> 16);
}

inline float BF16BitsToF32(uint16_t h) { return BitsFloat(static_cast<uint32_t>(h) << 16); }

}  // namespace dvm

#endif  // DVM_B200_NUMERIC_H_
