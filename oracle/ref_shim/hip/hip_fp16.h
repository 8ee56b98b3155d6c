// The two half intrinsics the reference's device code names unconditionally
// (kv_load<F16>). The hardware conversion they stand for is exact, so an exact
// bit-level widening (Inf/NaN included) is the same function.
#pragma once
#include <cstdint>
#include <cstring>
struct rdshim_half {
  uint16_t bits;
};
inline rdshim_half __ushort_as_half(uint16_t u) { return rdshim_half{u}; }
inline float __half2float(rdshim_half h) {
  const uint32_t s = (uint32_t)(h.bits >> 15) << 31;
  const uint32_t e = (h.bits >> 10) & 0x1fu;
  uint32_t m = h.bits & 0x3ffu;
  uint32_t u;
  if (e == 0) {
    if (m == 0) {
      u = s;
    } else {  // subnormal: normalise
      int sh = 0;
      while (!(m & 0x400u)) {
        m <<= 1;
        ++sh;
      }
      u = s | ((uint32_t)(113 - sh) << 23) | ((m & 0x3ffu) << 13);
    }
  } else if (e == 31) {
    u = s | 0x7f800000u | (m << 13);
  } else {
    u = s | ((e + 112u) << 23) | (m << 13);
  }
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
