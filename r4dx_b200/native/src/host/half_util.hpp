// Host-side fp16 / bf16 / fp8-e4m3 conversions (round to nearest even), bit exact with the device.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>
#include <immintrin.h>

namespace r4dxb {

inline uint16_t FloatToF16(float x) { return static_cast<uint16_t>(_cvtss_sh(x, _MM_FROUND_TO_NEAREST_INT)); }
inline float F16ToFloat(uint16_t h) { return _cvtsh_ss(h); }

inline uint16_t FloatToBf16(float x) {
  uint32_t u;
  std::memcpy(&u, &x, 4);
  if ((u & 0x7F800000u) == 0x7F800000u && (u & 0x007FFFFFu)) return static_cast<uint16_t>((u >> 16) | 0x40);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return static_cast<uint16_t>(u >> 16);
}
inline float Bf16ToFloat(uint16_t b) {
  uint32_t u = static_cast<uint32_t>(b) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

// fp8 e4m3fn: 1-4-3, bias 7, no inf, max 448, NaN = 0x7F.
inline float Fp8E4m3ToFloat(uint8_t v) {
  const int s = v >> 7, e = (v >> 3) & 0xF, m = v & 7;
  float f;
  if (e == 0xF && m == 7) f = NAN;
  else if (e == 0) f = std::ldexp(static_cast<float>(m), -9);
  else f = std::ldexp(1.0f + m / 8.0f, e - 7);
  return s ? -f : f;
}
inline uint8_t FloatToFp8E4m3(float x) {
  if (std::isnan(x)) return 0x7F;
  const uint8_t s = std::signbit(x) ? 0x80 : 0;
  float a = std::fabs(x);
  if (a >= 464.0f) return s | 0x7E;   // saturate (448 is the largest finite; ties above round down to it)
  if (a < std::ldexp(1.0f, -10)) return s;  // below half of the smallest subnormal
  int e;
  float fr = std::frexp(a, &e);  // a = fr * 2^e, fr in [0.5, 1)
  int E = e - 1 + 7;             // biased exponent for 1.m form
  float q;
  if (E <= 0) {                  // subnormal: units of 2^-9
    q = std::nearbyint(std::ldexp(a, 9));
    if (q >= 8.0f) return s | 0x08;
    return s | static_cast<uint8_t>(q);
  }
  q = std::nearbyint(std::ldexp(fr, 4));  // 1.mmm * 8 in [8, 16]
  if (q >= 16.0f) { q = 8.0f; ++E; }
  if (E >= 16 || (E == 15 && q - 8.0f >= 7.0f)) return s | 0x7E;
  return s | static_cast<uint8_t>((E << 3) | static_cast<int>(q - 8.0f));
}

}  // namespace r4dxb
