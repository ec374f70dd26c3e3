// w4a16: asymmetric 4-bit weights per (row, group of 32 or 64 along K), fp16 activations.
//
//   w ~= scale * (q - zero),  q in 0..15
//
// Layout (this engine's own; the reference pre-permutes into its WMMA fragment order instead,
// reference: docs/container-format.md:146-170):
//   wq  [N][K/8]  u32: nibble i (bits 4i..4i+3) of word j is q for k = 8 j + i.
//   wsz [N][K/g]  u32: low half = fp16 scale, high half = fp16 of -(1024 + zero).
// The second half lets a kernel turn a nibble n into fp16 (0x6400 | n) = 1024 + n and add
// -(1024 + zero) exactly, then scale the fp32 accumulator once per group.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <vector>

#include "half_util.hpp"

namespace r4dxb {

void W4a16Quantize(const float* W, int64_t N, int64_t K, int group, uint32_t* wq, uint32_t* wsz) {
  const int64_t groups = K / group;
  for (int64_t n = 0; n < N; ++n) {
    for (int64_t g = 0; g < groups; ++g) {
      const float* w = W + n * K + g * group;
      float lo = w[0], hi = w[0];
      for (int i = 1; i < group; ++i) { lo = std::min(lo, w[i]); hi = std::max(hi, w[i]); }
      lo = std::min(lo, 0.0f);
      hi = std::max(hi, 0.0f);
      float scale = (hi - lo) / 15.0f;
      if (scale <= 0) scale = 1.0f;
      scale = F16ToFloat(FloatToF16(scale));
      if (scale <= 0) scale = F16ToFloat(1);  // smallest subnormal
      int zero = static_cast<int>(std::nearbyint(-lo / scale));
      zero = std::min(15, std::max(0, zero));
      wsz[n * groups + g] = static_cast<uint32_t>(FloatToF16(scale)) |
                            (static_cast<uint32_t>(FloatToF16(-(1024.0f + zero))) << 16);
      for (int i = 0; i < group; ++i) {
        int q = static_cast<int>(std::nearbyint(w[i] / scale)) + zero;
        q = std::min(15, std::max(0, q));
        const int64_t k = g * group + i;
        uint32_t& word = wq[n * (K / 8) + k / 8];
        const int sh = 4 * static_cast<int>(k % 8);
        word = (word & ~(0xFu << sh)) | (static_cast<uint32_t>(q) << sh);
      }
    }
  }
}

void W4a16Dequantize(const uint32_t* wq, const uint32_t* wsz, int64_t N, int64_t K, int group, float* W) {
  const int64_t groups = K / group;
  for (int64_t n = 0; n < N; ++n)
    for (int64_t k = 0; k < K; ++k) {
      const uint32_t sz = wsz[n * groups + k / group];
      const float scale = F16ToFloat(static_cast<uint16_t>(sz & 0xFFFF));
      const float nz = F16ToFloat(static_cast<uint16_t>(sz >> 16));  // -(1024 + zero)
      const uint32_t q = (wq[n * (K / 8) + k / 8] >> (4 * (k % 8))) & 0xF;
      W[n * K + k] = scale * ((1024.0f + q) + nz);
    }
}

// w8a16: symmetric int8 (offset binary: stored = q + 128) with one fp16 scale per (row, group).
void W8a16Quantize(const float* W, int64_t N, int64_t K, int group, uint8_t* wq, uint16_t* ws) {
  const int64_t groups = K / group;
  for (int64_t n = 0; n < N; ++n)
    for (int64_t g = 0; g < groups; ++g) {
      const float* w = W + n * K + g * group;
      float amax = 0;
      for (int i = 0; i < group; ++i) amax = std::max(amax, std::fabs(w[i]));
      float scale = amax / 127.0f;
      scale = F16ToFloat(FloatToF16(scale > 0 ? scale : 1.0f));
      if (scale <= 0) scale = F16ToFloat(1);
      ws[n * groups + g] = FloatToF16(scale);
      for (int i = 0; i < group; ++i) {
        int q = static_cast<int>(std::nearbyint(w[i] / scale));
        q = std::min(127, std::max(-127, q));
        wq[n * K + g * group + i] = static_cast<uint8_t>(q + 128);
      }
    }
}

void W8a16Dequantize(const uint8_t* wq, const uint16_t* ws, int64_t N, int64_t K, int group, float* W) {
  const int64_t groups = K / group;
  for (int64_t n = 0; n < N; ++n)
    for (int64_t k = 0; k < K; ++k)
      W[n * K + k] = F16ToFloat(ws[n * groups + k / group]) * (static_cast<int>(wq[n * K + k]) - 128);
}

}  // namespace r4dxb

extern "C" {

int r4dxb_w4a16_quantize(const float* W, int64_t N, int64_t K, int group, uint32_t* wq, uint32_t* wsz) {
  if ((group != 32 && group != 64 && group != 128) || K % group || K % 8) return -1;
  r4dxb::W4a16Quantize(W, N, K, group, wq, wsz);
  return 0;
}
int r4dxb_w4a16_dequantize(const uint32_t* wq, const uint32_t* wsz, int64_t N, int64_t K, int group, float* W) {
  if (K % group || K % 8) return -1;
  r4dxb::W4a16Dequantize(wq, wsz, N, K, group, W);
  return 0;
}
int r4dxb_w8a16_quantize(const float* W, int64_t N, int64_t K, int group, uint8_t* wq, uint16_t* ws) {
  if (K % group) return -1;
  r4dxb::W8a16Quantize(W, N, K, group, wq, ws);
  return 0;
}
int r4dxb_w8a16_dequantize(const uint8_t* wq, const uint16_t* ws, int64_t N, int64_t K, int group, float* W) {
  if (K % group) return -1;
  r4dxb::W8a16Dequantize(wq, ws, N, K, group, W);
  return 0;
}

}  // extern "C"
