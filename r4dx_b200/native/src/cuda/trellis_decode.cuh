// Device-side trellis tile decode, shared by the T<=8 weight-streaming kernel and the tcgen05
// GEMM.  A lane decodes positions 8l .. 8l+7 of a 16x16 tile, i.e. 8 consecutive K values of
// output row n_local = l / 2 (k_local = 8 (l & 1) ..).  Format: r4dxb_trellis.h.
#pragma once
#include "common.cuh"
#include "r4dxb_trellis.h"

namespace r4dxb {

template <int KB>
struct TrellisLane {
  int i0, i1, i2;   // word indices of the lane's 64-bit window inside a tile (8*KB words)
  int off;          // bit offset of the window inside word i0

  __device__ __forceinline__ void Init(int lane) {
    constexpr int R = 256 * KB, NW = 8 * KB;
    int b0 = 8 * KB * (lane + 1) - 64;          // first stream bit of the window (ends at the lane's last state)
    if (b0 < 0) b0 += R;
    i0 = b0 >> 5;
    off = b0 & 31;
    i1 = (i0 + 1) % NW;
    i2 = (i0 + 2) % NW;
  }

  // words of one tile -> window (hi: stream bits [b0, b0+32), lo: the next 32)
  __device__ __forceinline__ void Window(uint32_t a, uint32_t b, uint32_t c, uint32_t& hi, uint32_t& lo) const {
    if constexpr (KB == 4) {   // off == 0 for every lane
      hi = a;
      lo = b;
    } else {
      hi = __funnelshift_l(b, a, off);
      lo = __funnelshift_l(c, b, off);
    }
  }
};

// Two code values from two 16-bit states: fp16x2( (1024 + bytesum(s * M)) * scale + bias ).
__device__ __forceinline__ __half2 TrellisCode2(uint32_t s0, uint32_t s1) {
  const uint32_t h0 = __dp4a(s0 * R4DXB_TRELLIS_MUL, 0x01010101u, 0x6400u);
  const uint32_t h1 = __dp4a(s1 * R4DXB_TRELLIS_MUL, 0x01010101u, 0x6400u);
  const uint32_t packed = __byte_perm(h0, h1, 0x5410);
  const __half2 scale = __halves2half2(__ushort_as_half(R4DXB_TRELLIS_SCALE_F16), __ushort_as_half(R4DXB_TRELLIS_SCALE_F16));
  const __half2 bias = __halves2half2(__ushort_as_half(R4DXB_TRELLIS_BIAS_F16), __ushort_as_half(R4DXB_TRELLIS_BIAS_F16));
  return __hfma2(*reinterpret_cast<const __half2*>(&packed), scale, bias);
}

// state of the lane's j-th position from its window
template <int KB, int J>
__device__ __forceinline__ uint32_t TrellisStateFromWindow(uint32_t hi, uint32_t lo) {
  constexpr int sh = KB * (7 - J);
  if constexpr (sh == 0) return lo & 0xFFFFu;
  else if constexpr (sh + 16 <= 32) return (lo >> sh) & 0xFFFFu;
  else if constexpr (sh < 32) return __funnelshift_r(lo, hi, sh) & 0xFFFFu;
  else return (hi >> (sh - 32)) & 0xFFFFu;
}

// 8 consecutive-K code values of the lane, as 4 x half2 (k, k+1 pairs).
template <int KB>
__device__ __forceinline__ void TrellisDecode8(uint32_t hi, uint32_t lo, __half2 (&w)[4]) {
  if constexpr (KB == 4) {
    // States sit on nibble boundaries: with the window also shifted by 4, 16 and 20 bits every state is two
    // whole bytes of some 32-bit word and one byte permute against a zero register extracts it
    // (11 instructions for 8 states instead of 15 shifts and masks).
    const uint32_t z = __funnelshift_r(lo, hi, 4), y = __funnelshift_r(lo, hi, 16), u = __funnelshift_r(lo, hi, 20);
    w[3] = TrellisCode2(__byte_perm(z, 0u, 0x4410), __byte_perm(lo, 0u, 0x4410));     // shifts 4, 0
    w[2] = TrellisCode2(__byte_perm(z, 0u, 0x4421), __byte_perm(lo, 0u, 0x4421));     // shifts 12, 8
    w[1] = TrellisCode2(__byte_perm(u, 0u, 0x4410), __byte_perm(y, 0u, 0x4410));      // shifts 20, 16
    w[0] = TrellisCode2(__byte_perm(u, 0u, 0x4421), __byte_perm(y, 0u, 0x4421));      // shifts 28, 24
    return;
  }
  w[0] = TrellisCode2(TrellisStateFromWindow<KB, 0>(hi, lo), TrellisStateFromWindow<KB, 1>(hi, lo));
  w[1] = TrellisCode2(TrellisStateFromWindow<KB, 2>(hi, lo), TrellisStateFromWindow<KB, 3>(hi, lo));
  w[2] = TrellisCode2(TrellisStateFromWindow<KB, 4>(hi, lo), TrellisStateFromWindow<KB, 5>(hi, lo));
  w[3] = TrellisCode2(TrellisStateFromWindow<KB, 6>(hi, lo), TrellisStateFromWindow<KB, 7>(hi, lo));
}

}  // namespace r4dxb
