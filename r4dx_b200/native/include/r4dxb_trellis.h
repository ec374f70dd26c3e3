// Trellis-coded weight format: definitions shared by host C++, CUDA kernels and tests.
//
// A linear y = W x with W [N, K] is stored as
//     y = svh (.) H_N( Q . H_K( suh (.) x ) )
// where H is the block-diagonal 128-point Sylvester Hadamard / sqrt(128), suh [K] and svh [N] are
// fp16 sign/scale vectors and Q [N, K] is a matrix of fp16 code values decoded from a bit trellis.
//
// Bit-exact decode definition (same as the reference engine's "mul1" code,
// reference: tests/kernels/trellis_ref.hpp:40-70, docs/container-format.md:538-556):
//   * a tile is 16 x 16 = 256 values coded by a tail-biting ring of 256*KB bits held in 8*KB u32
//     words; stream bit 32w is bit 31 of word w (MSB first);
//   * the state of position p is the 16 ring bits ending at bit KB*(p+1) (wrapping);
//   * value(s) = fp16( (1024 + bytesum((s * 0x83DCD12D) mod 2^32)) * fp16(0x1EEE) + fp16(0xC931) ),
//     one rounding; 1024 + bytesum is exact in fp16, so the value equals one fp16 FMA.
//   * KB in {3, 4, 5} bits per weight.
//
// Tile order (this engine's own, chosen for sm_100a): position p of a tile is element
// (n_local = p / 16, k_local = p % 16), so a lane that decodes 8 consecutive positions produces
// 8 consecutive K values of one output row = one 16-byte chunk of a K-major UMMA operand.
// Word order: [N/128][K/16][8][8*KB]; the tile (nb, tk, j) covers rows nb*128 + 16 j .. +15 and
// columns 16 tk .. +15.  A 128-row block's K range is therefore one contiguous byte run, which
// is what both the bulk-copy pipeline and the tensor-parallel K split rely on.
#pragma once
#include <stdint.h>

#define R4DXB_TRELLIS_MUL 0x83DCD12Du
#define R4DXB_TRELLIS_SCALE_F16 0x1EEEu
#define R4DXB_TRELLIS_BIAS_F16 0xC931u

#ifdef __cplusplus
namespace r4dxb {

// Words per tile.
constexpr int TrellisTileWords(int kb) { return 8 * kb; }

// Index of word 0 of tile (n-tile tn, k-tile tk) in the packed tensor.
inline int64_t TrellisTileWordIndex(int64_t K, int kb, int64_t tn, int64_t tk) {
  const int64_t nb = tn >> 3, j = tn & 7;
  return ((nb * (K / 16) + tk) * 8 + j) * TrellisTileWords(kb);
}

inline int64_t TrellisPackedWords(int64_t N, int64_t K, int kb) {
  return (N / 16) * (K / 16) * TrellisTileWords(kb);
}

}  // namespace r4dxb
#endif
