// Gated short convolution of the conv layers of the short-conv + attention MoE family.
//
// The layer's input projection yields three H-wide thirds per row, B | C | x.  With bx = B * x (one bf16
// rounding), the mixer is a causal depthwise FIR of L taps over bx, gated by C:
//     y[t, c] = C[t, c] * sum_{j < L} w[c, j] * bx[t - (L - 1) + j, c]
// (reference: src/kernels/include/r4dx/kernels/lfm2_kernels.h:14-34, the ShortConv entry points).
//
// State: the last rows of bx, kept in a ring of 32 rows keyed by ABSOLUTE position (slot = pos & 31), the same
// convention as the Gated DeltaNet conv ring.  A row always writes its own slot and reads the slots of earlier
// positions, so a speculative window that is only partly accepted needs no rollback: the rejected rows' slots
// are rewritten by the next call before anything reads them.
//
// Every (row, channel pair) is independent: taps that fall inside the call read the call's own bcx rows, taps
// before it read the ring.  While T + L - 1 <= 32 (every decode call and speculative window) the same kernel also
// writes the ring: reads touch the L - 1 slots before the call, writes the call's own T slots, all distinct.
// Longer calls (prefill chunks, always committed whole) would wrap onto the slots being read, so their ring
// update is a second, stream-ordered launch over the last 8 rows.
#include "common.cuh"

namespace r4dxb {
namespace {

constexpr int kRing = 32;
constexpr int kMaxTaps = 8;

__device__ __forceinline__ uint32_t MulBf16x2(uint32_t a, uint32_t b) {
  return PackBf16(BfLo(a) * BfLo(b), BfHi(a) * BfHi(b));
}

// grid (ceil(H / 2 / 128), T), block 128; one thread = two adjacent channels of one row
__global__ void ShortConvKernel(const __nv_bfloat16* __restrict__ bcx, const __nv_bfloat16* __restrict__ w,
                                __nv_bfloat16* __restrict__ ring, const int* __restrict__ positions,
                                __nv_bfloat16* __restrict__ out, int T, int H, int L, int write_ring) {
  PdlEnter();
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
  const int t = blockIdx.y;
  if (c >= H) return;
  const int pos0 = positions[0];
  float a0 = 0.f, a1 = 0.f;
  uint32_t own = 0;
  for (int j = 0; j < L; ++j) {
    const int s = t - (L - 1) + j;
    uint32_t bx;
    if (s >= 0) {
      const __nv_bfloat16* row = bcx + static_cast<size_t>(s) * 3 * H;
      bx = MulBf16x2(*reinterpret_cast<const uint32_t*>(row + c), *reinterpret_cast<const uint32_t*>(row + 2 * H + c));
    } else {
      const int p = pos0 + s;
      bx = p >= 0 ? *reinterpret_cast<const uint32_t*>(ring + static_cast<size_t>(p & (kRing - 1)) * H + c) : 0u;
    }
    a0 = fmaf(__bfloat162float(w[static_cast<size_t>(c) * L + j]), BfLo(bx), a0);
    a1 = fmaf(__bfloat162float(w[static_cast<size_t>(c + 1) * L + j]), BfHi(bx), a1);
    own = bx;                                  // the last tap is the row's own bx
  }
  const uint32_t g = *reinterpret_cast<const uint32_t*>(bcx + static_cast<size_t>(t) * 3 * H + H + c);
  *reinterpret_cast<uint32_t*>(out + static_cast<size_t>(t) * H + c) = PackBf16(a0 * BfLo(g), a1 * BfHi(g));
  if (write_ring)
    *reinterpret_cast<uint32_t*>(ring + static_cast<size_t>((pos0 + t) & (kRing - 1)) * H + c) = own;
}

// ring[(pos0 + t) & 31] = bx[t] for t in [t_begin, T); grid (ceil(H / 2 / 128), T - t_begin)
__global__ void ShortConvRingKernel(const __nv_bfloat16* __restrict__ bcx, __nv_bfloat16* __restrict__ ring,
                                    const int* __restrict__ positions, int t_begin, int H) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
  const int t = t_begin + blockIdx.y;
  if (c >= H) return;
  const __nv_bfloat16* row = bcx + static_cast<size_t>(t) * 3 * H;
  const uint32_t bx = MulBf16x2(*reinterpret_cast<const uint32_t*>(row + c), *reinterpret_cast<const uint32_t*>(row + 2 * H + c));
  *reinterpret_cast<uint32_t*>(ring + static_cast<size_t>((positions[0] + t) & (kRing - 1)) * H + c) = bx;
}

}  // namespace
}  // namespace r4dxb

using namespace r4dxb;

extern "C" {

/* bcx [T, 3H] bf16 (B | C | x), w [H, L] bf16, ring [32, H] bf16, positions[0] = absolute position of row 0,
 * out [T, H] bf16.  H even, 1 <= L <= 8. */
int r4dxb_short_conv(const void* bcx, const void* w, void* ring, const int* positions, void* out, int T, int H, int L,
                     void* stream) {
  if (T < 1 || T > 65535 || H < 2 || H % 2 || L < 1 || L > kMaxTaps) return R4DXB_BAD_ARG;
  auto s = static_cast<cudaStream_t>(stream);
  const dim3 grid((H / 2 + 127) / 128, T);
  const int single = T + L - 1 <= kRing;
  int rc = LaunchPdl(ShortConvKernel, grid, dim3(128), 0, s, static_cast<const __nv_bfloat16*>(bcx),
                     static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(ring), positions,
                     static_cast<__nv_bfloat16*>(out), T, H, L, single);
  if (rc != 0 || single) return rc;
  const int t_begin = T - 8;
  ShortConvRingKernel<<<dim3((H / 2 + 127) / 128, 8), 128, 0, s>>>(static_cast<const __nv_bfloat16*>(bcx),
                                                                  static_cast<__nv_bfloat16*>(ring), positions, t_begin, H);
  return FinishLaunch();
}

}  // extern "C"
