// Kernels of the block-diffusion drafter (a small bidirectional model that proposes a block of
// tokens at once; the target verifies them losslessly).
//
//   conv : dynamic grouped token mixer, out[t, c] = (base0[g] + dyn0[t, g]) h[t, c]
//                                                 + (base1[g] + dyn1[t, g]) h[t-1, c] [t >= 1],  g = c / 16
//   attn : the block's rows attend, without a causal mask, to the injected context ring (entries whose
//          position lies in [lo, n), stored at slot = position % window) and to the whole block.
//          One CTA per query head, one warp per block row, online softmax; the block has at most 8 rows
//          and the ring at most a few thousand entries, so a warp-per-row sweep is enough.
// (reference: docs/dflash2.md:117-160 defines the layer; src/model/dflash_draft.h:20-45 the round.)
#include "common.cuh"

namespace r4dxb {
namespace {

__global__ void DflashConvKernel(const __nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ base,
                                 const __nv_bfloat16* __restrict__ dyn, __nv_bfloat16* __restrict__ out, int T, int H) {
  const int t = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  const int G = H / 16, g = c / 16;
  // base is per channel [2, H]; the dynamic part is shared by the 16 channels of a group
  const float a0 = __bfloat162float(base[c]) + __bfloat162float(dyn[static_cast<size_t>(t) * 2 * G + g]);
  const float a1 = __bfloat162float(base[H + c]) + __bfloat162float(dyn[static_cast<size_t>(t) * 2 * G + G + g]);
  float v = a0 * __bfloat162float(h[static_cast<size_t>(t) * H + c]);
  if (t >= 1) v += a1 * __bfloat162float(h[static_cast<size_t>(t - 1) * H + c]);
  out[static_cast<size_t>(t) * H + c] = __float2bfloat16(v);
}

// In-place per-head RMSNorm (plain scale) + full-width NeoX rope on rows of [T, heads, D]; grid (heads, T), block D.
__global__ void DflashNormRopeKernel(__nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                     const int* __restrict__ positions, int heads, int D, float theta, float eps) {
  extern __shared__ float row[];
  __shared__ float red[32];
  const int t = blockIdx.y, hh = blockIdx.x, d = threadIdx.x;
  __nv_bfloat16* p = x + (static_cast<size_t>(t) * heads + hh) * D;
  float v = __bfloat162float(p[d]);
  const float ss = BlockSum(v * v, red);
  v = v * rsqrtf(ss / D + eps) * __bfloat162float(w[d]);
  row[d] = v;
  __syncthreads();
  const int half = D / 2, i = d < half ? d : d - half;
  const float inv = exp2f(-log2f(theta) * (2.0f * i / D));
  float s, c;
  sincosf(static_cast<float>(positions[t]) * inv, &s, &c);
  v = d < half ? row[d] * c - row[d + half] * s : row[d] * c + row[d - half] * s;
  p[d] = __float2bfloat16(v);
}

// grid Hq, block 32 * T.  q [T, Hq, D], kb / vb (block) [T, Hkv, D], ring_k / ring_v [window, Hkv, D] (bf16)
template <int D>
__global__ void DflashAttnKernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kb,
                                 const __nv_bfloat16* __restrict__ vb, const __nv_bfloat16* __restrict__ ring_k,
                                 const __nv_bfloat16* __restrict__ ring_v, __nv_bfloat16* __restrict__ out, int T, int Hq, int Hkv,
                                 int window, int lo, int n) {
  constexpr int PER = D / 32;
  const int hq = blockIdx.x, hkv = hq / (Hq / Hkv);
  const int t = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (t >= T) return;
  float qv[PER], acc[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    qv[i] = __bfloat162float(q[(static_cast<size_t>(t) * Hq + hq) * D + lane * PER + i]);
    acc[i] = 0.f;
  }
  const float scale = rsqrtf(static_cast<float>(D)) * 1.4426950408889634f;
  float m = -INFINITY, l = 0.f;
  const int n_ring = n - lo;
  for (int j = 0; j < n_ring + T; ++j) {
    const __nv_bfloat16 *kp, *vp;
    if (j < n_ring) {
      const size_t slot = static_cast<size_t>((lo + j) % window);
      kp = ring_k + (slot * Hkv + hkv) * D;
      vp = ring_v + (slot * Hkv + hkv) * D;
    } else {
      kp = kb + (static_cast<size_t>(j - n_ring) * Hkv + hkv) * D;
      vp = vb + (static_cast<size_t>(j - n_ring) * Hkv + hkv) * D;
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) s = fmaf(qv[i], __bfloat162float(kp[lane * PER + i]), s);
    s = WarpSum(s) * scale;
    const float mn = fmaxf(m, s);
    const float al = exp2f(m - mn), p = exp2f(s - mn);
    l = l * al + p;
#pragma unroll
    for (int i = 0; i < PER; ++i) acc[i] = acc[i] * al + p * __bfloat162float(vp[lane * PER + i]);
    m = mn;
  }
  const float inv = 1.f / l;
#pragma unroll
  for (int i = 0; i < PER; ++i) out[(static_cast<size_t>(t) * Hq + hq) * D + lane * PER + i] = __float2bfloat16(acc[i] * inv);
}

}  // namespace
}  // namespace r4dxb

using namespace r4dxb;

extern "C" {

/* base: bf16 [2, H/16]; dyn: bf16 [T, 2, H/16] */
int r4dxb_dflash_conv(const void* h, const void* base, const void* dyn, void* out, int T, int H, void* stream) {
  if (T < 1 || H % 16) return R4DXB_BAD_ARG;
  DflashConvKernel<<<dim3((H + 255) / 256, T), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(h), static_cast<const __nv_bfloat16*>(base), static_cast<const __nv_bfloat16*>(dyn),
      static_cast<__nv_bfloat16*>(out), T, H);
  return FinishLaunch();
}

int r4dxb_dflash_norm_rope(void* x, const void* w, const int* positions, int T, int heads, int D, float theta, float eps,
                           void* stream) {
  if (T < 1 || heads < 1 || D % 32 || D > 1024) return R4DXB_BAD_ARG;
  DflashNormRopeKernel<<<dim3(heads, T), D, D * sizeof(float), static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w), positions, heads, D, theta, eps);
  return FinishLaunch();
}

/* ring entries at positions [lo, n) are visible (n - lo <= window); the block's rows sit at positions n .. n + T - 1 */
int r4dxb_dflash_attention(const void* q, const void* kb, const void* vb, const void* ring_k, const void* ring_v, void* out,
                           int T, int Hq, int Hkv, int D, int window, int lo, int n, void* stream) {
  if (T < 1 || T > 16 || Hq % Hkv || lo > n || n - lo > window || lo < 0) return R4DXB_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  auto a = [&](const void* p) { return static_cast<const __nv_bfloat16*>(p); };
  if (D == 128) DflashAttnKernel<128><<<Hq, 32 * T, 0, s>>>(a(q), a(kb), a(vb), a(ring_k), a(ring_v), static_cast<__nv_bfloat16*>(out), T, Hq, Hkv, window, lo, n);
  else if (D == 64) DflashAttnKernel<64><<<Hq, 32 * T, 0, s>>>(a(q), a(kb), a(vb), a(ring_k), a(ring_v), static_cast<__nv_bfloat16*>(out), T, Hq, Hkv, window, lo, n);
  else return R4DXB_UNSUPPORTED;
  return FinishLaunch();
}

}  // extern "C"
