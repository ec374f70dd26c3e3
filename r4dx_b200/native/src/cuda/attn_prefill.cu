// Causal GQA attention for a long chunk of query rows over the fp8 paged KV cache (prefill).
//
// One CTA = one KV head x 16 query tokens; warp j handles query head (kv_head * gqa + j), so the
// K/V tiles a CTA dequantises (fp8 -> fp16, 32 keys at a time) are shared by all gqa heads.  Scores
// and the PV product run on warp-level tensor-core MMAs (m16n8k16, fp16 in, fp32 accumulate) with an
// online softmax in the log2 domain; the epilogue applies o * sigmoid(gate) and rounds to bf16.
// The raw fp8 rows of the next key tile are fetched with cp.async while the current tile is in the
// MMAs; shared memory and registers are sized so that two CTAs share an SM (12 warps hide the rest of
// the latency); tiles entirely below the diagonal skip the mask, and the accumulator is only rescaled
// when a row maximum actually moved.
// The chunk's own K/V rows must already be in the cache (the pre-core kernel writes them first).
//
// This is the first-generation prefill kernel: it is not yet on tcgen05/TMEM (the GEMMs are).
// The reference's counterpart is a query-tiled WMMA kernel with split-KV modes
// (reference: third_party/libr4d/r4d_attn_prefill_h256_gqa6.hip:112).
#include <cuda_pipeline.h>

#include "common.cuh"

namespace r4dxb {
namespace {

constexpr int kBlockTokens = 16;
constexpr int kKeyTile = 32;
constexpr int kQTile = 16;

__device__ __forceinline__ void LdMatrixX4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void LdMatrixX4T(uint32_t (&r)[4], const void* p) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void MmaF16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t PackHalf2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t Fp8x2ToHalf2Bits(uint16_t v) {
  __half2_raw r = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(v), __NV_E4M3);
  return *reinterpret_cast<uint32_t*>(&r);
}

struct PrefillArgs {
  const __nv_bfloat16* q;      // [T, Hq, D] normed + roped
  const __nv_bfloat16* qg;     // [T, Hq, 2D] (gate in the upper half), may be null when !gated
  const uint8_t* cache;        // [block][Hkv][2][16][D] fp8
  const int* block_table;
  const float* k_descale;
  const float* v_descale;
  __nv_bfloat16* out;          // [T, Hq, D]
  int T, Hq, Hkv, pos0, gated;
  int window;                  // sliding-window length in tokens (0: causal over the whole sequence)
  const int* key_limit;        // optional [T]: a row also sees keys up to this absolute position (-1: none), for rows of an
                               // image block that attend to the whole block; the block's keys are part of the same call
};

template <int D, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, (WARPS <= 6 ? 2 : 1)) AttnPrefillKernel(PrefillArgs a) {
  constexpr int LD = D + 8;                 // padded row length (halves)
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int gqa = a.Hq / a.Hkv;
  __half* Qs = reinterpret_cast<__half*>(smem_raw);             // [gqa * 16][LD]
  __half* Ks = Qs + gqa * kQTile * LD;                           // [32][LD]
  __half* Vs = Ks + kKeyTile * LD;                               // [32][LD]
  uint8_t* raw = reinterpret_cast<uint8_t*>(Vs + kKeyTile * LD);  // [2][32][D] fp8 rows of the next tile (K then V)
  const int qt = blockIdx.x, hkv = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nthreads = blockDim.x;
  const int t_base = qt * kQTile;
  const int hq = hkv * gqa + warp;

  // stage Q (bf16 -> fp16)
  for (int i = threadIdx.x; i < gqa * kQTile * (D / 8); i += nthreads) {
    const int row = i / (D / 8), c8 = (i % (D / 8)) * 8;
    const int j = row / kQTile, tt = row % kQTile;
    const int t = t_base + tt;
    uint4 o = make_uint4(0, 0, 0, 0);
    if (t < a.T) {
      const uint4 v = *reinterpret_cast<const uint4*>(a.q + (static_cast<size_t>(t) * a.Hq + hkv * gqa + j) * D + c8);
      o.x = PackHalf2(BfLo(v.x), BfHi(v.x));
      o.y = PackHalf2(BfLo(v.y), BfHi(v.y));
      o.z = PackHalf2(BfLo(v.z), BfHi(v.z));
      o.w = PackHalf2(BfLo(v.w), BfHi(v.w));
    }
    *reinterpret_cast<uint4*>(Qs + row * LD + c8) = o;
  }

  const float sm_scale = rsqrtf(static_cast<float>(D)) * a.k_descale[hkv] * 1.4426950408889634f;
  const int g = lane >> 2, tq = lane & 3;
  const int pos_r0 = a.pos0 + t_base + g, pos_r1 = pos_r0 + 8;   // positions of this lane's two rows
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float O[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) { O[n][0] = O[n][1] = O[n][2] = O[n][3] = 0.f; }

  int last_pos = a.pos0 + min(a.T, t_base + kQTile) - 1;
  int lim0 = pos_r0, lim1 = pos_r1;               // last visible key of this lane's two rows
  if (a.key_limit != nullptr) {
    if (t_base + g < a.T) lim0 = max(lim0, a.key_limit[t_base + g]);
    if (t_base + g + 8 < a.T) lim1 = max(lim1, a.key_limit[t_base + g + 8]);
    for (int i = 0; i < kQTile && t_base + i < a.T; ++i) last_pos = max(last_pos, a.key_limit[t_base + i]);
    last_pos = min(last_pos, a.pos0 + a.T - 1);
  }
  const int key_tiles = last_pos / kKeyTile + 1;
  auto fetch = [&](int kt) {      // raw fp8 rows of key tile kt -> shared memory (16-byte pieces, zero past the end)
    for (int i = threadIdx.x; i < 2 * kKeyTile * (D / 16); i += nthreads) {
      const int which = i / (kKeyTile * (D / 16));                 // 0 = K, 1 = V
      const int rem = i % (kKeyTile * (D / 16));
      const int key = rem / (D / 16), c16 = (rem % (D / 16)) * 16;
      const int kp = kt * kKeyTile + key;
      uint8_t* dst = raw + (which * kKeyTile + key) * D + c16;
      if (kp <= last_pos) {
        const int blk = a.block_table[kp / kBlockTokens];
        const uint8_t* src = a.cache + ((static_cast<size_t>(blk) * a.Hkv + hkv) * 2 + which) * kBlockTokens * D +
                             (kp % kBlockTokens) * D + c16;
        __pipeline_memcpy_async(dst, src, 16);
      } else {
        *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
      }
    }
    __pipeline_commit();
  };
  // sliding window: tiles entirely older than the first row's window are never touched
  const int kt_first = a.window > 0 ? max(0, a.pos0 + t_base - a.window + 1) / kKeyTile : 0;
  fetch(kt_first);
  for (int kt = kt_first; kt < key_tiles; ++kt) {
    __pipeline_wait_prior(0);
    __syncthreads();     // raw tile landed; previous tile fully consumed (also orders the Q staging before first use)
    // ---- dequantise the K and V tiles ----
    for (int i = threadIdx.x; i < 2 * kKeyTile * (D / 16); i += nthreads) {
      const int which = i / (kKeyTile * (D / 16));
      const int rem = i % (kKeyTile * (D / 16));
      const int key = rem / (D / 16), c16 = (rem % (D / 16)) * 16;
      const uint4 rw = *reinterpret_cast<const uint4*>(raw + (which * kKeyTile + key) * D + c16);
      uint4 lo, hi;
      lo.x = Fp8x2ToHalf2Bits(rw.x & 0xFFFF); lo.y = Fp8x2ToHalf2Bits(rw.x >> 16);
      lo.z = Fp8x2ToHalf2Bits(rw.y & 0xFFFF); lo.w = Fp8x2ToHalf2Bits(rw.y >> 16);
      hi.x = Fp8x2ToHalf2Bits(rw.z & 0xFFFF); hi.y = Fp8x2ToHalf2Bits(rw.z >> 16);
      hi.z = Fp8x2ToHalf2Bits(rw.w & 0xFFFF); hi.w = Fp8x2ToHalf2Bits(rw.w >> 16);
      __half* dst = (which == 0 ? Ks : Vs) + key * LD + c16;
      *reinterpret_cast<uint4*>(dst) = lo;
      *reinterpret_cast<uint4*>(dst + 8) = hi;
    }
    __syncthreads();
    if (kt + 1 < key_tiles) fetch(kt + 1);      // overlaps with the MMAs below
    if (warp >= gqa) continue;

    // ---- S = Q K^T (16 x 64 per warp) ----
    float S[kKeyTile / 8][4];
#pragma unroll
    for (int n = 0; n < kKeyTile / 8; ++n) { S[n][0] = S[n][1] = S[n][2] = S[n][3] = 0.f; }
#pragma unroll 4
    for (int k0 = 0; k0 < D; k0 += 16) {
      uint32_t af[4];
      LdMatrixX4(af, Qs + (warp * kQTile + (lane & 15)) * LD + k0 + (lane >> 4) * 8);
#pragma unroll
      for (int n2 = 0; n2 < kKeyTile / 16; ++n2) {
        uint32_t bf[4];
        // matrices: (keys 0-7, k 0-7), (keys 0-7, k 8-15), (keys 8-15, k 0-7), (keys 8-15, k 8-15)
        LdMatrixX4(bf, Ks + (n2 * 16 + (lane & 7) + ((lane >> 4) << 3)) * LD + k0 + ((lane >> 3) & 1) * 8);
        MmaF16(S[2 * n2], af, bf[0], bf[1]);
        MmaF16(S[2 * n2 + 1], af, bf[2], bf[3]);
      }
    }
    // ---- mask + online softmax (log2 domain) ----
    float mx0 = m0, mx1 = m1;
    if (kt * kKeyTile + kKeyTile - 1 <= a.pos0 + t_base &&
        (a.window == 0 || kt * kKeyTile > a.pos0 + t_base + kQTile - 1 - a.window)) {      // the whole tile is visible to every row of the CTA
#pragma unroll
      for (int n = 0; n < kKeyTile / 8; ++n) {
        S[n][0] *= sm_scale; S[n][1] *= sm_scale; S[n][2] *= sm_scale; S[n][3] *= sm_scale;
        mx0 = fmaxf(mx0, fmaxf(S[n][0], S[n][1]));
        mx1 = fmaxf(mx1, fmaxf(S[n][2], S[n][3]));
      }
    } else {
#pragma unroll
      for (int n = 0; n < kKeyTile / 8; ++n) {
        const int kp = kt * kKeyTile + n * 8 + tq * 2;
        const int w0 = a.window > 0 ? pos_r0 - a.window : -1, w1 = a.window > 0 ? pos_r1 - a.window : -1;
        S[n][0] = (kp <= lim0 && kp > w0) ? S[n][0] * sm_scale : -INFINITY;
        S[n][1] = (kp + 1 <= lim0 && kp + 1 > w0) ? S[n][1] * sm_scale : -INFINITY;
        S[n][2] = (kp <= lim1 && kp > w1) ? S[n][2] * sm_scale : -INFINITY;
        S[n][3] = (kp + 1 <= lim1 && kp + 1 > w1) ? S[n][3] * sm_scale : -INFINITY;
        mx0 = fmaxf(mx0, fmaxf(S[n][0], S[n][1]));
        mx1 = fmaxf(mx1, fmaxf(S[n][2], S[n][3]));
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float al0 = (mx0 == -INFINITY) ? 1.f : exp2f(m0 - mx0);
    const float al1 = (mx1 == -INFINITY) ? 1.f : exp2f(m1 - mx1);
    const float sub0 = (mx0 == -INFINITY) ? 0.f : mx0, sub1 = (mx1 == -INFINITY) ? 0.f : mx1;
    float rs0 = 0.f, rs1 = 0.f;
    uint32_t P[kKeyTile / 16][4];
#pragma unroll
    for (int n = 0; n < kKeyTile / 8; ++n) {
      const float p0 = exp2f(S[n][0] - sub0), p1 = exp2f(S[n][1] - sub0);
      const float p2 = exp2f(S[n][2] - sub1), p3 = exp2f(S[n][3] - sub1);
      rs0 += p0 + p1;
      rs1 += p2 + p3;
      P[n >> 1][(n & 1) * 2] = PackHalf2(p0, p1);
      P[n >> 1][(n & 1) * 2 + 1] = PackHalf2(p2, p3);
    }
    l0 = l0 * al0 + rs0;
    l1 = l1 * al1 + rs1;
    m0 = mx0;
    m1 = mx1;
    if (!__all_sync(0xffffffffu, al0 == 1.f && al1 == 1.f)) {     // no row maximum moved: nothing to rescale
#pragma unroll
      for (int n = 0; n < D / 8; ++n) { O[n][0] *= al0; O[n][1] *= al0; O[n][2] *= al1; O[n][3] *= al1; }
    }
    // ---- O += P V ----
#pragma unroll
    for (int j = 0; j < kKeyTile / 16; ++j) {
#pragma unroll
      for (int n2 = 0; n2 < D / 16; ++n2) {
        uint32_t bf[4];
        // transposed loads: matrices (keys 0-7, d 0-7), (keys 8-15, d 0-7), (keys 0-7, d 8-15), (keys 8-15, d 8-15)
        LdMatrixX4T(bf, Vs + (j * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + n2 * 16 + (lane >> 4) * 8);
        MmaF16(O[2 * n2], P[j], bf[0], bf[1]);
        MmaF16(O[2 * n2 + 1], P[j], bf[2], bf[3]);
      }
    }
  }
  if (warp >= gqa) return;
  // ---- epilogue ----
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float vds = a.v_descale[hkv];
  const float inv0 = l0 > 0.f ? vds / l0 : 0.f, inv1 = l1 > 0.f ? vds / l1 : 0.f;
  const int t0 = t_base + g, t1 = t0 + 8;
#pragma unroll
  for (int n = 0; n < D / 8; ++n) {
    const int d = n * 8 + tq * 2;
    if (t0 < a.T) {
      float x0 = O[n][0] * inv0, x1 = O[n][1] * inv0;
      if (a.gated) {
        const uint32_t gv = *reinterpret_cast<const uint32_t*>(a.qg + (static_cast<size_t>(t0) * a.Hq + hq) * 2 * D + D + d);
        x0 *= Sigmoid(BfLo(gv));
        x1 *= Sigmoid(BfHi(gv));
      }
      *reinterpret_cast<uint32_t*>(a.out + (static_cast<size_t>(t0) * a.Hq + hq) * D + d) = PackBf16(x0, x1);
    }
    if (t1 < a.T) {
      float x2 = O[n][2] * inv1, x3 = O[n][3] * inv1;
      if (a.gated) {
        const uint32_t gv = *reinterpret_cast<const uint32_t*>(a.qg + (static_cast<size_t>(t1) * a.Hq + hq) * 2 * D + D + d);
        x2 *= Sigmoid(BfLo(gv));
        x3 *= Sigmoid(BfHi(gv));
      }
      *reinterpret_cast<uint32_t*>(a.out + (static_cast<size_t>(t1) * a.Hq + hq) * D + d) = PackBf16(x2, x3);
    }
  }
}

}  // namespace
}  // namespace r4dxb

using namespace r4dxb;

/* key_limit (optional, [T] int32, -1 = none): row t also attends to keys up to that absolute position (image blocks). */
extern "C" int r4dxb_attn_prefill_ex(const void* q, const void* qg, const void* cache, const int* block_table,
                                     const float* k_descale, const float* v_descale, void* out, int T, int Hq, int Hkv, int D,
                                     int pos0, int flags, const int* key_limit, void* stream) {
  const int gated = flags & 1;      // bit 0: sigmoid output gate; bits 1..: sliding-window length (0 = none)
  if (T < 1 || Hq % Hkv || (D != 256 && D != 64 && D != 128)) return R4DXB_BAD_ARG;
  const int gqa = Hq / Hkv;
  if (gqa > 8) return R4DXB_UNSUPPORTED;
  PrefillArgs a;
  a.q = static_cast<const __nv_bfloat16*>(q);
  a.qg = static_cast<const __nv_bfloat16*>(qg);
  a.cache = static_cast<const uint8_t*>(cache);
  a.block_table = block_table;
  a.k_descale = k_descale;
  a.v_descale = v_descale;
  a.out = static_cast<__nv_bfloat16*>(out);
  a.T = T; a.Hq = Hq; a.Hkv = Hkv; a.pos0 = pos0; a.gated = gated; a.window = flags >> 1;
  a.key_limit = key_limit;
  const int warps = gqa <= 2 ? 2 : (gqa <= 4 ? 4 : (gqa <= 6 ? 6 : 8));   // idle warps still help the tile conversion
  const size_t smem = static_cast<size_t>(gqa * kQTile + 2 * kKeyTile) * (D + 8) * 2 + 2 * kKeyTile * D;
  dim3 grid((T + kQTile - 1) / kQTile, Hkv);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  auto launch = [&](auto kern) -> int {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    kern<<<grid, warps * 32, smem, s>>>(a);
    return 0;
  };
  int rc = R4DXB_BAD_ARG;
#define R4DXB_ATTN_CASE(DD, WW) if (D == DD && warps == WW) rc = launch(AttnPrefillKernel<DD, WW>);
  R4DXB_ATTN_CASE(256, 2) R4DXB_ATTN_CASE(256, 4) R4DXB_ATTN_CASE(256, 6) R4DXB_ATTN_CASE(256, 8)
  R4DXB_ATTN_CASE(128, 2) R4DXB_ATTN_CASE(128, 4) R4DXB_ATTN_CASE(128, 6) R4DXB_ATTN_CASE(128, 8)
  R4DXB_ATTN_CASE(64, 2) R4DXB_ATTN_CASE(64, 4) R4DXB_ATTN_CASE(64, 6) R4DXB_ATTN_CASE(64, 8)
#undef R4DXB_ATTN_CASE
  if (rc) return rc;
  return FinishLaunch();
}

extern "C" int r4dxb_attn_prefill(const void* q, const void* qg, const void* cache, const int* block_table,
                                  const float* k_descale, const float* v_descale, void* out, int T, int Hq, int Hkv, int D,
                                  int pos0, int flags, void* stream) {
  return r4dxb_attn_prefill_ex(q, qg, cache, block_table, k_descale, v_descale, out, T, Hq, Hkv, D, pos0, flags, nullptr, stream);
}
