// Weight-streaming GEMMs for T <= 8 rows over 4-bit grouped weights (LM / MTP / drafter heads)
// and over small dense bf16 matrices (gate projections, MoE router), plus the row argmax.
//
// w4a16: w = scale * (q - zero); a nibble n becomes fp16 (0x6400 | n) = 1024 + n, the stored
// fp16 -(1024 + zero) makes n - zero exact, eight products are summed in fp16x2 and the group
// sum is scaled in fp32 (the reference uses the same exact-nibble trick on its WMMA path:
// reference third_party/libr4d/r4d_gemm_w4a16_nt_m64.hip:1-67).  One warp streams one weight
// row with 16-byte loads (32 weights per lane per load); rows are independent, so there is no
// cross-CTA reduction.
#include "common.cuh"

namespace r4dxb {
namespace {

constexpr int kThreads = 256;

template <int TMAX>
__global__ void __launch_bounds__(kThreads)
W4Gemv(const uint4* __restrict__ wq, const uint32_t* __restrict__ wsz, const __nv_bfloat16* __restrict__ x,
       void* __restrict__ y, int T, int N, int K, int group, int out_f32, int rows_per_cta) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __half* xs = reinterpret_cast<__half*>(smem_raw);   // [TMAX][K], every 8 values stored as 0,4,1,5,2,6,3,7
  for (int i = threadIdx.x; i < TMAX * K; i += kThreads) {
    const int t = i / K, k = i % K;
    const int j = k & 7;
    const int slot = (j < 4) ? 2 * j : 2 * (j - 4) + 1;
    xs[t * K + (k & ~7) + slot] = (t < T) ? __float2half(__bfloat162float(x[static_cast<size_t>(t) * K + k])) : __half(0);
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int vec_per_row = K / 32;            // uint4 per row
  const int groups = K / group;
  const int row0 = blockIdx.x * rows_per_cta;
  if constexpr (TMAX == 1) {
    // single-row decode (the vocabulary head): two weight rows per warp iteration, so that twice as many 16-byte
    // loads are in flight per warp and every activation vector read from shared memory serves two rows
    for (int r = warp; r < rows_per_cta; r += 2 * (kThreads / 32)) {
      const int n0 = row0 + r, n1 = n0 + kThreads / 32;
      if (n0 >= N) break;
      const bool two = (r + kThreads / 32 < rows_per_cta) && n1 < N;
      const uint4* rp0 = wq + static_cast<size_t>(n0) * vec_per_row;
      const uint4* rp1 = wq + static_cast<size_t>(two ? n1 : n0) * vec_per_row;
      const uint32_t* sz0p = wsz + static_cast<size_t>(n0) * groups;
      const uint32_t* sz1p = wsz + static_cast<size_t>(two ? n1 : n0) * groups;
      float a0 = 0.f, a1 = 0.f;
      for (int v = lane; v < vec_per_row; v += 32) {
        const uint4 q0 = __ldg(rp0 + v), q1 = __ldg(rp1 + v);
        const int k0 = v * 32;
        const uint32_t s0 = __ldg(sz0p + k0 / group), s1 = __ldg(sz1p + k0 / group);
        const uint32_t nzb0 = (s0 >> 16) | (s0 & 0xFFFF0000u), nzb1 = (s1 >> 16) | (s1 & 0xFFFF0000u);
        const __half2 nz0 = *reinterpret_cast<const __half2*>(&nzb0), nz1 = *reinterpret_cast<const __half2*>(&nzb1);
        const uint32_t w0[4] = {q0.x, q0.y, q0.z, q0.w}, w1[4] = {q1.x, q1.y, q1.z, q1.w};
        float g0 = 0.f, g1 = 0.f;
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {
          const uint4 xv = *reinterpret_cast<const uint4*>(xs + k0 + wi * 8);
          const __half2 x0 = *reinterpret_cast<const __half2*>(&xv.x), x1 = *reinterpret_cast<const __half2*>(&xv.y);
          const __half2 x2 = *reinterpret_cast<const __half2*>(&xv.z), x3 = *reinterpret_cast<const __half2*>(&xv.w);
          __half2 p0, p1;
          {
            uint32_t b;
            b = ((w0[wi]) & 0x000F000Fu) | 0x64006400u;        p0 = __hmul2(__hadd2(*reinterpret_cast<const __half2*>(&b), nz0), x0);
            b = ((w0[wi] >> 4) & 0x000F000Fu) | 0x64006400u;   p0 = __hfma2(__hadd2(*reinterpret_cast<const __half2*>(&b), nz0), x1, p0);
            b = ((w0[wi] >> 8) & 0x000F000Fu) | 0x64006400u;   p0 = __hfma2(__hadd2(*reinterpret_cast<const __half2*>(&b), nz0), x2, p0);
            b = ((w0[wi] >> 12) & 0x000F000Fu) | 0x64006400u;  p0 = __hfma2(__hadd2(*reinterpret_cast<const __half2*>(&b), nz0), x3, p0);
            b = ((w1[wi]) & 0x000F000Fu) | 0x64006400u;        p1 = __hmul2(__hadd2(*reinterpret_cast<const __half2*>(&b), nz1), x0);
            b = ((w1[wi] >> 4) & 0x000F000Fu) | 0x64006400u;   p1 = __hfma2(__hadd2(*reinterpret_cast<const __half2*>(&b), nz1), x1, p1);
            b = ((w1[wi] >> 8) & 0x000F000Fu) | 0x64006400u;   p1 = __hfma2(__hadd2(*reinterpret_cast<const __half2*>(&b), nz1), x2, p1);
            b = ((w1[wi] >> 12) & 0x000F000Fu) | 0x64006400u;  p1 = __hfma2(__hadd2(*reinterpret_cast<const __half2*>(&b), nz1), x3, p1);
          }
          g0 += __low2float(p0) + __high2float(p0);
          g1 += __low2float(p1) + __high2float(p1);
        }
        a0 = fmaf(g0, __half2float(__ushort_as_half(static_cast<unsigned short>(s0 & 0xFFFF))), a0);
        a1 = fmaf(g1, __half2float(__ushort_as_half(static_cast<unsigned short>(s1 & 0xFFFF))), a1);
      }
      a0 = WarpSum(a0);
      a1 = WarpSum(a1);
      if (lane == 0 && T >= 1) {
        if (out_f32) {
          static_cast<float*>(y)[n0] = a0;
          if (two) static_cast<float*>(y)[n1] = a1;
        } else {
          static_cast<__nv_bfloat16*>(y)[n0] = __float2bfloat16(a0);
          if (two) static_cast<__nv_bfloat16*>(y)[n1] = __float2bfloat16(a1);
        }
      }
    }
    return;
  }
  for (int r = warp; r < rows_per_cta; r += kThreads / 32) {
    const int n = row0 + r;
    if (n >= N) break;
    float acc[TMAX];
#pragma unroll
    for (int t = 0; t < TMAX; ++t) acc[t] = 0.f;
    const uint4* rowp = wq + static_cast<size_t>(n) * vec_per_row;
    for (int v = lane; v < vec_per_row; v += 32) {
      const uint4 q = __ldg(rowp + v);
      const int k0 = v * 32;
      const uint32_t sz = __ldg(wsz + static_cast<size_t>(n) * groups + k0 / group);
      const float scale = __half2float(__ushort_as_half(static_cast<unsigned short>(sz & 0xFFFF)));
      const uint32_t nzb = (sz >> 16) | (sz & 0xFFFF0000u);
      const __half2 nz = *reinterpret_cast<const __half2*>(&nzb);
      const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
      float gsum[TMAX];
#pragma unroll
      for (int t = 0; t < TMAX; ++t) gsum[t] = 0.f;
#pragma unroll
      for (int wi = 0; wi < 4; ++wi) {
        __half2 wv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint32_t bits = ((qw[wi] >> (4 * i)) & 0x000F000Fu) | 0x64006400u;
          wv[i] = __hadd2(*reinterpret_cast<const __half2*>(&bits), nz);   // (n_i - zero, n_{i+4} - zero), exact
        }
#pragma unroll
        for (int t = 0; t < TMAX; ++t) {
          const uint4 xv = *reinterpret_cast<const uint4*>(xs + t * K + k0 + wi * 8);
          __half2 s = __hmul2(wv[0], *reinterpret_cast<const __half2*>(&xv.x));
          s = __hfma2(wv[1], *reinterpret_cast<const __half2*>(&xv.y), s);
          s = __hfma2(wv[2], *reinterpret_cast<const __half2*>(&xv.z), s);
          s = __hfma2(wv[3], *reinterpret_cast<const __half2*>(&xv.w), s);
          gsum[t] += __low2float(s) + __high2float(s);
        }
      }
#pragma unroll
      for (int t = 0; t < TMAX; ++t) acc[t] = fmaf(gsum[t], scale, acc[t]);
    }
#pragma unroll
    for (int t = 0; t < TMAX; ++t) {
      const float s = WarpSum(acc[t]);
      if (lane == 0 && t < T) {
        if (out_f32) static_cast<float*>(y)[static_cast<size_t>(t) * N + n] = s;
        else static_cast<__nv_bfloat16*>(y)[static_cast<size_t>(t) * N + n] = __float2bfloat16(s);
      }
    }
  }
}

__global__ void Bf16Gemv(const __nv_bfloat16* __restrict__ W, const __nv_bfloat16* __restrict__ x, float* __restrict__ y,
                         int T, int N, int K) {
  __shared__ float red[32];
  const int n = blockIdx.x;
  const __nv_bfloat16* w = W + static_cast<size_t>(n) * K;
  for (int t = 0; t < T; ++t) {
    float s = 0.f;
    for (int k = threadIdx.x * 2; k < K; k += blockDim.x * 2) {
      const uint32_t a = *reinterpret_cast<const uint32_t*>(w + k);
      const uint32_t b = *reinterpret_cast<const uint32_t*>(x + static_cast<size_t>(t) * K + k);
      s += BfLo(a) * BfLo(b) + BfHi(a) * BfHi(b);
    }
    s = BlockSum(s, red);
    if (threadIdx.x == 0) y[static_cast<size_t>(t) * N + n] = s;
  }
}

// Small-batch variant with the RMSNorm of the residual stream folded in:
// y[t, n] = W[n, :] . bf16(x[t] * rsqrt(mean x[t]^2 + eps) * (1 + nw))
__global__ void Bf16GemvNorm(const __nv_bfloat16* __restrict__ W, const __nv_bfloat16* __restrict__ x,
                             const __nv_bfloat16* __restrict__ nw, float eps, float* __restrict__ y, int T, int N, int K) {
  PdlEnter();
  __shared__ float red[32];
  const int n = blockIdx.x;
  const __nv_bfloat16* w = W + static_cast<size_t>(n) * K;
  for (int t = 0; t < T; ++t) {
    const __nv_bfloat16* xr = x + static_cast<size_t>(t) * K;
    float ss = 0.f;
    for (int k = threadIdx.x * 2; k < K; k += blockDim.x * 2) {
      const uint32_t b = *reinterpret_cast<const uint32_t*>(xr + k);
      ss += BfLo(b) * BfLo(b) + BfHi(b) * BfHi(b);
    }
    const float r = rsqrtf(BlockSum(ss, red) / K + eps);
    float s = 0.f;
    for (int k = threadIdx.x * 2; k < K; k += blockDim.x * 2) {
      const uint32_t a = *reinterpret_cast<const uint32_t*>(w + k);
      const uint32_t b = *reinterpret_cast<const uint32_t*>(xr + k);
      const uint32_t g = *reinterpret_cast<const uint32_t*>(nw + k);
      const uint32_t h = PackBf16(BfLo(b) * r * (1.f + BfLo(g)), BfHi(b) * r * (1.f + BfHi(g)));
      s += BfLo(a) * BfLo(h) + BfHi(a) * BfHi(h);
    }
    s = BlockSum(s, red);
    if (threadIdx.x == 0) y[static_cast<size_t>(t) * N + n] = s;
  }
}

// Many-row variant: one CTA stages 8 activation rows in shared memory and its warps sweep the
// weight rows, so W is read once per 8 tokens instead of once per token.
__global__ void __launch_bounds__(256) Bf16GemvTiled(const __nv_bfloat16* __restrict__ W, const __nv_bfloat16* __restrict__ x,
                                                     float* __restrict__ y, int T, int N, int K) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [8][K]
  const int t0 = blockIdx.x * 8;
  for (int i = threadIdx.x; i < 8 * (K / 8); i += 256) {
    const int tt = i / (K / 8), c = (i % (K / 8)) * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (t0 + tt < T) v = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(t0 + tt) * K + c);
    *reinterpret_cast<uint4*>(xs + tt * K + c) = v;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // grid.y splits the weight rows so that a few activation tiles still fill the machine
  const int rows_per_cta = (N + gridDim.y - 1) / gridDim.y;
  const int n_begin = blockIdx.y * rows_per_cta, n_end = min(N, n_begin + rows_per_cta);
  for (int n = n_begin + warp; n < n_end; n += 8) {
    float acc[8];
#pragma unroll
    for (int tt = 0; tt < 8; ++tt) acc[tt] = 0.f;
    const __nv_bfloat16* w = W + static_cast<size_t>(n) * K;
    for (int k = lane * 8; k < K; k += 256) {
      const uint4 wv = __ldg(reinterpret_cast<const uint4*>(w + k));
#pragma unroll
      for (int tt = 0; tt < 8; ++tt) {
        const uint4 xv = *reinterpret_cast<const uint4*>(xs + tt * K + k);
        acc[tt] += BfLo(wv.x) * BfLo(xv.x) + BfHi(wv.x) * BfHi(xv.x) + BfLo(wv.y) * BfLo(xv.y) + BfHi(wv.y) * BfHi(xv.y) +
                   BfLo(wv.z) * BfLo(xv.z) + BfHi(wv.z) * BfHi(xv.z) + BfLo(wv.w) * BfLo(xv.w) + BfHi(wv.w) * BfHi(xv.w);
      }
    }
#pragma unroll
    for (int tt = 0; tt < 8; ++tt) {
      const float s = WarpSum(acc[tt]);
      if (lane == 0 && t0 + tt < T) y[static_cast<size_t>(t0 + tt) * N + n] = s;
    }
  }
}

// ---- argmax ------------------------------------------------------------------------------------
constexpr int kArgParts = 256;

__device__ __forceinline__ void ArgBetter(float v, int i, float& bv, int& bi) {
  if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
}

template <bool kF32>
__global__ void ArgmaxPartial(const void* __restrict__ logits, int V, float* __restrict__ pv, int* __restrict__ pi) {
  __shared__ float sv[32];
  __shared__ int si[32];
  const int t = blockIdx.y, part = blockIdx.x;
  const int chunk = (V + kArgParts - 1) / kArgParts;
  const int b = part * chunk, e = min(V, b + chunk);
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = b + threadIdx.x; i < e; i += blockDim.x) {
    float v;
    if (kF32) v = static_cast<const float*>(logits)[static_cast<size_t>(t) * V + i];
    else v = __bfloat162float(static_cast<const __nv_bfloat16*>(logits)[static_cast<size_t>(t) * V + i]);
    if (v != v) v = -INFINITY;   // a NaN never wins
    ArgBetter(v, i, bv, bi);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    ArgBetter(ov, oi, bv, bi);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    bv = lane < nw ? sv[lane] : -INFINITY;
    bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      ArgBetter(ov, oi, bv, bi);
    }
    if (lane == 0) { pv[t * kArgParts + part] = bv; pi[t * kArgParts + part] = bi; }
  }
}

__global__ void ArgmaxFinal(const float* __restrict__ pv, const int* __restrict__ pi, int id_offset,
                            int* __restrict__ out_ids, float* __restrict__ out_vals) {
  __shared__ float sv[8];
  __shared__ int si[8];
  const int t = blockIdx.x;
  float bv = pv[t * kArgParts + threadIdx.x];
  int bi = pi[t * kArgParts + threadIdx.x];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    ArgBetter(ov, oi, bv, bi);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < kArgParts / 32; ++w) ArgBetter(sv[w], si[w], bv, bi);
    // a row of NaNs / -inf leaves the index unset: report the shard's first id instead of overflowing
    out_ids[t] = (bi == 0x7fffffff ? 0 : bi) + id_offset;
    if (out_vals) out_vals[t] = bv;
  }
}

template <int TMAX>
int LaunchW4(const void* wq, const void* wsz, const void* x, void* y, int T, int N, int K, int group, int out_f32,
             cudaStream_t stream) {
  const size_t smem = static_cast<size_t>(TMAX) * K * 2;
  if (smem > 200 * 1024) return R4DXB_TOO_LARGE;
  auto kern = W4Gemv<TMAX>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  // enough CTAs to fill 148 SMs a few times over, but rows_per_cta >= 8 so that every warp has work
  int rows_per_cta = (N + 148 * 8 - 1) / (148 * 8);
  rows_per_cta = ((rows_per_cta + 7) / 8) * 8;
  const int grid = (N + rows_per_cta - 1) / rows_per_cta;
  kern<<<grid, kThreads, smem, stream>>>(static_cast<const uint4*>(wq), static_cast<const uint32_t*>(wsz),
                                         static_cast<const __nv_bfloat16*>(x), y, T, N, K, group, out_f32, rows_per_cta);
  return FinishLaunch();
}

}  // namespace
}  // namespace r4dxb

using namespace r4dxb;

extern "C" {

int r4dxb_w4a16_gemv(const void* wq, const void* wsz, const void* x, void* y, int T, int N, int K, int group,
                     int out_f32, void* stream) {
  if (T < 1 || T > 8 || K % 32 || (group != 32 && group != 64 && group != 128) || K % group) return R4DXB_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (T == 1) return LaunchW4<1>(wq, wsz, x, y, T, N, K, group, out_f32, s);
  if (T == 2) return LaunchW4<2>(wq, wsz, x, y, T, N, K, group, out_f32, s);
  if (T <= 4) return LaunchW4<4>(wq, wsz, x, y, T, N, K, group, out_f32, s);
  return LaunchW4<8>(wq, wsz, x, y, T, N, K, group, out_f32, s);
}

int r4dxb_bf16_gemv(const void* W, const void* x, float* y, int T, int N, int K, void* stream) {
  if (T < 1 || N < 1 || K % 2) return R4DXB_BAD_ARG;
  if (T > 8 && K % 8 == 0 && static_cast<size_t>(K) * 16 <= 200 * 1024) {
    const int smem = K * 16;
    cudaError_t e = cudaFuncSetAttribute(Bf16GemvTiled, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    const int tiles = (T + 7) / 8;
    const int ysplit = max(1, min((N + 7) / 8, 296 / tiles));
    Bf16GemvTiled<<<dim3(tiles, ysplit), 256, smem, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(W), static_cast<const __nv_bfloat16*>(x), y, T, N, K);
    return FinishLaunch();
  }
  Bf16Gemv<<<N, 128, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(W),
                                                             static_cast<const __nv_bfloat16*>(x), y, T, N, K);
  return FinishLaunch();
}

int r4dxb_bf16_gemv_norm(const void* W, const void* x, const void* norm_w, float eps, float* y, int T, int N, int K,
                         void* stream) {
  if (T < 1 || T > 8 || N < 1 || K % 2) return R4DXB_BAD_ARG;
  return LaunchPdl(Bf16GemvNorm, dim3(N), dim3(256), 0, static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(W),
                   static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(norm_w), eps, y, T, N, K);
}

int r4dxb_argmax_rows(const void* logits, int is_f32, int T, int V, int id_offset, int* out_ids, float* out_vals,
                      void* scratch, void* stream) {
  if (T < 1 || V < 1) return R4DXB_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* pv = static_cast<float*>(scratch);
  int* pi = reinterpret_cast<int*>(pv + static_cast<size_t>(T) * kArgParts);
  dim3 grid(kArgParts, T);
  if (is_f32) ArgmaxPartial<true><<<grid, 256, 0, s>>>(logits, V, pv, pi);
  else ArgmaxPartial<false><<<grid, 256, 0, s>>>(logits, V, pv, pi);
  int e = FinishLaunch();
  if (e) return e;
  ArgmaxFinal<<<T, kArgParts, 0, s>>>(pv, pi, id_offset, out_ids, out_vals);
  return FinishLaunch();
}

}  // extern "C"

// ---- row argmax for callers that cannot allocate -------------------------------------------------
// Declared in r4dxb_noalloc.h.  Same two kernels as r4dxb_argmax_rows, but the per-part
// (value, index) partials live in a fixed array inside this library instead of a caller buffer.
#include <mutex>

#include "r4dxb_noalloc.h"

namespace r4dxb {
namespace {

// [rows][256 parts] floats followed by [rows][256 parts] ints; every GPU that loads the library
// carries one copy (128 KiB) until the process exits.
static __device__ __align__(256) unsigned char g_argmax_static_scratch[R4DXB_ARGMAX_STATIC_MAX_ROWS * kArgParts * 8];

constexpr int kMaxDevices = 64;
void* g_static_scratch_addr[kMaxDevices] = {};   // device address of the array, per device ordinal
std::mutex g_static_scratch_mutex;

// In host code the array's name is only a handle; the address a kernel can use comes from
// cudaGetSymbolAddress, looked up once per device while that device is current.
int StaticScratchFor(int device, void** out) {
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_addr[device] == nullptr) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_argmax_static_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    g_static_scratch_addr[device] = p;
  }
  *out = g_static_scratch_addr[device];
  return 0;
}

}  // namespace
}  // namespace r4dxb

extern "C" int r4dxb_argmax_rows_static(const void* logits, int is_f32, int T, int V, int id_offset, int* out_ids,
                                        float* out_vals, void* stream) {
  using namespace r4dxb;
  if (T < 1 || V < 1 || logits == nullptr || out_ids == nullptr) return R4DXB_BAD_ARG;
  if (T > R4DXB_ARGMAX_STATIC_MAX_ROWS) return R4DXB_TOO_LARGE;
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (device < 0 || device >= kMaxDevices) return R4DXB_UNSUPPORTED;
  void* scratch = nullptr;
  const int rc = StaticScratchFor(device, &scratch);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* pv = static_cast<float*>(scratch);
  int* pi = reinterpret_cast<int*>(pv + static_cast<size_t>(T) * kArgParts);
  // Every (row, part) slot that ArgmaxFinal reads is written by ArgmaxPartial in this same call,
  // so nothing left over from an earlier call is ever consumed and nothing needs clearing.
  dim3 grid(kArgParts, T);
  if (is_f32) ArgmaxPartial<true><<<grid, 256, 0, s>>>(logits, V, pv, pi);
  else ArgmaxPartial<false><<<grid, 256, 0, s>>>(logits, V, pv, pi);
  int err = FinishLaunch();
  if (err) return err;
  ArgmaxFinal<<<T, kArgParts, 0, s>>>(pv, pi, id_offset, out_ids, out_vals);
  return FinishLaunch();
}
