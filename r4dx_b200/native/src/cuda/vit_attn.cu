// Vision-tower kernels: axial (height / width) rotary embedding and bidirectional attention over
// packed image segments.
//
//   rope : q and k inside the packed qkv rows [T, 3, H, D]; rotary pairs are (d, d + D/2); the first
//          D/4 frequencies turn with the patch's row index, the next D/4 with its column index.
//   attn : every token attends to all tokens of its own segment (one image or video frame group,
//          given by cu_seqlens); 64 query rows per CTA (4 warps x 16 rows), 64-key tiles converted
//          to fp16 in shared memory, m16n8k16 tensor-core products with an online softmax.  The head
//          width is padded to a multiple of 16 in shared memory, so the 72-wide heads of the 27-block
//          tower run as 80 (reference: third_party/libr4d/r4d_attn_vit_h72_bf16.hip:1-40 is the
//          dedicated 72-wide kernel there).
#include "common.cuh"

namespace r4dxb {
namespace {

__global__ void VitRopeKernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ pos_hw, int T, int H, int D, float theta) {
  const int t = blockIdx.x, which = blockIdx.y;          // which: 0 = q, 1 = k
  const int half = D / 2, quarter = D / 4;
  const int ph = pos_hw[2 * t], pw = pos_hw[2 * t + 1];
  __nv_bfloat16* base = qkv + (static_cast<size_t>(t) * 3 + which) * H * D;
  for (int i = threadIdx.x; i < H * half; i += blockDim.x) {
    const int h = i / half, d = i % half;
    const int fi = d < quarter ? d : d - quarter;
    const float inv = exp2f(-log2f(theta) * (2.0f * fi / half));
    float s, c;
    sincosf(static_cast<float>(d < quarter ? ph : pw) * inv, &s, &c);
    const float x1 = __bfloat162float(base[h * D + d]), x2 = __bfloat162float(base[h * D + d + half]);
    base[h * D + d] = __float2bfloat16(x1 * c - x2 * s);
    base[h * D + d + half] = __float2bfloat16(x2 * c + x1 * s);
  }
}

__device__ __forceinline__ void LdsmX4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void LdsmX4T(uint32_t (&r)[4], const void* p) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void Mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t PackH2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

constexpr int kQRows = 64, kKeys = 64;

// grid (ceil(T / 64), H), 128 threads.  DP = head width rounded up to 16.
template <int DP>
__global__ void __launch_bounds__(128) VitAttnKernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ out,
                                                     const int* __restrict__ cu_seqlens, int nseg, int T, int H, int D,
                                                     float scale_log2) {
  constexpr int LD = DP + 8;
  __shared__ __align__(16) __half Qs[kQRows * LD];
  __shared__ __align__(16) __half Ks[kKeys * LD];
  __shared__ __align__(16) __half Vs[kKeys * LD];
  __shared__ int seg_lo[kQRows], seg_hi[kQRows];
  const int q0 = blockIdx.x * kQRows, h = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t row_stride = static_cast<size_t>(3) * H * D;

  auto stage = [&](__half* dst, int which, int first, int limit) {     // rows [first, first + 64) of q / k / v, zero padded
    for (int i = threadIdx.x; i < 64 * (DP / 2); i += 128) {
      const int r = i / (DP / 2), d = (i % (DP / 2)) * 2;
      const int t = first + r;
      uint32_t v = 0;
      if (t < limit && d < D) {
        const uint32_t raw = *reinterpret_cast<const uint32_t*>(qkv + t * row_stride + (static_cast<size_t>(which) * H + h) * D + d);
        v = PackH2(BfLo(raw), BfHi(raw));
      }
      *reinterpret_cast<uint32_t*>(dst + r * LD + d) = v;
    }
  };
  stage(Qs, 0, q0, T);
  if (threadIdx.x < kQRows) {
    const int t = min(q0 + static_cast<int>(threadIdx.x), T - 1);
    int s = 0;
    while (s + 1 < nseg && cu_seqlens[s + 1] <= t) ++s;
    seg_lo[threadIdx.x] = cu_seqlens[s];
    seg_hi[threadIdx.x] = cu_seqlens[s + 1];
  }
  __syncthreads();
  const int g = lane >> 2, tq = lane & 3;
  const int r0 = warp * 16 + g, r1 = r0 + 8;
  const int lo0 = seg_lo[r0], hi0 = seg_hi[r0], lo1 = seg_lo[r1], hi1 = seg_hi[r1];
  // the CTA walks the union of its rows' segments (rows are sorted, so it is one contiguous range)
  const int k_begin = seg_lo[0], k_end = seg_hi[min(kQRows - 1, T - 1 - q0)];
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float O[DP / 8][4];
#pragma unroll
  for (int n = 0; n < DP / 8; ++n) O[n][0] = O[n][1] = O[n][2] = O[n][3] = 0.f;

  for (int kt = k_begin; kt < k_end; kt += kKeys) {
    __syncthreads();
    stage(Ks, 1, kt, k_end);
    stage(Vs, 2, kt, k_end);
    __syncthreads();
    float S[kKeys / 8][4];
#pragma unroll
    for (int n = 0; n < kKeys / 8; ++n) S[n][0] = S[n][1] = S[n][2] = S[n][3] = 0.f;
#pragma unroll
    for (int k0 = 0; k0 < DP; k0 += 16) {
      uint32_t af[4];
      LdsmX4(af, Qs + (warp * 16 + (lane & 15)) * LD + k0 + (lane >> 4) * 8);
#pragma unroll
      for (int n2 = 0; n2 < kKeys / 16; ++n2) {
        uint32_t bf[4];
        LdsmX4(bf, Ks + (n2 * 16 + (lane & 7) + ((lane >> 4) << 3)) * LD + k0 + ((lane >> 3) & 1) * 8);
        Mma16816(S[2 * n2], af, bf[0], bf[1]);
        Mma16816(S[2 * n2 + 1], af, bf[2], bf[3]);
      }
    }
    float mx0 = m0, mx1 = m1;
#pragma unroll
    for (int n = 0; n < kKeys / 8; ++n) {
      const int kp = kt + n * 8 + tq * 2;
      S[n][0] = (kp >= lo0 && kp < hi0) ? S[n][0] * scale_log2 : -INFINITY;
      S[n][1] = (kp + 1 >= lo0 && kp + 1 < hi0) ? S[n][1] * scale_log2 : -INFINITY;
      S[n][2] = (kp >= lo1 && kp < hi1) ? S[n][2] * scale_log2 : -INFINITY;
      S[n][3] = (kp + 1 >= lo1 && kp + 1 < hi1) ? S[n][3] * scale_log2 : -INFINITY;
      mx0 = fmaxf(mx0, fmaxf(S[n][0], S[n][1]));
      mx1 = fmaxf(mx1, fmaxf(S[n][2], S[n][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float al0 = (mx0 == -INFINITY) ? 1.f : exp2f(m0 - mx0), al1 = (mx1 == -INFINITY) ? 1.f : exp2f(m1 - mx1);
    const float sub0 = (mx0 == -INFINITY) ? 0.f : mx0, sub1 = (mx1 == -INFINITY) ? 0.f : mx1;
    float rs0 = 0.f, rs1 = 0.f;
    uint32_t P[kKeys / 16][4];
#pragma unroll
    for (int n = 0; n < kKeys / 8; ++n) {
      const float p0 = exp2f(S[n][0] - sub0), p1 = exp2f(S[n][1] - sub0);
      const float p2 = exp2f(S[n][2] - sub1), p3 = exp2f(S[n][3] - sub1);
      rs0 += p0 + p1;
      rs1 += p2 + p3;
      P[n >> 1][(n & 1) * 2] = PackH2(p0, p1);
      P[n >> 1][(n & 1) * 2 + 1] = PackH2(p2, p3);
    }
    l0 = l0 * al0 + rs0;
    l1 = l1 * al1 + rs1;
    m0 = mx0;
    m1 = mx1;
#pragma unroll
    for (int n = 0; n < DP / 8; ++n) { O[n][0] *= al0; O[n][1] *= al0; O[n][2] *= al1; O[n][3] *= al1; }
#pragma unroll
    for (int j = 0; j < kKeys / 16; ++j) {
#pragma unroll
      for (int n2 = 0; n2 < DP / 16; ++n2) {
        uint32_t bf[4];
        LdsmX4T(bf, Vs + (j * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + n2 * 16 + (lane >> 4) * 8);
        Mma16816(O[2 * n2], P[j], bf[0], bf[1]);
        Mma16816(O[2 * n2 + 1], P[j], bf[2], bf[3]);
      }
    }
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
  const int t0 = q0 + r0, t1 = q0 + r1;
#pragma unroll
  for (int n = 0; n < DP / 8; ++n) {
    const int d = n * 8 + tq * 2;
    if (d < D) {
      if (t0 < T) *reinterpret_cast<uint32_t*>(out + (static_cast<size_t>(t0) * H + h) * D + d) = PackBf16(O[n][0] * inv0, O[n][1] * inv0);
      if (t1 < T) *reinterpret_cast<uint32_t*>(out + (static_cast<size_t>(t1) * H + h) * D + d) = PackBf16(O[n][2] * inv1, O[n][3] * inv1);
    }
  }
}

}  // namespace
}  // namespace r4dxb

using namespace r4dxb;

extern "C" {

/* in-place axial rope on q and k of packed qkv [T, 3, H, D]; pos_hw: int [T, 2] (row, column) */
int r4dxb_vit_rope(void* qkv, const int* pos_hw, int T, int H, int D, float theta, void* stream) {
  if (T < 1 || D % 4) return R4DXB_BAD_ARG;
  VitRopeKernel<<<dim3(T, 2), 128, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<__nv_bfloat16*>(qkv), pos_hw, T, H, D, theta);
  return FinishLaunch();
}

/* out[T, H, D] = softmax(q k^T / sqrt(D)) v inside each segment [cu_seqlens[s], cu_seqlens[s+1]); D even, <= 96 */
int r4dxb_vit_attention(const void* qkv, void* out, const int* cu_seqlens, int nseg, int T, int H, int D, void* stream) {
  if (T < 1 || nseg < 1 || D % 2 || D > 96) return R4DXB_BAD_ARG;
  const float scale_log2 = rsqrtf(static_cast<float>(D)) * 1.4426950408889634f;
  dim3 grid((T + kQRows - 1) / kQRows, H);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* in = static_cast<const __nv_bfloat16*>(qkv);
  __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out);
  const int dp = (D + 15) / 16 * 16;
  switch (dp) {
    case 16: VitAttnKernel<16><<<grid, 128, 0, s>>>(in, o, cu_seqlens, nseg, T, H, D, scale_log2); break;
    case 32: VitAttnKernel<32><<<grid, 128, 0, s>>>(in, o, cu_seqlens, nseg, T, H, D, scale_log2); break;
    case 48: VitAttnKernel<48><<<grid, 128, 0, s>>>(in, o, cu_seqlens, nseg, T, H, D, scale_log2); break;
    case 64: VitAttnKernel<64><<<grid, 128, 0, s>>>(in, o, cu_seqlens, nseg, T, H, D, scale_log2); break;
    case 80: VitAttnKernel<80><<<grid, 128, 0, s>>>(in, o, cu_seqlens, nseg, T, H, D, scale_log2); break;
    case 96: VitAttnKernel<96><<<grid, 128, 0, s>>>(in, o, cu_seqlens, nseg, T, H, D, scale_log2); break;
    default: return R4DXB_UNSUPPORTED;
  }
  return FinishLaunch();
}

}  // extern "C"
