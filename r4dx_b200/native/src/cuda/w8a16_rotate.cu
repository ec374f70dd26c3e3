// Two small members of the linear family:
//   * w8a16 weight-streaming product for 1..8 rows: offset-binary int8 weights with one fp16 scale per
//     (row, group), y[t, n] = sum_g scale[n, g] * sum_{k in g} (q[n, k] - 128) * x[t, k]
//     (layout: native/src/host/w4a16.cpp; the reference serves two model families in this format,
//     reference: docs/w8a16.md:1-60);
//   * in-place block-Hadamard rotation of bf16 rows (128-wide blocks, optional sign vector before or
//     after), the primitive behind rotated residual streams and offline weight rotation
//     (reference: src/kernels/include/r4dx/kernels/kernels.h:420-470).
#include "common.cuh"

namespace r4dxb {
namespace {

constexpr int kThreads = 256;

template <int TMAX>
__global__ void __launch_bounds__(kThreads)
W8Gemv(const uint4* __restrict__ wq, const __half* __restrict__ ws, const __nv_bfloat16* __restrict__ x, void* __restrict__ y,
       int T, int N, int K, int group, int out_f32, int rows_per_cta) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __half* xs = reinterpret_cast<__half*>(smem_raw);   // [TMAX][K]
  for (int i = threadIdx.x; i < TMAX * K; i += kThreads) {
    const int t = i / K, k = i % K;
    xs[i] = (t < T) ? __float2half(__bfloat162float(x[static_cast<size_t>(t) * K + k])) : __half(0);
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int vec_per_row = K / 16, groups = K / group;
  const __half2 bias = __floats2half2_rn(1152.f, 1152.f);    // 1024 (exponent trick) + 128 (offset binary)
  for (int r = warp; r < rows_per_cta; r += kThreads / 32) {
    const int n = blockIdx.x * rows_per_cta + r;
    if (n >= N) break;
    float acc[TMAX];
#pragma unroll
    for (int t = 0; t < TMAX; ++t) acc[t] = 0.f;
    const uint4* rowp = wq + static_cast<size_t>(n) * vec_per_row;
    for (int v = lane; v < vec_per_row; v += 32) {
      const uint4 q = __ldg(rowp + v);
      const int k0 = v * 16;
      const float scale = __half2float(ws[static_cast<size_t>(n) * groups + k0 / group]);
      const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
      __half2 hs[TMAX];
#pragma unroll
      for (int t = 0; t < TMAX; ++t) hs[t] = __float2half2_rn(0.f);
#pragma unroll
      for (int wi = 0; wi < 4; ++wi) {
        // 0x6400 | byte is the fp16 number 1024 + byte, so two byte-permutes build four exact code values
        const uint32_t lo = __byte_perm(qw[wi], 0x64646464u, 0x4140), hi = __byte_perm(qw[wi], 0x64646464u, 0x4342);
        const __half2 w01 = __hsub2(*reinterpret_cast<const __half2*>(&lo), bias);
        const __half2 w23 = __hsub2(*reinterpret_cast<const __half2*>(&hi), bias);
#pragma unroll
        for (int t = 0; t < TMAX; ++t) {
          const uint2 xv = *reinterpret_cast<const uint2*>(xs + static_cast<size_t>(t) * K + k0 + wi * 4);
          hs[t] = __hfma2(w01, *reinterpret_cast<const __half2*>(&xv.x), hs[t]);
          hs[t] = __hfma2(w23, *reinterpret_cast<const __half2*>(&xv.y), hs[t]);
        }
      }
#pragma unroll
      for (int t = 0; t < TMAX; ++t) acc[t] = fmaf(scale, __low2float(hs[t]) + __high2float(hs[t]), acc[t]);
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

// one warp per (row, 128-block); mode 0: x <- H x / sqrt(128); 1: x <- H (s * x) / sqrt(128); 2: x <- s * H x / sqrt(128)
__global__ void RotateKernel(__nv_bfloat16* __restrict__ x, const __half* __restrict__ signs, long long items, int H, int mode) {
  const long long item = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= items) return;
  const int lane = threadIdx.x & 31;
  const int blocks = H / 128;
  const long long row = item / blocks;
  const int b = static_cast<int>(item % blocks);
  __nv_bfloat16* p = x + row * H + b * 128 + lane * 4;
  const uint2 xv = *reinterpret_cast<const uint2*>(p);
  float v[4] = {BfLo(xv.x), BfHi(xv.x), BfLo(xv.y), BfHi(xv.y)};
  float s[4] = {1.f, 1.f, 1.f, 1.f};
  if (mode != 0) {
    const uint2 sv = *reinterpret_cast<const uint2*>(signs + b * 128 + lane * 4);
    const __half2 s01 = *reinterpret_cast<const __half2*>(&sv.x), s23 = *reinterpret_cast<const __half2*>(&sv.y);
    s[0] = __low2float(s01); s[1] = __high2float(s01); s[2] = __low2float(s23); s[3] = __high2float(s23);
  }
  if (mode == 1) { v[0] *= s[0]; v[1] *= s[1]; v[2] *= s[2]; v[3] *= s[3]; }
  WarpFwht128(v);
  const float c = 0.08838834764831845f;
  if (mode == 2) { v[0] *= s[0]; v[1] *= s[1]; v[2] *= s[2]; v[3] *= s[3]; }
  uint2 ov;
  ov.x = PackBf16(v[0] * c, v[1] * c);
  ov.y = PackBf16(v[2] * c, v[3] * c);
  *reinterpret_cast<uint2*>(p) = ov;
}

// Residual-stream rotation, in place on bf16 rows [T, H]:  forward  x <- x Q,  inverse  x <- x Q^T  with
//   Q = diag(signs) . blockdiag(H_B / sqrt(B)) . (mix (x) I_B),   B a power of two <= 1024, H = nblk * B, nblk <= 8.
// One CTA per row: the row lives in shared memory as fp32; the block transform runs its first five butterfly levels in
// registers + shuffles (a lane holds one element per pass) and the rest through shared memory; the mix is an
// nblk x nblk product per column.  (reference: src/kernels/src/rotate_residual.hip:79-333 does the same job with one
// workgroup per row in LDS.)
constexpr int kRotThreads = 256;
constexpr int kRotMaxBlocks = 8;

__device__ __forceinline__ void RowFwht(float* row, int n, int tid, int nthreads) {
  // in-place unnormalised Hadamard transform of row[0..n) in shared memory, n a power of two >= 2
  for (int h = 1; h < n; h <<= 1) {
    for (int i = tid; i < n / 2; i += nthreads) {
      const int lo = (i / h) * 2 * h + (i % h);
      const float a = row[lo], b = row[lo + h];
      row[lo] = a + b;
      row[lo + h] = a - b;
    }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(kRotThreads)
RotateResidualKernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ signs, const float* __restrict__ mix, int H, int B,
                     int inverse) {
  extern __shared__ float rsm[];            // [H] the row, [H] scratch for the mix
  float* row = rsm;
  float* tmp = rsm + H;
  __shared__ float m[kRotMaxBlocks * kRotMaxBlocks];
  const int nblk = H / B;
  __nv_bfloat16* xr = x + static_cast<size_t>(blockIdx.x) * H;
  if (threadIdx.x < nblk * nblk) m[threadIdx.x] = mix[threadIdx.x];
  for (int i = threadIdx.x; i < H; i += kRotThreads) {
    const float v = __bfloat162float(xr[i]);
    row[i] = inverse ? v : v * signs[i];
  }
  __syncthreads();
  const float scale = rsqrtf(static_cast<float>(B));
  if (inverse) {
    // h_b = sum_d mix[b, d] x_d
    for (int i = threadIdx.x; i < H; i += kRotThreads) {
      const int b = i / B, c = i % B;
      float acc = 0.f;
      for (int d = 0; d < nblk; ++d) acc = fmaf(m[b * nblk + d], row[d * B + c], acc);
      tmp[i] = acc;
    }
    __syncthreads();
    for (int b = 0; b < nblk; ++b) RowFwht(tmp + b * B, B, threadIdx.x, kRotThreads);
    for (int i = threadIdx.x; i < H; i += kRotThreads) xr[i] = __float2bfloat16(tmp[i] * scale * signs[i]);
  } else {
    for (int b = 0; b < nblk; ++b) RowFwht(row + b * B, B, threadIdx.x, kRotThreads);
    // y_d = sum_b mix[b, d] h_b
    for (int i = threadIdx.x; i < H; i += kRotThreads) {
      const int d = i / B, c = i % B;
      float acc = 0.f;
      for (int b = 0; b < nblk; ++b) acc = fmaf(m[b * nblk + d], row[b * B + c], acc);
      xr[i] = __float2bfloat16(acc * scale);
    }
  }
}

template <int TMAX>
int LaunchW8(const void* wq, const void* ws, const void* x, void* y, int T, int N, int K, int group, int out_f32, cudaStream_t s) {
  const size_t smem = static_cast<size_t>(TMAX) * K * sizeof(__half);
  auto kern = W8Gemv<TMAX>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  const int rows_per_cta = N >= 148 * 64 ? 32 : 8;
  kern<<<(N + rows_per_cta - 1) / rows_per_cta, kThreads, smem, s>>>(static_cast<const uint4*>(wq), static_cast<const __half*>(ws),
                                                                    static_cast<const __nv_bfloat16*>(x), y, T, N, K, group,
                                                                    out_f32, rows_per_cta);
  return FinishLaunch();
}

}  // namespace
}  // namespace r4dxb

using namespace r4dxb;

extern "C" {

/* y[T, N] = x[T, K] W^T for w8a16 weights; T <= 8; out_f32 selects fp32 or bf16 output. */
int r4dxb_w8a16_gemv(const void* wq, const void* ws, const void* x, void* y, int T, int N, int K, int group, int out_f32,
                     void* stream) {
  if (T < 1 || T > 8 || K % 16 || group % 16 || K % group) return R4DXB_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (static_cast<size_t>(T <= 1 ? 1 : (T <= 4 ? 4 : 8)) * K * 2 > 200 * 1024) return R4DXB_UNSUPPORTED;
  if (T == 1) return LaunchW8<1>(wq, ws, x, y, T, N, K, group, out_f32, s);
  if (T <= 4) return LaunchW8<4>(wq, ws, x, y, T, N, K, group, out_f32, s);
  return LaunchW8<8>(wq, ws, x, y, T, N, K, group, out_f32, s);
}

/* in-place block-Hadamard rotation of bf16 rows [T, H]; signs: fp16 [H] (modes 1 and 2), see RotateKernel */
int r4dxb_rotate_rows(void* x, const void* signs, long long T, int H, int mode, void* stream) {
  if (T < 1 || H % 128 || mode < 0 || mode > 2 || (mode != 0 && signs == nullptr)) return R4DXB_BAD_ARG;
  const long long items = T * (H / 128);
  RotateKernel<<<static_cast<unsigned>((items + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(x), static_cast<const __half*>(signs), items, H, mode);
  return FinishLaunch();
}

/* Residual-stream rotation in place on bf16 rows [T, H]: x <- x Q (inverse 0) or x <- x Q^T (inverse 1);
 * signs fp32 [H] (+-1), mix fp32 [H/B, H/B] orthogonal, B a power of two, H/B <= 8, H <= 16384. */
int r4dxb_rotate_residual(void* x, const float* signs, const float* mix, long long T, int H, int B, int inverse, void* stream) {
  if (T < 1 || H < 2 || B < 2 || (B & (B - 1)) || H % B || H / B > kRotMaxBlocks || H > 16384 || signs == nullptr || mix == nullptr)
    return R4DXB_BAD_ARG;
  const size_t smem = static_cast<size_t>(H) * 2 * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(RotateResidualKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  RotateResidualKernel<<<static_cast<unsigned>(T), kRotThreads, smem, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(x), signs, mix, H, B, inverse);
  return FinishLaunch();
}

}  // extern "C"
