// Memory-bound glue kernels: embedding gather, RMSNorm family, SwiGLU, residual add, LayerNorm,
// GELU, bias.  One CTA per token row, 16-byte vector loads, fp32 math, one bf16 rounding per
// output.  Semantics follow the documented ops of the reference
// (reference: src/kernels/include/r4dx/kernels/kernels.h:42-108, 336-370, 556-640).
#include "common.cuh"

namespace r4dxb {

unsigned long long g_launch_count = 0;

namespace {

constexpr int kRowThreads = 256;

__global__ void EmbedGatherKernel(const int* __restrict__ ids, const uint4* __restrict__ table,
                                  uint4* __restrict__ out, int H8, int V) {
  const int t = blockIdx.x;
  int id = ids[t];
  id = id < 0 ? 0 : (id >= V ? V - 1 : id);   // clamping gather: a bad id never reads out of bounds
  const uint4* src = table + static_cast<size_t>(id) * H8;
  uint4* dst = out + static_cast<size_t>(t) * H8;
  for (int i = threadIdx.x; i < H8; i += blockDim.x) dst[i] = src[i];
}

// mode bit 0: weight is zero-centred (multiply by 1 + w); bit 1: no weight.
template <bool kAdd>
__global__ void RmsNormKernel(__nv_bfloat16* __restrict__ res, const __nv_bfloat16* __restrict__ delta,
                              const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out, int H,
                              float eps, int mode) {
  extern __shared__ float row[];
  __shared__ float red[32];
  const size_t base = static_cast<size_t>(blockIdx.x) * H;
  float ss = 0.0f;
  for (int i = threadIdx.x * 2; i < H; i += blockDim.x * 2) {
    uint32_t p = *reinterpret_cast<const uint32_t*>(res + base + i);
    float a = BfLo(p), b = BfHi(p);
    if (kAdd) {
      const uint32_t q = *reinterpret_cast<const uint32_t*>(delta + base + i);
      a += BfLo(q);
      b += BfHi(q);
      const uint32_t r = PackBf16(a, b);     // the residual stream is bf16: round, then normalise what is stored
      *reinterpret_cast<uint32_t*>(res + base + i) = r;
      a = BfLo(r);
      b = BfHi(r);
    }
    row[i] = a;
    row[i + 1] = b;
    ss += a * a + b * b;
  }
  ss = BlockSum(ss, red);
  const float r = rsqrtf(ss / H + eps);
  for (int i = threadIdx.x * 2; i < H; i += blockDim.x * 2) {
    float wa = 1.0f, wb = 1.0f;
    if (!(mode & 2)) {
      const uint32_t q = *reinterpret_cast<const uint32_t*>(w + i);
      wa = BfLo(q);
      wb = BfHi(q);
      if (mode & 1) { wa += 1.0f; wb += 1.0f; }
    }
    *reinterpret_cast<uint32_t*>(out + base + i) = PackBf16(row[i] * r * wa, row[i + 1] * r * wb);
  }
}

// Sandwich-norm residual update: res[t] += rmsnorm(delta[t]) * (1 + w)  (the block's output is normalised BEFORE it
// joins the residual stream; reference: src/model/gemma_layer.cpp post-attention / post-feed-forward norms).
__global__ void NormAddKernel(__nv_bfloat16* __restrict__ res, const __nv_bfloat16* __restrict__ delta,
                              const __nv_bfloat16* __restrict__ w, int H, float eps) {
  __shared__ float red[32];
  const size_t base = static_cast<size_t>(blockIdx.x) * H;
  float ss = 0.0f;
  for (int i = threadIdx.x * 2; i < H; i += blockDim.x * 2) {
    const uint32_t p = *reinterpret_cast<const uint32_t*>(delta + base + i);
    ss += BfLo(p) * BfLo(p) + BfHi(p) * BfHi(p);
  }
  ss = BlockSum(ss, red);
  const float r = rsqrtf(ss / H + eps);
  for (int i = threadIdx.x * 2; i < H; i += blockDim.x * 2) {
    const uint32_t p = *reinterpret_cast<const uint32_t*>(delta + base + i);
    const uint32_t q = *reinterpret_cast<const uint32_t*>(w + i);
    const uint32_t x = *reinterpret_cast<const uint32_t*>(res + base + i);
    // the normalised block output is a bf16 tensor in the unfused graph: round it, then add
    const uint32_t n = PackBf16(BfLo(p) * r * (1.0f + BfLo(q)), BfHi(p) * r * (1.0f + BfHi(q)));
    *reinterpret_cast<uint32_t*>(res + base + i) = PackBf16(BfLo(x) + BfLo(n), BfHi(x) + BfHi(n));
  }
}

__global__ void LayerNormKernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ out, int H, float eps) {
  extern __shared__ float row[];
  __shared__ float red[32];
  const size_t base = static_cast<size_t>(blockIdx.x) * H;
  float s = 0.0f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    row[i] = __bfloat162float(x[base + i]);
    s += row[i];
  }
  const float mean = BlockSum(s, red) / H;
  float v = 0.0f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float d = row[i] - mean;
    v += d * d;
  }
  const float r = rsqrtf(BlockSum(v, red) / H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    out[base + i] = __float2bfloat16((row[i] - mean) * r * __bfloat162float(w[i]) + __bfloat162float(b[i]));
}

__global__ void SiluMulKernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int I) {
  const size_t t = blockIdx.y;
  const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (i >= I) return;
  const uint32_t g = *reinterpret_cast<const uint32_t*>(gu + t * 2 * I + i);
  const uint32_t u = *reinterpret_cast<const uint32_t*>(gu + t * 2 * I + I + i);
  *reinterpret_cast<uint32_t*>(out + t * I + i) = PackBf16(Silu(BfLo(g)) * BfLo(u), Silu(BfHi(g)) * BfHi(u));
}

__global__ void ResidualAddKernel(__nv_bfloat16* __restrict__ res, const __nv_bfloat16* __restrict__ delta, size_t n2) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n2) return;
  const uint32_t a = reinterpret_cast<const uint32_t*>(res)[i], b = reinterpret_cast<const uint32_t*>(delta)[i];
  reinterpret_cast<uint32_t*>(res)[i] = PackBf16(BfLo(a) + BfLo(b), BfHi(a) + BfHi(b));
}

// act: 0 = bias only, 1 = gelu tanh, 2 = gelu erf (bias optional)
__global__ void BiasActKernel(__nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ bias, int H, size_t n, int act) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float v = __bfloat162float(x[i]);
  if (bias) v += __bfloat162float(bias[i % H]);
  if (act == 1) {
    const float c = 0.7978845608028654f;
    v = 0.5f * v * (1.0f + tanhf(c * (v + 0.044715f * v * v * v)));
  } else if (act == 2) {
    v = 0.5f * v * (1.0f + erff(v * 0.7071067811865476f));
  }
  x[i] = __float2bfloat16(v);
}

// Lossless greedy verification of a speculative window: row i's argmax must equal draft i+1.
// out[0] = rows to commit (accepted drafts + 1), out[1..] = emitted tokens (accepted drafts, then the
// correction / bonus token).  (reference: src/model/model.cpp:3344-3426 does this walk on the host)
__global__ void SpecAcceptKernel(const int* __restrict__ next_ids, const int* __restrict__ draft, int T,
                                 int* __restrict__ out, int* __restrict__ n_replay) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  int n = 1;
  while (n < T && next_ids[n - 1] == draft[n - 1]) ++n;
  for (int i = 0; i + 1 < n; ++i) out[1 + i] = draft[i];
  out[n] = next_ids[n - 1];
  out[0] = n;
  if (n_replay) n_replay[0] = n;
}

// (Sample-and-match uses the same kernel: next_ids then holds the token drawn per row from the
// target distribution, and a draft is accepted while the draw equals it.)
}  // namespace
}  // namespace r4dxb

using namespace r4dxb;

extern "C" {

unsigned long long r4dxb_launch_count() { return g_launch_count; }
void r4dxb_launch_count_reset() { g_launch_count = 0; }

int r4dxb_embed_gather_bf16(const int* ids, const void* table, void* out, int T, int H, int V, void* stream) {
  if (H % 8 || T <= 0) return R4DXB_BAD_ARG;
  EmbedGatherKernel<<<T, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      ids, static_cast<const uint4*>(table), static_cast<uint4*>(out), H / 8, V);
  return FinishLaunch();
}

int r4dxb_rmsnorm_bf16(const void* x, const void* w, void* out, int T, int H, float eps, int mode, void* stream) {
  if (H % 2 || T <= 0) return R4DXB_BAD_ARG;
  RmsNormKernel<false><<<T, kRowThreads, H * sizeof(float), static_cast<cudaStream_t>(stream)>>>(
      const_cast<__nv_bfloat16*>(static_cast<const __nv_bfloat16*>(x)), nullptr,
      static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(out), H, eps, mode);
  return FinishLaunch();
}

int r4dxb_add_rmsnorm_bf16(void* res, const void* delta, const void* w, void* out, int T, int H, float eps, int mode,
                           void* stream) {
  if (H % 2 || T <= 0) return R4DXB_BAD_ARG;
  RmsNormKernel<true><<<T, kRowThreads, H * sizeof(float), static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(res), static_cast<const __nv_bfloat16*>(delta),
      static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(out), H, eps, mode);
  return FinishLaunch();
}

int r4dxb_norm_add_bf16(void* res, const void* delta, const void* w, int T, int H, float eps, void* stream) {
  if (H % 2 || T <= 0) return R4DXB_BAD_ARG;
  NormAddKernel<<<T, kRowThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(res), static_cast<const __nv_bfloat16*>(delta), static_cast<const __nv_bfloat16*>(w), H, eps);
  return FinishLaunch();
}

int r4dxb_layernorm_bf16(const void* x, const void* w, const void* b, void* out, int T, int H, float eps, void* stream) {
  if (T <= 0) return R4DXB_BAD_ARG;
  LayerNormKernel<<<T, kRowThreads, H * sizeof(float), static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
      static_cast<const __nv_bfloat16*>(b), static_cast<__nv_bfloat16*>(out), H, eps);
  return FinishLaunch();
}

int r4dxb_silu_mul_bf16(const void* gate_up, void* out, int T, int I, void* stream) {
  if (I % 2 || T <= 0) return R4DXB_BAD_ARG;
  dim3 grid((I / 2 + 255) / 256, T);
  SiluMulKernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gate_up), static_cast<__nv_bfloat16*>(out), I);
  return FinishLaunch();
}

int r4dxb_residual_add_bf16(void* res, const void* delta, long long n, void* stream) {
  if (n % 2 || n <= 0) return R4DXB_BAD_ARG;
  const size_t n2 = n / 2;
  ResidualAddKernel<<<static_cast<unsigned>((n2 + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(res), static_cast<const __nv_bfloat16*>(delta), n2);
  return FinishLaunch();
}

int r4dxb_spec_accept(const int* next_ids, const int* draft, int T, int* out, int* n_replay, void* stream) {
  if (T < 1 || T > 64) return R4DXB_BAD_ARG;
  SpecAcceptKernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(next_ids, draft, T, out, n_replay);
  return FinishLaunch();
}

int r4dxb_bias_act_bf16(void* x, const void* bias, int T, int H, int act, void* stream) {
  const size_t n = static_cast<size_t>(T) * H;
  BiasActKernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(bias), H, n, act);
  return FinishLaunch();
}

}  // extern "C"
