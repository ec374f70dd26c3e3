// Kernels of the qwen4_exp family that the other families do not have: the gated 4-stream residual, the hashed n-gram
// embedding layer and the block-selecting ("sparse") attention.  (reference: docs/qwen4exp-plan.md 2.2-2.4; contracts of
// the reference's kernels in src/model/qwen4exp/include/r4dx/model/qwen4exp/{hc_kernels,ple_kernels,qsa_kernels}.h.)
//
// Design notes (B200): the n-gram table lives in device memory, so the row ids are hashed and the rows gathered by one
// kernel from a device-resident token history (no host work per token, graph-capturable); every piece of per-sequence
// state added here is keyed by absolute position (token history, indexer keys, block keys) or by position modulo a ring
// (the n-gram layer's conv inputs), so chunks of any size compose exactly and a rewind needs no repair.  All tensors that
// cross kernels are bf16, rounded where the checkpoint's own bf16 graph rounds; sums are fp32.
#include <math.h>

#include "common.cuh"

namespace r4dxb {
namespace {

__device__ __forceinline__ float Rb(float v) { return __bfloat162float(__float2bfloat16(v)); }

// ---- grouped RMSNorm with (1 + w): grid (rows, groups), 256 threads ------------------------------------------------
__global__ void GroupedRmsNormKernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                     __nv_bfloat16* __restrict__ out, int groups, int gs, float eps) {
  __shared__ float red[32];
  const size_t base = (static_cast<size_t>(blockIdx.x) * groups + blockIdx.y) * gs;
  const int wbase = blockIdx.y * gs;
  float ss = 0.f;
  for (int d = threadIdx.x; d < gs; d += blockDim.x) {
    const float v = __bfloat162float(x[base + d]);
    ss += v * v;
  }
  ss = BlockSum(ss, red);
  const float r = rsqrtf(ss / gs + eps);
  for (int d = threadIdx.x; d < gs; d += blockDim.x)
    out[base + d] = __float2bfloat16(__bfloat162float(x[base + d]) * r * (1.0f + __bfloat162float(w[wbase + d])));
}

// ---- stream gate: mid = silu(Rb(down / hc)) over the first L columns of the [rows, L + hc] fp32 product ----------------
__global__ void HcMidKernel(const float* __restrict__ dn, __nv_bfloat16* __restrict__ mid, int rows, int L, int stride, float scale) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * L) return;
  const int r = i / L, c = i - r * L;
  mid[i] = __float2bfloat16(Silu(Rb(Rb(dn[static_cast<size_t>(r) * stride + c]) * scale)));
}

// x[r, d] = Rb( (1/hc) sum_g Rb( Rb(sigmoid(up[r, g H + d])) * n[r, g H + d] ) ); up is the fp32 product
__global__ void HcMixKernel(const __nv_bfloat16* __restrict__ n, const float* __restrict__ up, __nv_bfloat16* __restrict__ x,
                            int rows, int hc, int H) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * H) return;
  const int r = i / H, d = i - r * H;
  float acc = 0.f;
  for (int g = 0; g < hc; ++g) {
    const size_t at = (static_cast<size_t>(r) * hc + g) * H + d;
    acc += Rb(Rb(Sigmoid(Rb(up[at]))) * __bfloat162float(n[at]));
  }
  x[i] = __float2bfloat16(acc / hc);
}

// h[r, g H + d] = Rb( h + Rb(out[r, d] * inj[r, g]) ), inj = Rb(2 Rb(sigmoid(Rb(v / hc)))); v = columns L.. of the product
__global__ void HcInjectKernel(__nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ out, const float* __restrict__ v,
                               int rows, int hc, int H, int stride) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * hc * H) return;
  const int r = i / (hc * H), rem = i - r * hc * H, g = rem / H, d = rem - g * H;
  const float inj = Rb(2.0f * Rb(Sigmoid(Rb(Rb(v[static_cast<size_t>(r) * stride + g]) / hc))));
  h[i] = __float2bfloat16(__bfloat162float(h[i]) + Rb(__bfloat162float(out[static_cast<size_t>(r) * H + d]) * inj));
}

// ---- the stream gate in two launches (decode: every intermediate of the five-kernel chain stays on chip) ----------------
// Kernel 1, grid (L + hc) CTAs of 512 threads: CTA n owns output n of the [down; inject] product for all T <= 8 rows.  Every
// CTA recomputes the per-stream RMS statistics of the rows (the rows are 20 KB each and come from L2), normalises on the
// fly with the same roundings as the separate norm kernel, and finishes its output: mid = silu(Rb(Rb(down) / hc)) for
// n < L, the raw injection logit otherwise.  CTA 0 also leaves the statistics for kernel 2.
constexpr int kGateThreads = 512;
constexpr int kGateRows = 8;
__global__ void __launch_bounds__(kGateThreads)
HcDownKernel(const __nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ norm_w, const __nv_bfloat16* __restrict__ W,
             __nv_bfloat16* __restrict__ mid, float* __restrict__ injv, float* __restrict__ rstd, int T, int hc, int H, int L,
             int n_inject, float eps) {
  __shared__ float s_r[kGateRows][8];                   // [row][stream] reciprocal RMS
  __shared__ float red[kGateThreads / 32][kGateRows];
  const int n = blockIdx.x, C = hc * H, nvec = C / 8;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // statistics: one stream at a time, all rows
  for (int g = 0; g < hc; ++g) {
    float ss[kGateRows];
#pragma unroll
    for (int t = 0; t < kGateRows; ++t) ss[t] = 0.f;
    for (int v = threadIdx.x; v < H / 8; v += kGateThreads) {
#pragma unroll
      for (int t = 0; t < kGateRows; ++t) {
        if (t >= T) break;
        const uint4 x = *reinterpret_cast<const uint4*>(h + static_cast<size_t>(t) * C + g * H + v * 8);
        const uint32_t w4[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) ss[t] += BfLo(w4[j]) * BfLo(w4[j]) + BfHi(w4[j]) * BfHi(w4[j]);
      }
    }
#pragma unroll
    for (int t = 0; t < kGateRows; ++t) ss[t] = WarpSum(ss[t]);
    __syncthreads();
    if (lane == 0)
      for (int t = 0; t < kGateRows; ++t) red[warp][t] = ss[t];
    __syncthreads();
    if (threadIdx.x < T) {
      float tot = 0.f;
      for (int w = 0; w < kGateThreads / 32; ++w) tot += red[w][threadIdx.x];
      s_r[threadIdx.x][g] = rsqrtf(tot / H + eps);
    }
  }
  __syncthreads();
  if (n == 0 && threadIdx.x < T * hc) rstd[threadIdx.x] = s_r[threadIdx.x / hc][threadIdx.x % hc];
  float acc[kGateRows];
#pragma unroll
  for (int t = 0; t < kGateRows; ++t) acc[t] = 0.f;
  const __nv_bfloat16* wrow = W + static_cast<size_t>(n) * C;
  for (int v = threadIdx.x; v < nvec; v += kGateThreads) {
    const uint4 wv = *reinterpret_cast<const uint4*>(wrow + v * 8);
    const uint4 nv = *reinterpret_cast<const uint4*>(norm_w + v * 8);
    const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w}, nn[4] = {nv.x, nv.y, nv.z, nv.w};
    const int g = (v * 8) / H;
#pragma unroll
    for (int t = 0; t < kGateRows; ++t) {
      if (t >= T) break;
      const uint4 x = *reinterpret_cast<const uint4*>(h + static_cast<size_t>(t) * C + v * 8);
      const uint32_t xx[4] = {x.x, x.y, x.z, x.w};
      const float r = s_r[t][g];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[t] += BfLo(ww[j]) * Rb(BfLo(xx[j]) * r * (1.0f + BfLo(nn[j]))) + BfHi(ww[j]) * Rb(BfHi(xx[j]) * r * (1.0f + BfHi(nn[j])));
      }
    }
  }
#pragma unroll
  for (int t = 0; t < kGateRows; ++t) acc[t] = WarpSum(acc[t]);
  __syncthreads();
  if (lane == 0)
    for (int t = 0; t < kGateRows; ++t) red[warp][t] = acc[t];
  __syncthreads();
  if (threadIdx.x < T) {
    float tot = 0.f;
    for (int w = 0; w < kGateThreads / 32; ++w) tot += red[w][threadIdx.x];
    if (n < L) mid[static_cast<size_t>(threadIdx.x) * L + n] = __float2bfloat16(Silu(Rb(Rb(tot) * (1.0f / hc))));
    else if (n - L < n_inject) injv[threadIdx.x * n_inject + (n - L)] = tot;
  }
}

// Kernel 2, grid H / 8 CTAs of 8 warps: warp d computes the hc rows g H + d of the up product for all rows, gates the
// normalised streams with them and averages: x[t, d] = Rb(mean_g Rb(Rb(sigmoid(Rb(up))) * n)).
__global__ void __launch_bounds__(256)
HcUpMixKernel(const __nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ norm_w, const __nv_bfloat16* __restrict__ Wup,
              const __nv_bfloat16* __restrict__ mid, const float* __restrict__ rstd, __nv_bfloat16* __restrict__ x, int T, int hc,
              int H, int L) {
  extern __shared__ float s_mid[];                      // [T][L]
  for (int i = threadIdx.x; i < T * L; i += blockDim.x) s_mid[i] = __bfloat162float(mid[i]);
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int d = blockIdx.x * 8 + warp;
  if (d >= H) return;
  const int C = hc * H;
  float out[kGateRows];
#pragma unroll
  for (int t = 0; t < kGateRows; ++t) out[t] = 0.f;
  for (int g = 0; g < hc; ++g) {
    const __nv_bfloat16* wrow = Wup + static_cast<size_t>(g * H + d) * L;
    float up[kGateRows];
#pragma unroll
    for (int t = 0; t < kGateRows; ++t) up[t] = 0.f;
    for (int j = lane * 2; j < L; j += 64) {
      const uint32_t wv = *reinterpret_cast<const uint32_t*>(wrow + j);
      const float w0 = BfLo(wv), w1 = BfHi(wv);
#pragma unroll
      for (int t = 0; t < kGateRows; ++t) {
        if (t >= T) break;
        up[t] += w0 * s_mid[t * L + j] + w1 * s_mid[t * L + j + 1];
      }
    }
    const float wn = 1.0f + __bfloat162float(norm_w[g * H + d]);
#pragma unroll
    for (int t = 0; t < kGateRows; ++t) {
      if (t >= T) break;
      const float u = WarpSum(up[t]);
      const float nv = Rb(__bfloat162float(h[static_cast<size_t>(t) * C + g * H + d]) * rstd[t * hc + g] * wn);
      out[t] += Rb(Rb(Sigmoid(Rb(u))) * nv);
    }
  }
  if (lane == 0)
    for (int t = 0; t < T; ++t) x[static_cast<size_t>(t) * H + d] = __float2bfloat16(out[t] / hc);
}

// h0[r, g H + d] = table[ids[r], d]
__global__ void EmbedRepeatKernel(const __nv_bfloat16* __restrict__ table, const int* __restrict__ ids, __nv_bfloat16* __restrict__ out,
                                  int rows, int vocab, int H, int hc) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * hc * H) return;
  const int r = i / (hc * H), d = (i - r * hc * H) % H;
  const int id = ids[r];
  out[i] = (id >= 0 && id < vocab) ? table[static_cast<size_t>(id) * H + d] : __float2bfloat16(nanf(""));
}

// ---- n-gram rows: ids hashed from the token history, rows gathered from the device table ---------------------------
struct NgramArgs {
  long long mult[3];
  unsigned long long primes[16];
  unsigned long long offsets[16];
  long long eos, rows;
  int heads, head_dim;
};

// grid (T, heads), 32 threads.  hist[p] = token at position p (written here for this call's rows).
__global__ void NgramGatherKernel(const int* __restrict__ ids, const int* __restrict__ positions, int* __restrict__ hist,
                                  const __nv_bfloat16* __restrict__ table, __nv_bfloat16* __restrict__ emb, NgramArgs a) {
  const int t = blockIdx.x, hd = blockIdx.y;
  const int p = positions[t];
  const long long tok = ids[t];
  long long s1 = a.eos, s2 = a.eos;
  if (p >= 1) s1 = t >= 1 ? ids[t - 1] : hist[p - 1];
  if (p >= 2) s2 = t >= 2 ? ids[t - 2] : hist[p - 2];
  if (s1 == a.eos || s2 == a.eos) s2 = a.eos;              // anything before the most recent end-of-sequence token reads as it
  if (hd == 0 && threadIdx.x == 0) hist[p] = static_cast<int>(tok);
  unsigned long long key = static_cast<unsigned long long>(tok * a.mult[0]) ^ static_cast<unsigned long long>(s1 * a.mult[1]);
  if (hd >= a.heads / 2) key ^= static_cast<unsigned long long>(s2 * a.mult[2]);
  const unsigned long long row = key % a.primes[hd] + a.offsets[hd];
  __nv_bfloat16* dst = emb + (static_cast<size_t>(t) * a.heads + hd) * a.head_dim;
  const bool ok = tok >= 0 && row < static_cast<unsigned long long>(a.rows);
  for (int d = threadIdx.x; d < a.head_dim; d += 32)
    dst[d] = ok ? table[row * a.head_dim + d] : __float2bfloat16(nanf(""));     // loud, never a silent zero row
}

// ---- n-gram layer: gate and gated value, grid (rows, hc), 256 threads ------------------------------------------------
__global__ void PleGateValueKernel(const float* __restrict__ kp, const __nv_bfloat16* __restrict__ h, const float* __restrict__ value,
                                   const __nv_bfloat16* __restrict__ wk, const __nv_bfloat16* __restrict__ wq,
                                   __nv_bfloat16* __restrict__ gv, int hc, int H, float eps) {
  __shared__ float red[32];
  const int r = blockIdx.x, g = blockIdx.y;
  const size_t base = (static_cast<size_t>(r) * hc + g) * H;
  const int wb = g * H;
  float sk = 0.f, sq = 0.f;
  for (int d = threadIdx.x; d < H; d += blockDim.x) {
    const float a = Rb(kp[base + d]), b = __bfloat162float(h[base + d]);
    sk += a * a;
    sq += b * b;
  }
  sk = BlockSum(sk, red);
  sq = BlockSum(sq, red);
  const float rk = rsqrtf(sk / H + eps), rq = rsqrtf(sq / H + eps);
  float dot = 0.f;
  for (int d = threadIdx.x; d < H; d += blockDim.x) {
    const float kn = Rb(Rb(kp[base + d]) * rk * (1.0f + __bfloat162float(wk[wb + d])));
    const float qn = Rb(__bfloat162float(h[base + d]) * rq * (1.0f + __bfloat162float(wq[wb + d])));
    dot += Rb(kn * qn);
  }
  dot = BlockSum(dot, red);
  float gate = Rb(Rb(dot) / sqrtf(static_cast<float>(H)));
  const float mag = Rb(sqrtf(fmaxf(fabsf(gate), 1e-6f)));
  gate = gate > 0.f ? mag : (gate < 0.f ? -mag : 0.f);
  const float sg = Rb(Sigmoid(gate));
  for (int d = threadIdx.x; d < H; d += blockDim.x)
    gv[base + d] = __float2bfloat16(sg * Rb(value[static_cast<size_t>(r) * H + d]));
}

// Dilated depthwise causal conv over the normalised gated values + silu + the layer's two adds; one thread per channel
// walks the rows in order.  ring [32][C]: the normalised gated value of position p sits in row p & 31.
__global__ void PleConvKernel(const __nv_bfloat16* __restrict__ gvn, const __nv_bfloat16* __restrict__ gv,
                              const __nv_bfloat16* __restrict__ cw, __nv_bfloat16* __restrict__ ring, __nv_bfloat16* __restrict__ h,
                              const int* __restrict__ positions, int rows, int C, int kernel, int dilation) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float w[8];
  for (int j = 0; j < kernel; ++j) w[j] = __bfloat162float(cw[static_cast<size_t>(c) * kernel + j]);
  for (int t = 0; t < rows; ++t) {
    const int p = positions[t];
    ring[static_cast<size_t>(p & 31) * C + c] = gvn[static_cast<size_t>(t) * C + c];
    float conv = 0.f;
    for (int j = 0; j < kernel; ++j) {
      const int src = p - (kernel - 1 - j) * dilation;
      if (src >= 0) conv += w[j] * __bfloat162float(ring[static_cast<size_t>(src & 31) * C + c]);
    }
    const size_t at = static_cast<size_t>(t) * C + c;
    h[at] = __float2bfloat16(__bfloat162float(h[at]) + Rb(__bfloat162float(gv[at]) + Rb(Silu(Rb(conv)))));
  }
}

// ---- block-selecting attention -------------------------------------------------------------------------------------
__device__ __forceinline__ void RopeAngles(int pos, int i, int rotary_dim, float theta, float* fs, float* fc) {
  const double inv = exp2(-log2(static_cast<double>(theta)) * (2.0 * i / rotary_dim));
  double s, c;
  sincos(static_cast<double>(pos) * inv, &s, &c);
  *fs = static_cast<float>(s);
  *fc = static_cast<float>(c);
}

// RMSNorm (1 + w) + partial NeoX rope of one Di-wide row held one element per thread (blockDim.x == Di)
__device__ __forceinline__ float NormRope(float x, const __nv_bfloat16* w, int pos, int Di, int rotary_dim, float theta, float eps,
                                          float* row, float* red) {
  const int d = threadIdx.x;
  const float ss = BlockSum(x * x, red);
  x = Rb(x * rsqrtf(ss / Di + eps) * (1.0f + __bfloat162float(w[d])));
  row[d] = x;
  __syncthreads();
  const int half = rotary_dim / 2;
  if (d < rotary_dim) {
    float fs, fc;
    RopeAngles(pos, d < half ? d : d - half, rotary_dim, theta, &fs, &fc);
    x = d < half ? row[d] * fc - row[d + half] * fs : row[d] * fc + row[d - half] * fs;
  }
  __syncthreads();
  return x;
}

// grid (T, Hi + 1), Di threads: indexer queries normed + roped; the raw key of position p stored at raw_keys[p]
__global__ void QsaIndexPrepKernel(const float* __restrict__ qk, const __nv_bfloat16* __restrict__ q_norm, const int* __restrict__ positions,
                                   __nv_bfloat16* __restrict__ idx_q, __nv_bfloat16* __restrict__ raw_keys, int Hi, int Di,
                                   int rotary_dim, float theta, float eps) {
  __shared__ float row[128], red[32];
  const int t = blockIdx.x, hh = blockIdx.y, d = threadIdx.x;
  const int pos = positions[t];
  const float x = Rb(qk[(static_cast<size_t>(t) * (Hi + 1) + hh) * Di + d]);
  if (hh == Hi) {
    raw_keys[static_cast<size_t>(pos) * Di + d] = __float2bfloat16(x);
    return;
  }
  const float y = NormRope(x, q_norm, pos, Di, rotary_dim, theta, eps, row, red);
  idx_q[(static_cast<size_t>(t) * Hi + hh) * Di + d] = __float2bfloat16(y);
}

// grid (T / ratio + 2), Di threads: block b = positions[0] / ratio + blockIdx.x is completed when its last position lies in
// this call's rows: mean of its raw keys (fp32, one rounding), RMSNorm, rope at the block's first position.
__global__ void QsaBlockKeysKernel(const __nv_bfloat16* __restrict__ raw_keys, const __nv_bfloat16* __restrict__ k_norm,
                                   const int* __restrict__ positions, __nv_bfloat16* __restrict__ block_keys, int T, int ratio, int Di,
                                   int rotary_dim, float theta, float eps) {
  __shared__ float row[128], red[32];
  const int p0 = positions[0], p1 = positions[T - 1];
  const int b = p0 / ratio + blockIdx.x;
  const int last = b * ratio + ratio - 1;
  if (last < p0 || last > p1) return;
  const int d = threadIdx.x;
  float s = 0.f;
  for (int j = 0; j < ratio; ++j) s += __bfloat162float(raw_keys[static_cast<size_t>(b * ratio + j) * Di + d]);
  const float x = Rb(s * (1.0f / ratio));
  const float y = NormRope(x, k_norm, b * ratio, Di, rotary_dim, theta, eps, row, red);
  block_keys[static_cast<size_t>(b) * Di + d] = __float2bfloat16(y);
}

// grid (ceil(nb_max / 256), T), 256 threads, one block key per thread: score = sum_h relu(q_h . k) / sqrt(Di)
__global__ void QsaScoresKernel(const __nv_bfloat16* __restrict__ idx_q, const __nv_bfloat16* __restrict__ block_keys,
                                const int* __restrict__ positions, float* __restrict__ scores, int Hi, int Di, int ratio, int topk,
                                int stride) {
  extern __shared__ float sq[];                         // [Hi][Di]
  const int t = blockIdx.y;
  const int nb = (positions[t] + 1) / ratio;
  if (nb <= topk) return;                               // a dense row
  for (int i = threadIdx.x; i < Hi * Di; i += blockDim.x) sq[i] = __bfloat162float(idx_q[static_cast<size_t>(t) * Hi * Di + i]);
  __syncthreads();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nb) return;
  const uint4* kr = reinterpret_cast<const uint4*>(block_keys + static_cast<size_t>(b) * Di);
  float acc[8];
  for (int h = 0; h < Hi; ++h) acc[h] = 0.f;
  for (int c = 0; c < Di / 8; ++c) {
    const uint4 v = kr[c];
    const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float k0 = BfLo(w4[j]), k1 = BfHi(w4[j]);
      for (int h = 0; h < Hi; ++h) acc[h] += sq[h * Di + c * 8 + 2 * j] * k0 + sq[h * Di + c * 8 + 2 * j + 1] * k1;
    }
  }
  float s = 0.f;
  for (int h = 0; h < Hi; ++h) s += fmaxf(acc[h], 0.f);
  scores[static_cast<size_t>(t) * stride + b] = s / sqrtf(static_cast<float>(Di));
}

// One CTA of 1024 threads per row: the exact top-`topk` blocks by (score descending, block index descending), written as
// ascending token lists, then the open tail.  The order is a total order on the 64-bit key (score bits << 32 | index)
// (scores are >= 0, so their bit patterns order like the values); the k-th largest key is found by an 8-pass radix
// select, every block whose key is at least that large is selected, and an ordered compaction writes them ascending.
constexpr int kSelThreads = 1024;
__global__ void __launch_bounds__(kSelThreads)
QsaSelectKernel(const float* __restrict__ scores, const int* __restrict__ positions, int* __restrict__ sel_tokens,
                int* __restrict__ sel_count, int ratio, int topk, int stride, int sel_stride) {
  __shared__ unsigned hist[256];
  __shared__ unsigned long long s_prefix;
  __shared__ int s_k, s_base;
  __shared__ int wsum[32];
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int nb = (pos + 1) / ratio;
  if (nb <= topk) {
    if (threadIdx.x == 0) sel_count[t] = -1;
    return;
  }
  const float* sc = scores + static_cast<size_t>(t) * stride;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  auto key_of = [&](int b) { return (static_cast<unsigned long long>(__float_as_uint(fmaxf(sc[b], 0.f))) << 32) | static_cast<unsigned>(b); };
  if (threadIdx.x == 0) { s_prefix = 0ull; s_k = topk; }
  for (int byte = 7; byte >= 0; --byte) {
    if (byte == 3) continue;                            // block indices stay below 2^24: this byte of every key is 0
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0u;
    __syncthreads();
    const unsigned long long prefix = s_prefix;
    const unsigned long long hi_mask = byte == 7 ? 0ull : (~0ull << (8 * (byte + 1)));
    for (int b = threadIdx.x; b < nb; b += blockDim.x) {
      const unsigned long long k = key_of(b);
      if ((k & hi_mask) == prefix) atomicAdd(&hist[(k >> (8 * byte)) & 0xFF], 1u);
    }
    __syncthreads();
    // the bin that holds the k-th largest: above(d) = count in bins > d, by a suffix scan over 256 bins (8 warps)
    const int kk = s_k;
    int above = 0, mine = 0;
    if (threadIdx.x < 256) {
      mine = static_cast<int>(hist[255 - threadIdx.x]);                      // thread i looks at bin 255 - i
      int incl = mine;
      for (int d = 1; d < 32; d <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += u;
      }
      if (lane == 31) wsum[warp] = incl;
      above = incl - mine;
    }
    __syncthreads();
    if (threadIdx.x < 256) {
      for (int w = 0; w < warp; ++w) above += wsum[w];
      if (above < kk && kk <= above + mine) {                                  // exactly one bin qualifies
        s_k = kk - above;
        s_prefix = prefix | (static_cast<unsigned long long>(255 - threadIdx.x) << (8 * byte));
      }
    }
    __syncthreads();
  }
  const unsigned long long kth = s_prefix;
  if (threadIdx.x == 0) s_base = 0;
  __syncthreads();
  int* out = sel_tokens + static_cast<size_t>(t) * sel_stride;
  for (int b0 = 0; b0 < nb; b0 += kSelThreads) {
    const int b = b0 + threadIdx.x;
    const int flag = (b < nb && key_of(b) >= kth) ? 1 : 0;
    int incl = flag;
    for (int d = 1; d < 32; d <<= 1) {
      const int u = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += u;
    }
    if (lane == 31) wsum[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int v = wsum[lane];
      for (int d = 1; d < 32; d <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, v, d);
        if (lane >= d) v += u;
      }
      wsum[lane] = v;                                   // inclusive over warps
    }
    __syncthreads();
    const int rank = s_base + (warp ? wsum[warp - 1] : 0) + incl - flag;
    if (flag)
      for (int j = 0; j < ratio; ++j) out[rank * ratio + j] = b * ratio + j;
    __syncthreads();
    if (threadIdx.x == 0) s_base += wsum[31];
    __syncthreads();
  }
  const int tail = pos + 1 - nb * ratio;
  if (threadIdx.x < tail) out[topk * ratio + threadIdx.x] = nb * ratio + threadIdx.x;
  if (threadIdx.x == 0) sel_count[t] = topk * ratio + tail;
}

// Attention partials over a row's token list (its selection, or every position up to its own when sel_count < 0).
// grid (nsplit, Hkv, T), G warps (one per query head of the KV head).  Tiles of 32 tokens: K and V rows (fp8) gathered
// into shared memory by all warps, lane j scores token j, then every lane accumulates its D / 32 output columns.
constexpr int kTile = 32;
template <int D>
__global__ void QsaAttnKernel(const __nv_bfloat16* __restrict__ q, const uint8_t* __restrict__ cache, const int* __restrict__ block_table,
                              const int* __restrict__ positions, const int* __restrict__ sel_tokens, const int* __restrict__ sel_count,
                              const float* __restrict__ k_descale, float* __restrict__ part_acc, float* __restrict__ part_ml, int Hq,
                              int Hkv, int sel_stride, int per_split) {
  constexpr int RS = D + 16;                            // padded row stride (bytes): 16-byte reads of 32 rows hit distinct banks
  constexpr int CPL = D / 32;                           // output columns per lane
  extern __shared__ __align__(16) unsigned char smem[];
  unsigned char* sk = smem;                             // [kTile][RS]
  unsigned char* sv = smem + kTile * RS;                // [kTile][RS]
  float* sq = reinterpret_cast<float*>(smem + 2 * kTile * RS);      // [G][D]
  int* stok = reinterpret_cast<int*>(sq + (Hq / Hkv) * D);          // [kTile]
  const int G = Hq / Hkv;
  const int split = blockIdx.x, hkv = blockIdx.y, t = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hq = hkv * G + warp;
  const int cnt = sel_count != nullptr ? sel_count[t] : -1;
  const int n = cnt < 0 ? positions[t] + 1 : cnt;
  const int lo = split * per_split, hi = min(n, lo + per_split);
  const int* toks = sel_tokens + static_cast<size_t>(t) * sel_stride;
  for (int i = threadIdx.x; i < G * D; i += blockDim.x)
    sq[i] = __bfloat162float(q[(static_cast<size_t>(t) * Hq + hkv * G) * D + i]);
  const float scale = rsqrtf(static_cast<float>(D)) * k_descale[hkv];
  float m = -INFINITY, l = 0.f, acc[CPL];
#pragma unroll
  for (int c = 0; c < CPL; ++c) acc[c] = 0.f;
  for (int base = lo; base < hi; base += kTile) {
    const int nt = min(kTile, hi - base);
    __syncthreads();                                    // the previous tile is consumed (and sq is written, first time)
    if (threadIdx.x < kTile) stok[threadIdx.x] = threadIdx.x < nt ? (cnt < 0 ? base + threadIdx.x : toks[base + threadIdx.x]) : 0;
    __syncthreads();
    // gather: 16-byte pieces, D / 16 per row and tensor
    for (int i = threadIdx.x; i < nt * (D / 16) * 2; i += blockDim.x) {
      const int which = i / (nt * (D / 16)), rem = i - which * nt * (D / 16);
      const int j = rem / (D / 16), c = rem - j * (D / 16);
      const int tok = stok[j];
      const int blk = block_table[tok >> 4], slot = tok & 15;
      const uint8_t* src = cache + ((static_cast<size_t>(blk) * Hkv + hkv) * 2 + which) * 16 * D + static_cast<size_t>(slot) * D + c * 16;
      *reinterpret_cast<uint4*>((which ? sv : sk) + j * RS + c * 16) = *reinterpret_cast<const uint4*>(src);
    }
    __syncthreads();
    float s = -INFINITY;
    if (lane < nt) {
      const float* qh = sq + warp * D;
      float dot = 0.f;
      for (int c = 0; c < D / 16; ++c) {
        const uint4 v = *reinterpret_cast<const uint4*>(sk + lane * RS + c * 16);
        const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const __half2_raw r0 = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w4[j] & 0xFFFF), __NV_E4M3);
          const __half2_raw r1 = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w4[j] >> 16), __NV_E4M3);
          const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&r0));
          const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&r1));
          const float* qq = qh + c * 16 + j * 4;
          dot += qq[0] * f0.x + qq[1] * f0.y + qq[2] * f1.x + qq[3] * f1.y;
        }
      }
      s = dot * scale;
    }
    const float mt = WarpMax(s);
    const float mn = fmaxf(m, mt);
    const float corr = __expf(m - mn);                  // m = -inf on the first tile: exp(-inf) = 0
    const float p = lane < nt ? __expf(s - mn) : 0.f;
    l = l * corr + WarpSum(p);
#pragma unroll
    for (int c = 0; c < CPL; ++c) acc[c] *= corr;
    m = mn;
    for (int j = 0; j < nt; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const unsigned char* vr = sv + j * RS + lane * CPL;
#pragma unroll
      for (int c = 0; c < CPL; c += 2) {
        const __half2_raw r = __nv_cvt_fp8x2_to_halfraw2(*reinterpret_cast<const __nv_fp8x2_storage_t*>(vr + c), __NV_E4M3);
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&r));
        acc[c] += pj * f.x;
        acc[c + 1] += pj * f.y;
      }
    }
  }
  const size_t pi = (static_cast<size_t>(t) * Hq + hq) * gridDim.x + split;
#pragma unroll
  for (int c = 0; c < CPL; ++c) part_acc[pi * D + lane * CPL + c] = acc[c];
  if (lane == 0) {
    part_ml[pi * 2] = m;
    part_ml[pi * 2 + 1] = l;
  }
}

// grid (T, Hq), D threads: merge the splits, descale, round, gate
__global__ void QsaCombineKernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml, const __nv_bfloat16* __restrict__ qg,
                                 const float* __restrict__ v_descale, __nv_bfloat16* __restrict__ out, int Hq, int Hkv, int D, int nsplit,
                                 int gated) {
  const int t = blockIdx.x, hq = blockIdx.y, d = threadIdx.x;
  const size_t pi = (static_cast<size_t>(t) * Hq + hq) * nsplit;
  float m = -INFINITY;
  for (int s = 0; s < nsplit; ++s) m = fmaxf(m, part_ml[(pi + s) * 2]);
  float l = 0.f, o = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float ms = part_ml[(pi + s) * 2];
    if (ms == -INFINITY) continue;                      // a split past the end of this row's list
    const float w = __expf(ms - m);
    l += part_ml[(pi + s) * 2 + 1] * w;
    o += part_acc[(pi + s) * D + d] * w;
  }
  o = Rb(o * v_descale[hq / (Hq / Hkv)] / l);
  if (gated) o *= Rb(Sigmoid(__bfloat162float(qg[(static_cast<size_t>(t) * Hq + hq) * 2 * D + D + d])));
  out[(static_cast<size_t>(t) * Hq + hq) * D + d] = __float2bfloat16(o);
}

inline dim3 Flat(long long n) { return dim3(static_cast<unsigned>((n + 255) / 256)); }

}  // namespace
}  // namespace r4dxb

using namespace r4dxb;

extern "C" {

int r4dxb_q4x_grouped_rmsnorm(const void* x, const void* w, void* out, int rows, int groups, int group_size, float eps, void* stream) {
  if (rows < 1 || groups < 1 || group_size < 1) return R4DXB_BAD_ARG;
  GroupedRmsNormKernel<<<dim3(rows, groups), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(out), groups, group_size, eps);
  return FinishLaunch();
}

int r4dxb_q4x_hc_mid(const float* down, void* mid, int rows, int lowrank, int stride, int hc, void* stream) {
  if (rows < 1 || lowrank < 1 || stride < lowrank || hc < 1) return R4DXB_BAD_ARG;
  HcMidKernel<<<Flat(static_cast<long long>(rows) * lowrank), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      down, static_cast<__nv_bfloat16*>(mid), rows, lowrank, stride, 1.0f / hc);
  return FinishLaunch();
}

int r4dxb_q4x_hc_mix(const void* n, const float* up, void* x, int rows, int hc, int hidden, void* stream) {
  if (rows < 1 || hc < 1 || hidden < 1) return R4DXB_BAD_ARG;
  HcMixKernel<<<Flat(static_cast<long long>(rows) * hidden), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(n), up, static_cast<__nv_bfloat16*>(x), rows, hc, hidden);
  return FinishLaunch();
}

int r4dxb_q4x_hc_inject(void* h, const void* block_out, const float* inject, int rows, int hc, int hidden, int stride, void* stream) {
  if (rows < 1 || hc < 1 || hidden < 1 || stride < hc) return R4DXB_BAD_ARG;
  HcInjectKernel<<<Flat(static_cast<long long>(rows) * hc * hidden), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(h), static_cast<const __nv_bfloat16*>(block_out), inject, rows, hc, hidden, stride);
  return FinishLaunch();
}

/* The whole gate in two launches for T <= 8 rows: mid [T, L] bf16 scratch, injv [T, n_inject] fp32 (the raw injection
 * logits; n_inject = 0 for the final mixer), rstd [T, hc] fp32 scratch, x [T, H] the block input.  w_down_inject: the down
 * rows followed by the inject rows, [L + n_inject, hc * H]. */
int r4dxb_q4x_hc_gate(const void* h, const void* norm_w, const void* w_down_inject, const void* w_up, void* mid, float* injv,
                      float* rstd, void* x, int T, int hc, int hidden, int lowrank, int n_inject, float eps, void* stream) {
  if (T < 1 || T > kGateRows || hc < 1 || hc > 8 || hidden % 8 || lowrank % 2 || lowrank < 2 || n_inject < 0) return R4DXB_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  HcDownKernel<<<lowrank + n_inject, kGateThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(h), static_cast<const __nv_bfloat16*>(norm_w),
                                                           static_cast<const __nv_bfloat16*>(w_down_inject), static_cast<__nv_bfloat16*>(mid),
                                                           injv, rstd, T, hc, hidden, lowrank, n_inject, eps);
  ++g_launch_count;
  const size_t smem = static_cast<size_t>(T) * lowrank * sizeof(float);
  HcUpMixKernel<<<(hidden + 7) / 8, 256, smem, s>>>(static_cast<const __nv_bfloat16*>(h), static_cast<const __nv_bfloat16*>(norm_w),
                                                    static_cast<const __nv_bfloat16*>(w_up), static_cast<const __nv_bfloat16*>(mid), rstd,
                                                    static_cast<__nv_bfloat16*>(x), T, hc, hidden, lowrank);
  return FinishLaunch();
}

int r4dxb_q4x_embed_repeat(const void* table, const int* ids, void* out, int rows, int vocab, int hidden, int hc, void* stream) {
  if (rows < 1 || hc < 1 || hidden < 1) return R4DXB_BAD_ARG;
  EmbedRepeatKernel<<<Flat(static_cast<long long>(rows) * hc * hidden), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(table), ids, static_cast<__nv_bfloat16*>(out), rows, vocab, hidden, hc);
  return FinishLaunch();
}

/* emb [T, heads * head_dim] = the table rows of the tokens; hist [max positions] is the device token history (read for
 * the two positions before the call's first rows, written for the call's rows). mult[3], primes[heads], offsets[heads]: host. */
int r4dxb_q4x_ngram_gather(const int* ids, const int* positions, int* hist, const void* table, void* emb, int T, int heads,
                           int head_dim, long long table_rows, const long long* mult, const unsigned long long* primes,
                           const unsigned long long* offsets, long long eos, void* stream) {
  if (T < 1 || heads < 2 || heads > 16 || heads % 2 || head_dim < 1) return R4DXB_BAD_ARG;
  NgramArgs a = {};
  for (int i = 0; i < 3; ++i) a.mult[i] = mult[i];
  for (int i = 0; i < heads; ++i) {
    if (primes[i] == 0) return R4DXB_BAD_ARG;
    a.primes[i] = primes[i];
    a.offsets[i] = offsets[i];
  }
  a.eos = eos; a.rows = table_rows; a.heads = heads; a.head_dim = head_dim;
  NgramGatherKernel<<<dim3(T, heads), 32, 0, static_cast<cudaStream_t>(stream)>>>(ids, positions, hist, static_cast<const __nv_bfloat16*>(table),
                                                                                 static_cast<__nv_bfloat16*>(emb), a);
  return FinishLaunch();
}

int r4dxb_q4x_ple_gate_value(const float* key_proj, const void* h, const float* value, const void* norm_key, const void* norm_query,
                             void* gated_value, int rows, int hc, int hidden, float eps, void* stream) {
  if (rows < 1 || hc < 1 || hidden < 1) return R4DXB_BAD_ARG;
  PleGateValueKernel<<<dim3(rows, hc), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      key_proj, static_cast<const __nv_bfloat16*>(h), value, static_cast<const __nv_bfloat16*>(norm_key),
      static_cast<const __nv_bfloat16*>(norm_query), static_cast<__nv_bfloat16*>(gated_value), hc, hidden, eps);
  return FinishLaunch();
}

int r4dxb_q4x_ple_conv(const void* gvn, const void* gated_value, const void* conv_w, void* ring, void* h, const int* positions,
                       int rows, int channels, int kernel, int dilation, void* stream) {
  if (rows < 1 || channels < 1 || kernel < 1 || kernel > 8 || dilation < 1 || (kernel - 1) * dilation >= 32) return R4DXB_BAD_ARG;
  PleConvKernel<<<Flat(channels), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gvn), static_cast<const __nv_bfloat16*>(gated_value), static_cast<const __nv_bfloat16*>(conv_w),
      static_cast<__nv_bfloat16*>(ring), static_cast<__nv_bfloat16*>(h), positions, rows, channels, kernel, dilation);
  return FinishLaunch();
}

/* Indexer half of an attention layer's prologue: qk [T, (Hi + 1) * Di] fp32 (the indexer projection), queries normed and
 * roped into idx_q [T, Hi, Di], raw keys stored by position, and the block keys of every block completed by these rows. */
int r4dxb_q4x_qsa_index(const float* qk, const void* q_norm, const void* k_norm, const int* positions, void* idx_q, void* raw_keys,
                        void* block_keys, int T, int Hi, int Di, int ratio, int rotary_dim, float theta, float eps, void* stream) {
  if (T < 1 || Hi < 1 || Hi > 8 || Di % 32 || Di > 128 || ratio < 1 || rotary_dim % 2 || rotary_dim > Di) return R4DXB_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  QsaIndexPrepKernel<<<dim3(T, Hi + 1), Di, 0, s>>>(qk, static_cast<const __nv_bfloat16*>(q_norm), positions, static_cast<__nv_bfloat16*>(idx_q),
                                                    static_cast<__nv_bfloat16*>(raw_keys), Hi, Di, rotary_dim, theta, eps);
  ++g_launch_count;
  QsaBlockKeysKernel<<<T / ratio + 2, Di, 0, s>>>(static_cast<const __nv_bfloat16*>(raw_keys), static_cast<const __nv_bfloat16*>(k_norm),
                                                  positions, static_cast<__nv_bfloat16*>(block_keys), T, ratio, Di, rotary_dim, theta, eps);
  return FinishLaunch();
}

/* Scores and selection for T rows; nb_max = the largest complete-block count among them (host-known: positions are
 * consecutive).  scores [T, stride] scratch; sel_tokens [T, sel_stride] with sel_stride >= topk * ratio + ratio - 1. */
int r4dxb_q4x_qsa_select(const void* idx_q, const void* block_keys, const int* positions, float* scores, int* sel_tokens, int* sel_count,
                         int T, int Hi, int Di, int ratio, int topk, int nb_max, int stride, int sel_stride, void* stream) {
  if (T < 1 || Hi < 1 || Hi > 8 || Di % 32 || Di > 128 || ratio < 1 || ratio > 32 || topk < 1 || nb_max > stride ||
      sel_stride < topk * ratio + ratio - 1)
    return R4DXB_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (nb_max > topk) {
    QsaScoresKernel<<<dim3((nb_max + 255) / 256, T), 256, Hi * Di * sizeof(float), s>>>(
        static_cast<const __nv_bfloat16*>(idx_q), static_cast<const __nv_bfloat16*>(block_keys), positions, scores, Hi, Di, ratio, topk, stride);
    ++g_launch_count;
  }
  QsaSelectKernel<<<T, kSelThreads, 0, s>>>(scores, positions, sel_tokens, sel_count, ratio, topk, stride, sel_stride);
  return FinishLaunch();
}

/* Attention over each row's token list + merge + output gate.  part_acc [T, Hq, nsplit, D], part_ml [T, Hq, nsplit, 2]. */
int r4dxb_q4x_qsa_attn(const void* q, const void* qg, const void* cache, const int* block_table, const int* positions,
                       const int* sel_tokens, const int* sel_count, const float* k_descale, const float* v_descale, float* part_acc,
                       float* part_ml, void* out, int T, int Hq, int Hkv, int D, int sel_stride, int max_tokens, int nsplit, int gated,
                       void* stream) {
  if (T < 1 || Hkv < 1 || Hq % Hkv || Hq / Hkv > 16 || (D != 64 && D != 128 && D != 256) || nsplit < 1 || max_tokens < 1)
    return R4DXB_BAD_ARG;
  const int G = Hq / Hkv;
  const int per = ((max_tokens + nsplit - 1) / nsplit + kTile - 1) / kTile * kTile;
  const size_t smem = 2 * kTile * (D + 16) + static_cast<size_t>(G) * D * sizeof(float) + kTile * sizeof(int);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const dim3 grid(nsplit, Hkv, T);
  auto launch = [&](auto kern) {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      if (e != cudaSuccess) return static_cast<int>(e);
    }
    kern<<<grid, G * 32, smem, s>>>(static_cast<const __nv_bfloat16*>(q), static_cast<const uint8_t*>(cache), block_table, positions, sel_tokens,
                                    sel_count, k_descale, part_acc, part_ml, Hq, Hkv, sel_stride, per);
    ++g_launch_count;
    return static_cast<int>(cudaGetLastError());
  };
  int rc = D == 256 ? launch(QsaAttnKernel<256>) : (D == 128 ? launch(QsaAttnKernel<128>) : launch(QsaAttnKernel<64>));
  if (rc) return rc;
  QsaCombineKernel<<<dim3(T, Hq), D, 0, s>>>(part_acc, part_ml, static_cast<const __nv_bfloat16*>(qg), v_descale,
                                             static_cast<__nv_bfloat16*>(out), Hq, Hkv, D, nsplit, gated);
  return FinishLaunch();
}

}  // extern "C"
