// Gated DeltaNet over a long chunk of tokens (prefill): prep -> scan -> gated norm.
//
//   prep : depthwise causal conv1d (width 4) + SiLU on [q | k | v] channels, L2 norm of q and k per
//          head, gates e^g and beta; also refreshes the position-keyed conv ring
//          (reference splits the same work as conv_prep: third_party/libr4d/r4d.h:230-263).
//   scan : the delta-rule recurrence with the fp32 state held in registers for the whole chunk.
//          State rows are independent (u_v = beta (v_v - S[v,:] k), o_v = S[v,:] q), so a head is
//          split over 4 CTAs of 32 rows; 4 lanes share a row (32 K columns each) and meet in two
//          2-step shuffles per token.  q/k/v/gates stream through a double-buffered cp.async
//          pipeline of 16-token groups.
//   norm : out = rms(o) * w * silu(z), one warp per (token, head).
//
// The scan commits the state directly (prefill rows are never speculative); a pending decode log
// must have been committed first (r4dxb_gdn_decode with T = 0).
// The reference runs a chunked WY form on its matrix cores instead
// (reference: third_party/libr4d/r4d_gdn_chunk_scan_k128_v128_c64_bf16.hip:1-60).
#include <cuda_pipeline.h>

#include "common.cuh"

namespace r4dxb {
namespace {

constexpr int kRing = 16;

struct PrepArgs {
  const __nv_bfloat16* mixed;   // [T, conv_dim]
  const float* ab;              // [T, 2H]
  const __nv_bfloat16* conv_w;  // [conv_dim, 4]
  const float* A_log;
  const float* dt_bias;
  __nv_bfloat16* ring;          // [kRing, conv_dim]
  float* q;                     // [T, Hk, D] normalised
  float* k;                     // [T, Hk, D] normalised
  float* v;                     // [T, H, D]
  float* eg;                    // [T, H]
  float* beta;                  // [T, H]
  int T, H, Hk, D, conv_dim, pos0;
};

// grid T, 256 threads; a warp takes one head item (q head, k head or v head) at a time
__global__ void __launch_bounds__(256) GdnPrepKernel(PrepArgs a) {
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int D = a.D, key_dim = a.Hk * D;
  const int items = 2 * a.Hk + a.H;
  const int pos = a.pos0 + t;
  const int per_lane = D / 32;
  for (int item = warp; item < items; item += 8) {
    int ch0;
    float* dst;
    bool norm = true;
    if (item < a.Hk) { ch0 = item * D; dst = a.q + (static_cast<size_t>(t) * a.Hk + item) * D; }
    else if (item < 2 * a.Hk) { ch0 = key_dim + (item - a.Hk) * D; dst = a.k + (static_cast<size_t>(t) * a.Hk + item - a.Hk) * D; }
    else { ch0 = 2 * key_dim + (item - 2 * a.Hk) * D; dst = a.v + (static_cast<size_t>(t) * a.H + item - 2 * a.Hk) * D; norm = false; }
    float y[4];
    float ss = 0.f;
    for (int i = 0; i < per_lane; ++i) {
      const int ch = ch0 + lane * per_lane + i;
      const uint2 wv = *reinterpret_cast<const uint2*>(a.conv_w + static_cast<size_t>(ch) * 4);
      const float w0 = BfLo(wv.x), w1 = BfHi(wv.x), w2 = BfLo(wv.y), w3 = BfHi(wv.y);
      auto past = [&](int back) -> float {
        const int p = pos - back;
        if (p < 0) return 0.f;
        if (t - back >= 0) return __bfloat162float(a.mixed[static_cast<size_t>(t - back) * a.conv_dim + ch]);
        return __bfloat162float(a.ring[static_cast<size_t>(p % kRing) * a.conv_dim + ch]);
      };
      const float acc = w3 * past(0) + w2 * past(1) + w1 * past(2) + w0 * past(3);
      y[i] = Silu(acc);
      ss += y[i] * y[i];
    }
    if (norm) {
      ss = WarpSum(ss);
      const float inv = rsqrtf(ss + 1e-6f);
      for (int i = 0; i < per_lane; ++i) y[i] *= inv;
    }
    for (int i = 0; i < per_lane; ++i) dst[lane * per_lane + i] = y[i];
  }
  for (int h = threadIdx.x; h < a.H; h += 256) {
    const float av = a.ab[static_cast<size_t>(t) * 2 * a.H + h], bv = a.ab[static_cast<size_t>(t) * 2 * a.H + a.H + h];
    const float xs = av + a.dt_bias[h];
    const float sp = xs > 20.f ? xs : log1pf(__expf(xs));
    a.eg[static_cast<size_t>(t) * a.H + h] = __expf(-__expf(a.A_log[h]) * sp);
    a.beta[static_cast<size_t>(t) * a.H + h] = Sigmoid(bv);
  }
}

// ring refresh runs after prep (prep reads the ring rows of the previous chunk)
__global__ void GdnRingUpdateKernel(const __nv_bfloat16* __restrict__ mixed, __nv_bfloat16* __restrict__ ring, int T,
                                    int conv_dim, int pos0) {
  const int first = max(0, T - kRing);
  const int t = first + blockIdx.y;
  const int ch = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T || ch >= conv_dim) return;
  ring[static_cast<size_t>((pos0 + t) % kRing) * conv_dim + ch] = mixed[static_cast<size_t>(t) * conv_dim + ch];
}

constexpr int kGroup = 16;       // tokens per pipeline group

template <int D>
struct ScanSmem {
  float q[2][kGroup][D];
  float k[2][kGroup][D];
  float v[2][kGroup][32];
  float eg[2][kGroup];
  float beta[2][kGroup];
};

// grid (H, D/32), 128 threads: thread = (row r = tid / 4 of this CTA's 32 rows, K quarter c = tid % 4)
template <int D>
__global__ void __launch_bounds__(128) GdnScanKernel(const float* __restrict__ q, const float* __restrict__ k,
                                                     const float* __restrict__ v, const float* __restrict__ eg,
                                                     const float* __restrict__ beta, float* __restrict__ state,
                                                     float* __restrict__ o, int T, int H, int Hk) {
  constexpr int CPT = D / 4;       // K columns per thread
  extern __shared__ __align__(16) unsigned char smem_raw[];
  ScanSmem<D>& sm = *reinterpret_cast<ScanSmem<D>*>(smem_raw);
  const int h = blockIdx.x, rblk = blockIdx.y, hk = h / (H / Hk);
  const int tid = threadIdx.x, r = tid >> 2, c = tid & 3;
  const int row = rblk * 32 + r;
  float S[CPT];
  float* srow = state + (static_cast<size_t>(h) * D + row) * D + c * CPT;
#pragma unroll
  for (int i = 0; i < CPT; i += 4) {
    const float4 p = *reinterpret_cast<const float4*>(srow + i);
    S[i] = p.x; S[i + 1] = p.y; S[i + 2] = p.z; S[i + 3] = p.w;
  }
  const int groups = (T + kGroup - 1) / kGroup;
  auto issue = [&](int g, int buf) {
    const int tbase = g * kGroup;
    // q and k rows of the key head: kGroup x D floats each, 16-byte pieces
    for (int i = tid; i < kGroup * D / 4; i += 128) {
      const int tt = i / (D / 4), off = (i % (D / 4)) * 4;
      const int t = min(tbase + tt, T - 1);
      __pipeline_memcpy_async(&sm.q[buf][tt][off], q + (static_cast<size_t>(t) * Hk + hk) * D + off, 16);
      __pipeline_memcpy_async(&sm.k[buf][tt][off], k + (static_cast<size_t>(t) * Hk + hk) * D + off, 16);
    }
    for (int i = tid; i < kGroup * 8; i += 128) {
      const int tt = i / 8, off = (i % 8) * 4;
      const int t = min(tbase + tt, T - 1);
      __pipeline_memcpy_async(&sm.v[buf][tt][off], v + (static_cast<size_t>(t) * H + h) * D + rblk * 32 + off, 16);
    }
    if (tid < kGroup) {
      const int t = min(tbase + tid, T - 1);
      __pipeline_memcpy_async(&sm.eg[buf][tid], eg + static_cast<size_t>(t) * H + h, 4);
      __pipeline_memcpy_async(&sm.beta[buf][tid], beta + static_cast<size_t>(t) * H + h, 4);
    }
    __pipeline_commit();
  };
  issue(0, 0);
  const float scale = rsqrtf(static_cast<float>(D));
  for (int g = 0; g < groups; ++g) {
    const int buf = g & 1;
    if (g + 1 < groups) issue(g + 1, buf ^ 1);
    else __pipeline_commit();
    __pipeline_wait_prior(1);
    __syncthreads();
    const int nt = min(kGroup, T - g * kGroup);
    for (int tt = 0; tt < nt; ++tt) {
      const float e = sm.eg[buf][tt], b = sm.beta[buf][tt];
      const float* kp = &sm.k[buf][tt][c * CPT];
      const float* qp = &sm.q[buf][tt][c * CPT];
      float d0 = 0.f, d1 = 0.f;
#pragma unroll
      for (int i = 0; i < CPT; i += 4) {
        const float4 kv = *reinterpret_cast<const float4*>(kp + i);
        S[i] *= e; S[i + 1] *= e; S[i + 2] *= e; S[i + 3] *= e;
        d0 = fmaf(S[i], kv.x, d0); d1 = fmaf(S[i + 1], kv.y, d1);
        d0 = fmaf(S[i + 2], kv.z, d0); d1 = fmaf(S[i + 3], kv.w, d1);
      }
      float d = d0 + d1;
      d += __shfl_xor_sync(0xffffffffu, d, 1);
      d += __shfl_xor_sync(0xffffffffu, d, 2);
      const float u = b * (sm.v[buf][tt][r] - d);
      float o0 = 0.f, o1 = 0.f;
#pragma unroll
      for (int i = 0; i < CPT; i += 4) {
        const float4 kv = *reinterpret_cast<const float4*>(kp + i);
        const float4 qv = *reinterpret_cast<const float4*>(qp + i);
        S[i] = fmaf(u, kv.x, S[i]); S[i + 1] = fmaf(u, kv.y, S[i + 1]);
        S[i + 2] = fmaf(u, kv.z, S[i + 2]); S[i + 3] = fmaf(u, kv.w, S[i + 3]);
        o0 = fmaf(S[i], qv.x, o0); o1 = fmaf(S[i + 1], qv.y, o1);
        o0 = fmaf(S[i + 2], qv.z, o0); o1 = fmaf(S[i + 3], qv.w, o1);
      }
      float od = o0 + o1;
      od += __shfl_xor_sync(0xffffffffu, od, 1);
      od += __shfl_xor_sync(0xffffffffu, od, 2);
      if (c == 0) o[(static_cast<size_t>(g * kGroup + tt) * H + h) * D + row] = od * scale;
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < CPT; i += 4) *reinterpret_cast<float4*>(srow + i) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
}

// one warp per (token, head)
__global__ void GdnGatedNormKernel(const float* __restrict__ o, const __nv_bfloat16* __restrict__ z,
                                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out, long long rows,
                                   int D, float eps, int gate_act) {
  const long long item = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= rows) return;
  const int lane = threadIdx.x & 31;
  const int per = D / 32;
  float v[4];
  float ss = 0.f;
  for (int i = 0; i < per; ++i) {
    v[i] = o[item * D + lane * per + i];
    ss += v[i] * v[i];
  }
  ss = WarpSum(ss);
  const float r = rsqrtf(ss / D + eps);
  for (int i = 0; i < per; ++i) {
    const int d = lane * per + i;
    const float zv = __bfloat162float(z[item * D + d]);
    out[item * D + d] = __float2bfloat16(v[i] * r * __bfloat162float(w[d]) * (gate_act ? Sigmoid(zv) : Silu(zv)));
  }
}

}  // namespace

int LaunchGdnChunked(const float* q, const float* k, const float* v, const float* eg, const float* beta, float* state, float* o,
                     float* ws, int T, int H, int Hk, cudaStream_t s);   // gdn_chunk.cu

}  // namespace r4dxb

using namespace r4dxb;

extern "C" {

/* scratch (fp32): q [T,Hk,D], k [T,Hk,D], v [T,H,D], eg [T,H], beta [T,H], o [T,H,D];
 * ws: optional workspace of r4dxb_gdn_chunk_ws_floats(T, H) floats - with it, D = 128 and T >= 128 the
 * recurrence runs in its chunked tensor-core form, otherwise token by token */
int r4dxb_gdn_prefill_gate(const void* mixed, const void* z, const float* ab, const void* conv_w, const float* A_log,
                           const float* dt_bias, const void* norm_w, void* ring, float* state, float* q, float* k, float* v,
                           float* eg, float* beta, float* o, void* out, int T, int H, int Hk, int D, int pos0, float eps,
                           float* ws, int gate_act, void* stream);

int r4dxb_gdn_prefill(const void* mixed, const void* z, const float* ab, const void* conv_w, const float* A_log,
                      const float* dt_bias, const void* norm_w, void* ring, float* state, float* q, float* k, float* v,
                      float* eg, float* beta, float* o, void* out, int T, int H, int Hk, int D, int pos0, float eps,
                      float* ws, void* stream) {
  return r4dxb_gdn_prefill_gate(mixed, z, ab, conv_w, A_log, dt_bias, norm_w, ring, state, q, k, v, eg, beta, o, out, T, H, Hk, D,
                                pos0, eps, ws, 0, stream);
}

/* the same prefill with the norm's output gate chosen by the caller: 0 silu(z), 1 sigmoid(z) */
int r4dxb_gdn_prefill_gate(const void* mixed, const void* z, const float* ab, const void* conv_w, const float* A_log,
                           const float* dt_bias, const void* norm_w, void* ring, float* state, float* q, float* k, float* v,
                           float* eg, float* beta, float* o, void* out, int T, int H, int Hk, int D, int pos0, float eps,
                           float* ws, int gate_act, void* stream) {
  if (T < 1 || H % Hk || (D != 128 && D != 64) || (gate_act != 0 && gate_act != 1)) return R4DXB_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  PrepArgs a;
  a.mixed = static_cast<const __nv_bfloat16*>(mixed);
  a.ab = ab;
  a.conv_w = static_cast<const __nv_bfloat16*>(conv_w);
  a.A_log = A_log;
  a.dt_bias = dt_bias;
  a.ring = static_cast<__nv_bfloat16*>(ring);
  a.q = q; a.k = k; a.v = v; a.eg = eg; a.beta = beta;
  a.T = T; a.H = H; a.Hk = Hk; a.D = D; a.conv_dim = 2 * Hk * D + H * D; a.pos0 = pos0;
  GdnPrepKernel<<<T, 256, 0, s>>>(a);
  int e = FinishLaunch();
  if (e) return e;
  GdnRingUpdateKernel<<<dim3((a.conv_dim + 255) / 256, min(T, kRing)), 256, 0, s>>>(a.mixed, a.ring, T, a.conv_dim, pos0);
  e = FinishLaunch();
  if (e) return e;
  if (D == 128 && ws != nullptr && T >= 128) {
    e = LaunchGdnChunked(q, k, v, eg, beta, state, o, ws, T, H, Hk, s);
    if (e) return e;
  } else if (D == 128) {
    const int smem = sizeof(ScanSmem<128>);
    cudaFuncSetAttribute(GdnScanKernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    GdnScanKernel<128><<<dim3(H, 4), 128, smem, s>>>(q, k, v, eg, beta, state, o, T, H, Hk);
  } else {
    const int smem = sizeof(ScanSmem<64>);
    GdnScanKernel<64><<<dim3(H, 2), 128, smem, s>>>(q, k, v, eg, beta, state, o, T, H, Hk);
  }
  e = FinishLaunch();      // (a second check after the chunked path is harmless)
  if (e) return e;
  const long long rows = static_cast<long long>(T) * H;
  GdnGatedNormKernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, s>>>(
      o, static_cast<const __nv_bfloat16*>(z), static_cast<const __nv_bfloat16*>(norm_w),
      static_cast<__nv_bfloat16*>(out), rows, D, eps, gate_act);
  return FinishLaunch();
}

}  // extern "C"
