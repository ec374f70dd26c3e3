// Gated DeltaNet decode / verify step, fully fused: causal conv1d (width 4) + SiLU over a
// position-keyed ring, q/k L2 norm, gates, delta-rule recurrence on an fp32 state, gated RMSNorm.
//
// Per token and value head (reference math: tests/kernels/test_gdn_chunk_scan.cpp:5-11,
// third_party/libr4d/r4d.h:273-312):
//     S *= e^g;  u = beta (v - S k);  S += u k^T;  o = S q / sqrt(K);  out = rms(o) w silu(z)
//
// Speculation-safe state ("write once"): the kernel never writes the state its new rows produce.
// It logs (e^g, u, k) per row; the NEXT call first replays the accepted prefix of that log into the
// base state (n_replay rows, read from device memory) and stores it once.  Rejected rows simply
// are not replayed.  The conv ring is keyed by absolute position (slot = pos % 16), so rejected
// rows are overwritten by position, like KV rows.
//
// One CTA per value head (512 threads): warp w owns state rows w*D/16 .., a lane owns D/32
// consecutive K columns, so a state row is one coalesced 128-lane... 32-lane vector load.
#include "common.cuh"

namespace r4dxb {
namespace {

constexpr int kThreads = 512;
constexpr int kRing = 16;
constexpr int kMaxT = 8;

struct GdnArgs {
  const __nv_bfloat16* mixed;    // [T, conv_dim]  in_proj_qkv output (pre-conv)
  const __nv_bfloat16* z;        // [T, H*D]
  const float* ab;               // [T, 2H]: a then b
  const __nv_bfloat16* conv_w;   // [conv_dim, 4]
  const float* A_log;            // [H]
  const float* dt_bias;          // [H]
  const __nv_bfloat16* norm_w;   // [D]
  __nv_bfloat16* ring;           // [kRing, conv_dim]
  float* state;                  // [H, D, D]  (v-major rows, k columns)
  float* log_u;                  // [kMaxT, H, D]
  float* log_k;                  // [kMaxT, H, D]
  float* log_eg;                 // [kMaxT, H]
  const int* positions;          // [T] absolute positions of the rows (device)
  const int* n_replay;           // device scalar: rows of the previous log to commit first
  __nv_bfloat16* out;            // [T, H*D]
  int T, H, Hk, conv_dim;
  float eps;
  const int* row_slot;           // batched decode: grid.y = sequence b (one row each), its state lives in slot row_slot[b]
  // optional: the a / b projections computed here instead of read from `ab` (two K-long dot products per head and
  // row are too little work for a launch of their own): ab_w [2H, K] bf16 (a rows, then b rows), x [T, K] the
  // residual stream, in_norm_w [K] the layer's input RMSNorm weight (zero-centred), K columns
  const __nv_bfloat16* ab_w;
  const __nv_bfloat16* x;
  const __nv_bfloat16* in_norm_w;
  int K;
  float in_eps;
  int gate_act;                  // output gate of the norm: 0 silu(z), 1 sigmoid(z)
};

template <int D>
__global__ void __launch_bounds__(kThreads) GdnDecodeKernel(GdnArgs a) {
  PdlEnter();
  constexpr int RPW = D / 16;        // state rows per warp
  constexpr int CPL = D / 32;        // k columns per lane
  __shared__ float sq[kMaxT][D], sk[kMaxT][D], sv[kMaxT][D], so[kMaxT][D];
  __shared__ float seg[kMaxT], sbeta[kMaxT];
  __shared__ float rk[kMaxT][D], ru[kMaxT][D], reg[kMaxT];
  __shared__ float red[32], red2[32];
  if (a.row_slot != nullptr) {
    const int b = blockIdx.y, slot = a.row_slot[b];
    a.mixed += static_cast<size_t>(b) * a.conv_dim;
    a.z += static_cast<size_t>(b) * a.H * D;
    a.ab += static_cast<size_t>(b) * 2 * a.H;
    a.out += static_cast<size_t>(b) * a.H * D;
    a.positions += b;
    a.n_replay += slot;
    a.ring += static_cast<size_t>(slot) * kRing * a.conv_dim;
    a.state += static_cast<size_t>(slot) * a.H * D * D;
    a.log_u += static_cast<size_t>(slot) * kMaxT * a.H * D;
    a.log_k += static_cast<size_t>(slot) * kMaxT * a.H * D;
    a.log_eg += static_cast<size_t>(slot) * kMaxT * a.H;
  }
  const int h = blockIdx.x, hk = h / (a.H / a.Hk);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int T = a.T;
  const int key_dim = a.Hk * D;
  const int nrep = min(*a.n_replay, kMaxT);

  // ---- base state -> registers first: the kernel's largest load, independent of everything else, so it is in
  // flight while the conv / gate phase runs ------------------------------------------------------
  float S[RPW][CPL];
  float* base = a.state + static_cast<size_t>(h) * D * D;
#pragma unroll
  for (int r = 0; r < RPW; ++r) {
    const int v = warp * RPW + r;
    if constexpr (CPL == 4) {
      const float4 p = __ldcs(reinterpret_cast<const float4*>(base + static_cast<size_t>(v) * D + lane * 4));
      S[r][0] = p.x; S[r][1] = p.y; S[r][2] = p.z; S[r][3] = p.w;
    } else {
#pragma unroll
      for (int c = 0; c < CPL; ++c) S[r][c] = base[static_cast<size_t>(v) * D + lane * CPL + c];
    }
  }

  // ---- stage the previous log (before anything overwrites it) --------------------------------
  for (int i = threadIdx.x; i < nrep * D; i += kThreads) {
    const int r = i / D, c = i % D;
    rk[r][c] = a.log_k[(static_cast<size_t>(r) * a.H + h) * D + c];
    ru[r][c] = a.log_u[(static_cast<size_t>(r) * a.H + h) * D + c];
  }
  if (threadIdx.x < nrep) reg[threadIdx.x] = a.log_eg[threadIdx.x * a.H + h];

  // ---- phase A: ring write + conv + SiLU for this head's q, k, v channels ---------------------
  for (int i = threadIdx.x; i < T * 3 * D; i += kThreads) {
    const int t = i / (3 * D), j = i % (3 * D);
    const int part = j / D, c = j % D;
    const int ch = part == 0 ? hk * D + c : (part == 1 ? key_dim + hk * D + c : 2 * key_dim + h * D + c);
    const int pos = a.positions[t];
    const __nv_bfloat16 xin = a.mixed[static_cast<size_t>(t) * a.conv_dim + ch];
    a.ring[static_cast<size_t>(pos % kRing) * a.conv_dim + ch] = xin;
    // taps: weight index 3 multiplies the newest input
    const uint2 wv = *reinterpret_cast<const uint2*>(a.conv_w + static_cast<size_t>(ch) * 4);
    const float w0 = BfLo(wv.x), w1 = BfHi(wv.x), w2 = BfLo(wv.y), w3 = BfHi(wv.y);
    float acc = w3 * __bfloat162float(xin);
    // older inputs: rows of this call that precede t, else the ring
    auto past = [&](int back) -> float {
      const int p = pos - back;
      if (p < 0) return 0.f;
      if (t - back >= 0) return __bfloat162float(a.mixed[static_cast<size_t>(t - back) * a.conv_dim + ch]);
      return __bfloat162float(a.ring[static_cast<size_t>(p % kRing) * a.conv_dim + ch]);
    };
    acc += w2 * past(1) + w1 * past(2) + w0 * past(3);
    const float y = Silu(acc);
    if (part == 0) sq[t][c] = y; else if (part == 1) sk[t][c] = y; else sv[t][c] = y;
  }
  if (a.ab_w != nullptr) {
    // a[t, h] and b[t, h] = W rows . bf16(rmsnorm(x[t])): the same rounding points as the stand-alone kernel
    const __nv_bfloat16* wa = a.ab_w + static_cast<size_t>(h) * a.K;
    const __nv_bfloat16* wb = a.ab_w + static_cast<size_t>(a.H + h) * a.K;
    for (int t = 0; t < T; ++t) {
      const __nv_bfloat16* xr = a.x + static_cast<size_t>(t) * a.K;
      float ss = 0.f;
      for (int k = threadIdx.x * 2; k < a.K; k += kThreads * 2) {
        const uint32_t b = *reinterpret_cast<const uint32_t*>(xr + k);
        ss += BfLo(b) * BfLo(b) + BfHi(b) * BfHi(b);
      }
      const float r = rsqrtf(BlockSum(ss, red) / a.K + a.in_eps);
      float sa = 0.f, sb = 0.f;
      for (int k = threadIdx.x * 2; k < a.K; k += kThreads * 2) {
        const uint32_t b = *reinterpret_cast<const uint32_t*>(xr + k);
        const uint32_t g = *reinterpret_cast<const uint32_t*>(a.in_norm_w + k);
        const uint32_t hh = PackBf16(BfLo(b) * r * (1.f + BfLo(g)), BfHi(b) * r * (1.f + BfHi(g)));
        const uint32_t va = *reinterpret_cast<const uint32_t*>(wa + k), vb = *reinterpret_cast<const uint32_t*>(wb + k);
        sa += BfLo(va) * BfLo(hh) + BfHi(va) * BfHi(hh);
        sb += BfLo(vb) * BfLo(hh) + BfHi(vb) * BfHi(hh);
      }
      // both dot products through one block reduction (two values per warp slot)
      sa = WarpSum(sa);
      sb = WarpSum(sb);
      __syncthreads();
      if (lane == 0) { red[warp] = sa; red2[warp] = sb; }
      __syncthreads();
      sa = WarpSum(lane < kThreads / 32 ? red[lane] : 0.f);
      sb = WarpSum(lane < kThreads / 32 ? red2[lane] : 0.f);
      if (threadIdx.x == 0) {
        const float xs = sa + a.dt_bias[h];
        const float sp = xs > 20.f ? xs : log1pf(__expf(xs));
        seg[t] = __expf(-__expf(a.A_log[h]) * sp);
        sbeta[t] = Sigmoid(sb);
      }
    }
  } else if (threadIdx.x < T) {
    const int t = threadIdx.x;
    const float av = a.ab[static_cast<size_t>(t) * 2 * a.H + h], bv = a.ab[static_cast<size_t>(t) * 2 * a.H + a.H + h];
    const float xs = av + a.dt_bias[h];
    const float sp = xs > 20.f ? xs : log1pf(__expf(xs));
    seg[t] = __expf(-__expf(a.A_log[h]) * sp);
    sbeta[t] = Sigmoid(bv);
  }
  __syncthreads();
  // L2-normalise q and k rows (warp per row)
  for (int r = warp; r < 2 * T; r += kThreads / 32) {
    float* row = r < T ? sq[r] : sk[r - T];
    float ss = 0.f;
    for (int c = lane; c < D; c += 32) ss += row[c] * row[c];
    ss = WarpSum(ss);
    const float inv = rsqrtf(ss + 1e-6f);
    for (int c = lane; c < D; c += 32) row[c] *= inv;
  }
  __syncthreads();

  // ---- phase B: replay the accepted log prefix into the base state, store once ---------------------
  if (nrep > 0) {
    for (int i = 0; i < nrep; ++i) {
      const float eg = reg[i];
#pragma unroll
      for (int r = 0; r < RPW; ++r) {
        const float u = ru[i][warp * RPW + r];
#pragma unroll
        for (int c = 0; c < CPL; ++c) S[r][c] = fmaf(u, rk[i][lane * CPL + c], S[r][c] * eg);
      }
    }
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      const int v = warp * RPW + r;
      if constexpr (CPL == 4) {
        *reinterpret_cast<float4*>(base + static_cast<size_t>(v) * D + lane * 4) = make_float4(S[r][0], S[r][1], S[r][2], S[r][3]);
      } else {
#pragma unroll
        for (int c = 0; c < CPL; ++c) base[static_cast<size_t>(v) * D + lane * CPL + c] = S[r][c];
      }
    }
  }

  // ---- phase C: the new rows (state stays in registers; rows are logged, not stored) ----------
  const float scale = rsqrtf(static_cast<float>(D));
  for (int t = 0; t < T; ++t) {
    const float eg = seg[t], beta = sbeta[t];
    float kc[CPL], qc[CPL];
#pragma unroll
    for (int c = 0; c < CPL; ++c) { kc[c] = sk[t][lane * CPL + c]; qc[c] = sq[t][lane * CPL + c]; }
    float d1[RPW];
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      float s = 0.f;
#pragma unroll
      for (int c = 0; c < CPL; ++c) s = fmaf(S[r][c] * eg, kc[c], s);
      d1[r] = s;
    }
#pragma unroll
    for (int r = 0; r < RPW; ++r) d1[r] = WarpSum(d1[r]);
    float d2[RPW];
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      const int v = warp * RPW + r;
      const float u = beta * (sv[t][v] - d1[r]);
      float s = 0.f;
#pragma unroll
      for (int c = 0; c < CPL; ++c) {
        S[r][c] = fmaf(u, kc[c], S[r][c] * eg);
        s = fmaf(S[r][c], qc[c], s);
      }
      d2[r] = s;
      if (lane == 0) a.log_u[(static_cast<size_t>(t) * a.H + h) * D + v] = u;
    }
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      d2[r] = WarpSum(d2[r]);
      if (lane == 0) so[t][warp * RPW + r] = d2[r] * scale;
    }
    if (warp == 0) {
#pragma unroll
      for (int c = 0; c < CPL; ++c) a.log_k[(static_cast<size_t>(t) * a.H + h) * D + lane * CPL + c] = kc[c];
      if (lane == 0) a.log_eg[t * a.H + h] = eg;
    }
  }
  __syncthreads();

  // ---- phase D: gated RMSNorm ------------------------------------------------------------------
  for (int t = 0; t < T; ++t) {
    const float o = threadIdx.x < D ? so[t][threadIdx.x] : 0.f;
    const float ss = BlockSum(o * o, red);
    if (threadIdx.x < D) {
      const float r = rsqrtf(ss / D + a.eps);
      const float zv = __bfloat162float(a.z[(static_cast<size_t>(t) * a.H + h) * D + threadIdx.x]);
      a.out[(static_cast<size_t>(t) * a.H + h) * D + threadIdx.x] =
          __float2bfloat16(o * r * __bfloat162float(a.norm_w[threadIdx.x]) * (a.gate_act ? Sigmoid(zv) : Silu(zv)));
    }
  }
}

}  // namespace
}  // namespace r4dxb

/* ab_w != null: the a / b projections are computed inside the kernel from the residual rows x [T, K], the layer's
 * input RMSNorm weight and ab_w [2H, K] (a rows, then b rows); `ab` is then unused. */
static int GdnDecodeLaunch(const void* mixed, const void* z, const float* ab, const void* ab_w, const void* x,
                           const void* in_norm_w, int K, float in_eps, const void* conv_w,
                           const float* A_log, const float* dt_bias, const void* norm_w, void* ring,
                           float* state, float* log_u, float* log_k, float* log_eg, const int* positions,
                           const int* n_replay, void* out, int T, int H, int Hk, int D, float eps, int gate_act, void* stream) {
  using namespace r4dxb;
  if (T < 0 || T > kMaxT || H % Hk || (D != 128 && D != 64)) return R4DXB_BAD_ARG;
  if (ab_w != nullptr && (x == nullptr || in_norm_w == nullptr || K < 2 || K % 2)) return R4DXB_BAD_ARG;
  GdnArgs a;
  a.mixed = static_cast<const __nv_bfloat16*>(mixed);
  a.z = static_cast<const __nv_bfloat16*>(z);
  a.ab = ab;
  a.conv_w = static_cast<const __nv_bfloat16*>(conv_w);
  a.A_log = A_log;
  a.dt_bias = dt_bias;
  a.norm_w = static_cast<const __nv_bfloat16*>(norm_w);
  a.ring = static_cast<__nv_bfloat16*>(ring);
  a.state = state;
  a.log_u = log_u;
  a.log_k = log_k;
  a.log_eg = log_eg;
  a.positions = positions;
  a.n_replay = n_replay;
  a.out = static_cast<__nv_bfloat16*>(out);
  a.T = T;
  a.H = H;
  a.Hk = Hk;
  a.conv_dim = 2 * Hk * D + H * D;
  a.eps = eps;
  a.row_slot = nullptr;
  a.ab_w = static_cast<const __nv_bfloat16*>(ab_w);
  a.x = static_cast<const __nv_bfloat16*>(x);
  a.in_norm_w = static_cast<const __nv_bfloat16*>(in_norm_w);
  a.K = K;
  a.in_eps = in_eps;
  a.gate_act = gate_act;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (D == 128) return LaunchPdl(GdnDecodeKernel<128>, dim3(H), dim3(kThreads), 0, s, a);
  return LaunchPdl(GdnDecodeKernel<64>, dim3(H), dim3(kThreads), 0, s, a);
}

extern "C" int r4dxb_gdn_decode_ab(const void* mixed, const void* z, const float* ab, const void* ab_w, const void* x,
                                   const void* in_norm_w, int K, float in_eps, const void* conv_w,
                                   const float* A_log, const float* dt_bias, const void* norm_w, void* ring,
                                   float* state, float* log_u, float* log_k, float* log_eg, const int* positions,
                                   const int* n_replay, void* out, int T, int H, int Hk, int D, float eps, void* stream) {
  return GdnDecodeLaunch(mixed, z, ab, ab_w, x, in_norm_w, K, in_eps, conv_w, A_log, dt_bias, norm_w, ring, state, log_u, log_k,
                         log_eg, positions, n_replay, out, T, H, Hk, D, eps, 0, stream);
}

/* The step with the norm's output gate chosen by the caller (0 silu, 1 sigmoid: the qwen4_exp family; reference:
 * src/model/qwen4exp/include/r4dx/model/qwen4exp/gdn_sigmoid_norm.h:1-20). */
extern "C" int r4dxb_gdn_decode_gate(const void* mixed, const void* z, const float* ab, const void* conv_w,
                                     const float* A_log, const float* dt_bias, const void* norm_w, void* ring,
                                     float* state, float* log_u, float* log_k, float* log_eg, const int* positions,
                                     const int* n_replay, void* out, int T, int H, int Hk, int D, float eps, int gate_act,
                                     void* stream) {
  if (gate_act != 0 && gate_act != 1) return R4DXB_BAD_ARG;
  return GdnDecodeLaunch(mixed, z, ab, nullptr, nullptr, nullptr, 0, 0.f, conv_w, A_log, dt_bias, norm_w, ring, state, log_u,
                         log_k, log_eg, positions, n_replay, out, T, H, Hk, D, eps, gate_act, stream);
}

extern "C" int r4dxb_gdn_decode(const void* mixed, const void* z, const float* ab, const void* conv_w,
                                const float* A_log, const float* dt_bias, const void* norm_w, void* ring,
                                float* state, float* log_u, float* log_k, float* log_eg, const int* positions,
                                const int* n_replay, void* out, int T, int H, int Hk, int D, float eps, void* stream) {
  return r4dxb_gdn_decode_ab(mixed, z, ab, nullptr, nullptr, nullptr, 0, 0.f, conv_w, A_log, dt_bias, norm_w, ring, state, log_u,
                             log_k, log_eg, positions, n_replay, out, T, H, Hk, D, eps, stream);
}

/* Batched decode: B sequences, one row each; every per-sequence tensor (ring, state, logs, n_replay) carries a
 * leading slot dimension and row b uses slot row_slot[b]. */
extern "C" int r4dxb_gdn_decode_batch(const void* mixed, const void* z, const float* ab, const void* conv_w,
                                      const float* A_log, const float* dt_bias, const void* norm_w, void* ring,
                                      float* state, float* log_u, float* log_k, float* log_eg, const int* positions,
                                      const int* n_replay, const int* row_slot, void* out, int B, int H, int Hk, int D,
                                      float eps, void* stream) {
  using namespace r4dxb;
  if (B < 1 || H % Hk || (D != 128 && D != 64)) return R4DXB_BAD_ARG;
  GdnArgs a;
  a.mixed = static_cast<const __nv_bfloat16*>(mixed);
  a.z = static_cast<const __nv_bfloat16*>(z);
  a.ab = ab;
  a.conv_w = static_cast<const __nv_bfloat16*>(conv_w);
  a.A_log = A_log;
  a.dt_bias = dt_bias;
  a.norm_w = static_cast<const __nv_bfloat16*>(norm_w);
  a.ring = static_cast<__nv_bfloat16*>(ring);
  a.state = state; a.log_u = log_u; a.log_k = log_k; a.log_eg = log_eg;
  a.positions = positions;
  a.n_replay = n_replay;
  a.out = static_cast<__nv_bfloat16*>(out);
  a.T = 1; a.H = H; a.Hk = Hk; a.conv_dim = 2 * Hk * D + H * D; a.eps = eps;
  a.row_slot = row_slot;
  a.ab_w = nullptr; a.x = nullptr; a.in_norm_w = nullptr; a.K = 0; a.in_eps = 0.f; a.gate_act = 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (D == 128) return LaunchPdl(GdnDecodeKernel<128>, dim3(H, B), dim3(kThreads), 0, s, a);
  return LaunchPdl(GdnDecodeKernel<64>, dim3(H, B), dim3(kThreads), 0, s, a);
}
