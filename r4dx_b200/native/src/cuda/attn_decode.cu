// Gated full attention for T <= 8 query rows (decode / speculative verify) over an fp8 e4m3
// paged KV cache with 16-token blocks.
//
//   precore : per-head q|gate split, zero-centred RMSNorm on q and k, partial NeoX rope, fp8
//             quantisation of k and v with a static per-head descale, paged cache write
//             (reference fuses the same steps: src/kernels/src/r4dx_kernels.hip:647).
//   decode  : split-KV flash decoding; one CTA per (split, kv head) walks its share of the
//             sequence's blocks, all gqa*T query rows of the kv head at once, and writes an
//             (m, l, acc) partial (reference: third_party/libr4d/r4d_attn_decode_h256_gqa6.hip:1-16).
//   combine : merges the partials, applies o * sigmoid(gate), one bf16 rounding.
//
// Cache layout: [block][kv_head][2 (K, V)][16 tokens][D] fp8 -- a K tile and a V tile of one
// block are each one contiguous 16*D byte run.  The sequence length is read from device memory
// (positions[T-1] + 1) so that a captured CUDA graph can be replayed as the context grows.
#include <cuda_pipeline.h>

#include "common.cuh"

namespace r4dxb {
namespace {

constexpr int kBlockTokens = 16;
constexpr int kTileTokens = 64;    // decode attention works on four cache blocks at a time

__device__ __forceinline__ uint8_t ToFp8(float v) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}

__device__ __forceinline__ __half2 Fp8x2ToHalf2(uint16_t v) {
  __half2_raw r = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(v), __NV_E4M3);
  return *reinterpret_cast<__half2*>(&r);
}

struct PrecoreArgs {
  const __nv_bfloat16* qg;     // [T, Hq, 2D]
  const __nv_bfloat16* k;      // [T, Hkv, D]
  const __nv_bfloat16* v;      // [T, Hkv, D]
  const __nv_bfloat16* q_norm; // [D]
  const __nv_bfloat16* k_norm; // [D]
  const float* k_descale;      // [Hkv]
  const float* v_descale;      // [Hkv]
  const int* positions;        // [T]
  const int* block_table;      // [max_blocks]
  __nv_bfloat16* q_out;        // [T, Hq, D]
  uint8_t* cache;
  int T, Hq, Hkv, D, rotary_dim;
  int q_stride;                // elements between consecutive heads of qg (2D with the gate half, D without)
  float theta, eps;
  const int* row_slot;         // batched decode: row t belongs to sequence slot row_slot[t] (null: one sequence)
  int table_stride;            // ints between the block tables of consecutive slots
};

// grid (Hq + 2 Hkv, T), block D threads (one element each)
__global__ void PrecoreKernel(PrecoreArgs a) {
  PdlEnter();
  extern __shared__ float row[];
  __shared__ float red[32];
  const int t = blockIdx.y, hh = blockIdx.x, d = threadIdx.x, D = a.D;
  const int pos = a.positions[t];
  int kind, head;   // 0 = q, 1 = k, 2 = v
  if (hh < a.Hq) { kind = 0; head = hh; }
  else if (hh < a.Hq + a.Hkv) { kind = 1; head = hh - a.Hq; }
  else { kind = 2; head = hh - a.Hq - a.Hkv; }
  float x;
  if (kind == 0) x = __bfloat162float(a.qg[(static_cast<size_t>(t) * a.Hq + head) * a.q_stride + d]);
  else if (kind == 1) x = __bfloat162float(a.k[(static_cast<size_t>(t) * a.Hkv + head) * D + d]);
  else x = __bfloat162float(a.v[(static_cast<size_t>(t) * a.Hkv + head) * D + d]);
  if (kind != 2) {
    const __nv_bfloat16* nw = kind == 0 ? a.q_norm : a.k_norm;
    if (nw != nullptr) {        // families without per-head q/k normalisation pass null
      const float ss = BlockSum(x * x, red);
      x = x * rsqrtf(ss / D + a.eps) * (1.0f + __bfloat162float(nw[d]));
    }
    row[d] = x;
    __syncthreads();
    const int half = a.rotary_dim / 2;
    if (d < a.rotary_dim) {
      const int i = d < half ? d : d - half;
      const double inv = exp2(-log2(static_cast<double>(a.theta)) * (2.0 * i / a.rotary_dim));
      double s, c;
      sincos(static_cast<double>(pos) * inv, &s, &c);
      const float fs = static_cast<float>(s), fc = static_cast<float>(c);
      x = d < half ? row[d] * fc - row[d + half] * fs : row[d] * fc + row[d - half] * fs;
    }
  }
  if (kind == 0) {
    a.q_out[(static_cast<size_t>(t) * a.Hq + head) * D + d] = __float2bfloat16(x);
  } else {
    const int* table = a.row_slot ? a.block_table + static_cast<size_t>(a.row_slot[t]) * a.table_stride : a.block_table;
    const int blk = table[pos / kBlockTokens], tok = pos % kBlockTokens;
    const float ds = (kind == 1 ? a.k_descale : a.v_descale)[head];
    uint8_t* dst = a.cache + ((static_cast<size_t>(blk) * a.Hkv + head) * 2 + (kind - 1)) * kBlockTokens * D;
    dst[tok * D + d] = ToFp8(x / ds);
  }
}

struct DecodeArgs {
  const __nv_bfloat16* q;      // [T, Hq, D] (normed + roped)
  const uint8_t* cache;
  const int* block_table;
  const int* positions;        // [T]
  const float* k_descale;
  const float* v_descale;
  float* part_acc;             // [splits, Hkv, G, D]
  float* part_ml;              // [splits, Hkv, G, 2]
  int T, Hq, Hkv, D, splits;
  const int* row_slot;         // batched decode (grid.z = sequence, one query row each); null otherwise
  int table_stride;
  int window;                  // sliding-window length in tokens (0: the whole sequence is visible)
};

// grid (splits, Hkv), 256 threads.  G = gqa * T query rows, row g = t * gqa + j.
template <int GMAX>
__global__ void __launch_bounds__(256) DecodeKernel(DecodeArgs a) {
  PdlEnter();
  extern __shared__ __align__(16) unsigned char smem[];
  if (a.row_slot != nullptr) {
    // one CTA column per sequence: shift every per-sequence pointer, then proceed as a 1-row call
    const int b = blockIdx.z;
    a.q += static_cast<size_t>(b) * a.Hq * a.D;
    a.positions += b;
    a.block_table += static_cast<size_t>(a.row_slot[b]) * a.table_stride;
    const size_t per = static_cast<size_t>(a.splits) * a.Hkv * (a.Hq / a.Hkv);
    a.part_acc += b * per * a.D;
    a.part_ml += b * per * 2;
  }
  const int D = a.D, gqa = a.Hq / a.Hkv, G = gqa * a.T;
  const int split = blockIdx.x, hkv = blockIdx.y, tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int KS = D + 16;                          // padded K row stride (bytes) against bank conflicts
  // a tile is four cache blocks (64 tokens); two tiles of raw fp8 rows are in flight (cp.async double buffer)
  uint8_t* Kt = smem;                              // [2][64][KS]
  uint8_t* Vt = Kt + 2 * kTileTokens * KS;         // [2][64][D]
  __half* qs = reinterpret_cast<__half*>(Vt + 2 * kTileTokens * D);   // [GMAX][D]
  float* P = reinterpret_cast<float*>(qs + GMAX * D);                 // [GMAX][64]
  float* mrow = P + GMAX * kTileTokens;            // [GMAX]
  float* lrow = mrow + GMAX;
  float* arow = lrow + GMAX;                       // per-tile rescale factor
  int* qpos = reinterpret_cast<int*>(arow + GMAX); // [GMAX] position of each query row

  const int seqlen = a.positions[a.T - 1] + 1;
  const int nblocks = (seqlen + kBlockTokens - 1) / kBlockTokens;
  // sliding window: the oldest key any row of this call may see opens the range
  const int first_blk = a.window > 0 ? max(0, a.positions[0] - a.window + 1) / kBlockTokens : 0;
  const int per = ((((nblocks - first_blk) + a.splits - 1) / a.splits) + 3) & ~3;     // blocks per split, whole tiles
  const int b0 = first_blk + split * per, b1 = min(nblocks, b0 + per);
  const int ntiles = b1 > b0 ? (b1 - b0 + 3) / 4 : 0;

  auto issue = [&](int tile, int buf) {
    const int vpb = D;                              // 16-byte vectors per (block, K or V): 16 tokens x D bytes
    for (int i = tid; i < 2 * 4 * vpb; i += 256) {
      const int kv = i / (4 * vpb), r = i % (4 * vpb);
      const int bi = r / vpb, v = r % vpb;
      const int b = b0 + tile * 4 + bi;
      uint8_t* dst = kv == 0 ? Kt + (static_cast<size_t>(buf) * kTileTokens + bi * kBlockTokens + (v * 16) / D) * KS + (v * 16) % D
                             : Vt + (static_cast<size_t>(buf) * kTileTokens + bi * kBlockTokens) * D + v * 16;
      if (b < b1) {
        const int blk = a.block_table[b];
        const uint8_t* src = a.cache + ((static_cast<size_t>(blk) * a.Hkv + hkv) * 2 + kv) * kBlockTokens * D + v * 16;
        __pipeline_memcpy_async(dst, src, 16);
      } else {
        *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);     // past the end: zeros (masked, but never NaN)
      }
    }
    __pipeline_commit();
  };
  if (ntiles > 0) issue(0, 0);

  const float sm_scale = rsqrtf(static_cast<float>(D)) * a.k_descale[hkv] * 1.4426950408889634f;  // into log2 domain
  for (int i = tid; i < GMAX * D; i += 256) {
    const int g = i / D, d = i % D;
    float v = 0.f;
    if (g < G) {
      const int t = g / gqa, j = g % gqa;
      v = __bfloat162float(a.q[(static_cast<size_t>(t) * a.Hq + hkv * gqa + j) * D + d]) * sm_scale;
    }
    qs[i] = __float2half(v);
  }
  if (tid < GMAX) {
    mrow[tid] = -INFINITY;
    lrow[tid] = 0.f;
    qpos[tid] = tid < G ? a.positions[tid / gqa] : -1;
  }
  float acc[GMAX];
#pragma unroll
  for (int g = 0; g < GMAX; ++g) acc[g] = 0.f;

  for (int tile = 0; tile < ntiles; ++tile) {
    const int buf = tile & 1;
    __pipeline_wait_prior(0);
    __syncthreads();                 // this tile's rows have landed; the previous tile is fully consumed by every thread
    if (tile + 1 < ntiles) issue(tile + 1, buf ^ 1);      // its buffer was last read two tiles ago; overlaps the math below
    const uint8_t* Kb = Kt + static_cast<size_t>(buf) * kTileTokens * KS;
    const uint8_t* Vb = Vt + static_cast<size_t>(buf) * kTileTokens * D;
    const int kp0 = (b0 + tile * 4) * kBlockTokens;
    // scores: one thread per (g, tok)
    for (int i = tid; i < G * kTileTokens; i += 256) {
      const int g = i / kTileTokens, tok = i % kTileTokens;
      float s = -INFINITY;
      if (kp0 + tok <= qpos[g] && (a.window == 0 || kp0 + tok > qpos[g] - a.window)) {
        const uint2* kr = reinterpret_cast<const uint2*>(Kb + tok * KS);
        const uint4* qr = reinterpret_cast<const uint4*>(qs + g * D);
        float sum = 0.f;
        for (int c = 0; c < D / 8; ++c) {
          const uint2 kv = kr[c];
          const uint4 qv = qr[c];
          __half2 p = __hmul2(Fp8x2ToHalf2(kv.x & 0xFFFF), *reinterpret_cast<const __half2*>(&qv.x));
          p = __hfma2(Fp8x2ToHalf2(kv.x >> 16), *reinterpret_cast<const __half2*>(&qv.y), p);
          p = __hfma2(Fp8x2ToHalf2(kv.y & 0xFFFF), *reinterpret_cast<const __half2*>(&qv.z), p);
          p = __hfma2(Fp8x2ToHalf2(kv.y >> 16), *reinterpret_cast<const __half2*>(&qv.w), p);
          sum += __low2float(p) + __high2float(p);
        }
        s = sum;
      }
      P[i] = s;
    }
    __syncthreads();
    // online softmax (log2 domain): one warp per query row, two tokens per lane
    for (int g = warp; g < G; g += 8) {
      const float s0 = P[g * kTileTokens + lane], s1 = P[g * kTileTokens + 32 + lane];
      const float m_old = mrow[g];
      const float mx = WarpMax(fmaxf(m_old, fmaxf(s0, s1)));
      const float alpha = (mx == -INFINITY) ? 1.f : exp2f(m_old - mx);
      const float p0 = (s0 == -INFINITY) ? 0.f : exp2f(s0 - mx), p1 = (s1 == -INFINITY) ? 0.f : exp2f(s1 - mx);
      P[g * kTileTokens + lane] = p0;
      P[g * kTileTokens + 32 + lane] = p1;
      const float l = lrow[g] * alpha + WarpSum(p0 + p1);
      __syncwarp();
      if (lane == 0) {
        mrow[g] = mx;
        lrow[g] = l;
        arow[g] = alpha;
      }
    }
    __syncthreads();
    // PV: thread owns one output dim for every query row
    if (tid < D) {
#pragma unroll
      for (int g = 0; g < GMAX; ++g)
        if (g < G) acc[g] *= arow[g];
#pragma unroll 8
      for (int tok = 0; tok < kTileTokens; ++tok) {
        const __half_raw hr = __nv_cvt_fp8_to_halfraw(Vb[tok * D + tid], __NV_E4M3);
        const float v = __half2float(*reinterpret_cast<const __half*>(&hr));
#pragma unroll
        for (int g = 0; g < GMAX; ++g)
          if (g < G) acc[g] = fmaf(P[g * kTileTokens + tok], v, acc[g]);
      }
    }
  }
  __pipeline_wait_prior(0);
  const float vds = a.v_descale[hkv];
  const size_t base = (static_cast<size_t>(split) * a.Hkv + hkv) * G;
  if (tid < D) {
#pragma unroll
    for (int g = 0; g < GMAX; ++g)
      if (g < G) a.part_acc[(base + g) * D + tid] = acc[g] * vds;
  }
  if (tid < G) {
    a.part_ml[(base + tid) * 2] = mrow[tid];
    a.part_ml[(base + tid) * 2 + 1] = lrow[tid];
  }
}

// grid (G, Hkv), D threads
__global__ void CombineKernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                              const __nv_bfloat16* __restrict__ qg, __nv_bfloat16* __restrict__ out, int T, int Hq,
                              int Hkv, int D, int splits, int gated, int batched) {
  PdlEnter();
  const int g = blockIdx.x, hkv = blockIdx.y, d = threadIdx.x;
  const int gqa = Hq / Hkv, G = gqa * T;
  if (batched) {
    const int b = blockIdx.z;
    const size_t per = static_cast<size_t>(splits) * Hkv * G;
    part_acc += b * per * D;
    part_ml += b * per * 2;
    qg += static_cast<size_t>(b) * Hq * 2 * D;
    out += static_cast<size_t>(b) * Hq * D;
  }
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, part_ml[((static_cast<size_t>(s) * Hkv + hkv) * G + g) * 2]);
  float num = 0.f, den = 0.f;
  for (int s = 0; s < splits; ++s) {
    const size_t r = (static_cast<size_t>(s) * Hkv + hkv) * G + g;
    const float m = part_ml[r * 2];
    if (m == -INFINITY) continue;
    const float w = exp2f(m - M);
    num += w * part_acc[r * D + d];
    den += w * part_ml[r * 2 + 1];
  }
  float o = den > 0.f ? num / den : 0.f;
  const int t = g / gqa, hq = hkv * gqa + g % gqa;
  if (gated) {
    const float gate = __bfloat162float(qg[(static_cast<size_t>(t) * Hq + hq) * 2 * D + D + d]);
    o *= Sigmoid(gate);
  }
  out[(static_cast<size_t>(t) * Hq + hq) * D + d] = __float2bfloat16(o);
}

template <int GMAX>
int LaunchDecode(const DecodeArgs& a, cudaStream_t s, int batch = 1) {
  const int D = a.D;
  const size_t smem = 2 * kTileTokens * (D + 16) + 2 * kTileTokens * D + static_cast<size_t>(GMAX) * D * 2 +
                      static_cast<size_t>(GMAX) * kTileTokens * 4 + GMAX * 4 * 4;
  auto kern = DecodeKernel<GMAX>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  return LaunchPdl(kern, dim3(a.splits, a.Hkv, batch), dim3(256), smem, s, a);
}

}  // namespace
}  // namespace r4dxb

using namespace r4dxb;

extern "C" {

int r4dxb_attn_precore(const void* qg, const void* k, const void* v, const void* q_norm, const void* k_norm,
                       const float* k_descale, const float* v_descale, const int* positions, const int* block_table,
                       void* q_out, void* cache, int T, int Hq, int Hkv, int D, int rotary_dim, float theta, float eps,
                       int q_stride, void* stream) {
  if (T < 1 || D > 1024 || D % 32 || rotary_dim > D || rotary_dim % 2) return R4DXB_BAD_ARG;
  PrecoreArgs a;
  a.qg = static_cast<const __nv_bfloat16*>(qg);
  a.k = static_cast<const __nv_bfloat16*>(k);
  a.v = static_cast<const __nv_bfloat16*>(v);
  a.q_norm = static_cast<const __nv_bfloat16*>(q_norm);
  a.k_norm = static_cast<const __nv_bfloat16*>(k_norm);
  a.k_descale = k_descale;
  a.v_descale = v_descale;
  a.positions = positions;
  a.block_table = block_table;
  a.q_out = static_cast<__nv_bfloat16*>(q_out);
  a.cache = static_cast<uint8_t*>(cache);
  a.T = T; a.Hq = Hq; a.Hkv = Hkv; a.D = D; a.rotary_dim = rotary_dim; a.theta = theta; a.eps = eps;
  a.row_slot = nullptr; a.table_stride = 0;
  a.q_stride = q_stride > 0 ? q_stride : 2 * D;
  return LaunchPdl(PrecoreKernel, dim3(Hq + 2 * Hkv, T), dim3(D), D * sizeof(float), static_cast<cudaStream_t>(stream), a);
}

/* scratch: part_acc = splits*Hkv*G*D floats, part_ml = splits*Hkv*G*2 floats (G = Hq/Hkv*T) */
int r4dxb_attn_decode(const void* q, const void* qg, const void* cache, const int* block_table, const int* positions,
                      const float* k_descale, const float* v_descale, float* part_acc, float* part_ml, void* out,
                      int T, int Hq, int Hkv, int D, int splits, int flags, void* stream) {
  const int gated = flags & 1;      // bit 0: sigmoid output gate; bits 1..: sliding-window length (0 = none)
  if (T < 1 || T > 8 || Hq % Hkv || D % 16 || D > 256 || splits < 1) return R4DXB_BAD_ARG;
  const int G = Hq / Hkv * T;
  DecodeArgs a;
  a.q = static_cast<const __nv_bfloat16*>(q);
  a.cache = static_cast<const uint8_t*>(cache);
  a.block_table = block_table;
  a.positions = positions;
  a.k_descale = k_descale;
  a.v_descale = v_descale;
  a.part_acc = part_acc;
  a.part_ml = part_ml;
  a.T = T; a.Hq = Hq; a.Hkv = Hkv; a.D = D; a.splits = splits;
  a.row_slot = nullptr; a.table_stride = 0;
  a.window = flags >> 1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int e;
  if (G <= 8) e = LaunchDecode<8>(a, s);
  else if (G <= 16) e = LaunchDecode<16>(a, s);
  else if (G <= 32) e = LaunchDecode<32>(a, s);
  else if (G <= 64) e = LaunchDecode<64>(a, s);
  else return R4DXB_UNSUPPORTED;
  if (e) return e;
  return LaunchPdl(CombineKernel, dim3(G, Hkv), dim3(D), 0, s, static_cast<const float*>(part_acc), static_cast<const float*>(part_ml),
                   static_cast<const __nv_bfloat16*>(qg), static_cast<__nv_bfloat16*>(out), T, Hq, Hkv, D, splits, gated, 0);
}

/* Batched decode: B sequences, one new token each.  Row b belongs to slot row_slot[b]; block tables are
 * [slots][table_stride]; the cache is one shared block pool.  Scratch sized B x (single-sequence scratch at T=1). */
int r4dxb_attn_precore_batch(const void* qg, const void* k, const void* v, const void* q_norm, const void* k_norm,
                             const float* k_descale, const float* v_descale, const int* positions, const int* block_tables,
                             const int* row_slot, int table_stride, void* q_out, void* cache, int B, int Hq, int Hkv, int D,
                             int rotary_dim, float theta, float eps, int q_stride, void* stream) {
  if (B < 1 || D > 1024 || D % 32 || rotary_dim > D || rotary_dim % 2) return R4DXB_BAD_ARG;
  PrecoreArgs a;
  a.qg = static_cast<const __nv_bfloat16*>(qg);
  a.k = static_cast<const __nv_bfloat16*>(k);
  a.v = static_cast<const __nv_bfloat16*>(v);
  a.q_norm = static_cast<const __nv_bfloat16*>(q_norm);
  a.k_norm = static_cast<const __nv_bfloat16*>(k_norm);
  a.k_descale = k_descale; a.v_descale = v_descale; a.positions = positions; a.block_table = block_tables;
  a.q_out = static_cast<__nv_bfloat16*>(q_out);
  a.cache = static_cast<uint8_t*>(cache);
  a.T = B; a.Hq = Hq; a.Hkv = Hkv; a.D = D; a.rotary_dim = rotary_dim; a.theta = theta; a.eps = eps;
  a.row_slot = row_slot; a.table_stride = table_stride;
  a.q_stride = q_stride > 0 ? q_stride : 2 * D;
  return LaunchPdl(PrecoreKernel, dim3(Hq + 2 * Hkv, B), dim3(D), D * sizeof(float), static_cast<cudaStream_t>(stream), a);
}

int r4dxb_attn_decode_batch(const void* q, const void* qg, const void* cache, const int* block_tables, const int* row_slot,
                            int table_stride, const int* positions, const float* k_descale, const float* v_descale,
                            float* part_acc, float* part_ml, void* out, int B, int Hq, int Hkv, int D, int splits, int flags,
                            void* stream) {
  const int gated = flags & 1;
  if (B < 1 || Hq % Hkv || D % 16 || D > 256 || splits < 1 || Hq / Hkv > 64) return R4DXB_BAD_ARG;
  const int G = Hq / Hkv;
  DecodeArgs a;
  a.q = static_cast<const __nv_bfloat16*>(q);
  a.cache = static_cast<const uint8_t*>(cache);
  a.block_table = block_tables;
  a.positions = positions;
  a.k_descale = k_descale; a.v_descale = v_descale; a.part_acc = part_acc; a.part_ml = part_ml;
  a.T = 1; a.Hq = Hq; a.Hkv = Hkv; a.D = D; a.splits = splits;
  a.row_slot = row_slot; a.table_stride = table_stride;
  a.window = flags >> 1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int e;
  if (G <= 8) e = LaunchDecode<8>(a, s, B);
  else if (G <= 16) e = LaunchDecode<16>(a, s, B);
  else if (G <= 32) e = LaunchDecode<32>(a, s, B);
  else e = LaunchDecode<64>(a, s, B);
  if (e) return e;
  CombineKernel<<<dim3(G, Hkv, B), D, 0, s>>>(part_acc, part_ml, static_cast<const __nv_bfloat16*>(qg),
                                              static_cast<__nv_bfloat16*>(out), 1, Hq, Hkv, D, splits, gated, 1);
  return FinishLaunch();
}

}  // extern "C"
