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
bool g_decode_row = true;

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

// ---- one query token, at most 8 query heads per KV head: the shape of every decode step ----------------------
// Split-KV like DecodeKernel, but every warp walks its own 16-token cache blocks from global memory to registers
// with no block-wide barrier in the loop, so the eight warps of a CTA keep eight blocks (64 KiB per SM) in flight:
//   scores  : mma.sync m16n8k16, A = the query rows (fp16, pre-scaled, kept in registers for the whole kernel),
//             B = K read as fp8 and widened in registers.  The k index of the MMA is a permutation of the head
//             dimensions chosen so that a lane's B values are 16 consecutive cache bytes (one 128-bit load).
//   softmax : per row inside a lane quad (two shuffles), log2 domain, running (m, l) per row.
//   P V     : CUDA cores; a lane owns D / 32 output dimensions of all rows, P is handed over through a small
//             per-warp shared-memory tile as (p, p) half pairs, fp16 FMAs per block folded into fp32 sums.
// The warps' partials are merged through shared memory, the CTA writes one (m, l, acc) partial like DecodeKernel.
template <int D>
__global__ void __launch_bounds__(256, 1) DecodeRowKernel(DecodeArgs a) {
  PdlEnter();
  constexpr int DPL = D / 32;                   // output dimensions per lane
  constexpr int NJ = D / 64;                    // 64-dimension groups: one 128-bit K load per lane each
  extern __shared__ __align__(16) unsigned char smem[];
  if (a.row_slot != nullptr) {
    const int b = blockIdx.z;
    a.q += static_cast<size_t>(b) * a.Hq * D;
    a.positions += b;
    a.block_table += static_cast<size_t>(a.row_slot[b]) * a.table_stride;
    const size_t per = static_cast<size_t>(a.splits) * a.Hkv * (a.Hq / a.Hkv);
    a.part_acc += b * per * D;
    a.part_ml += b * per * 2;
  }
  const int G = a.Hq / a.Hkv;                   // <= 8, T == 1
  const int split = blockIdx.x, hkv = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gid = lane >> 2, c = lane & 3;
  __half2* P2 = reinterpret_cast<__half2*>(smem) + warp * (16 * 8 + 8);          // [16 tokens][8 rows] (p, p) + 8 alphas (as float)
  float* alpha_s = reinterpret_cast<float*>(P2 + 16 * 8);
  float* merge = reinterpret_cast<float*>(smem + 8 * (16 * 8 + 8) * 4);          // [4][8 rows][D + 2]

  const int pos = a.positions[0];
  const int seqlen = pos + 1;
  const int nblocks = (seqlen + kBlockTokens - 1) / kBlockTokens;
  const int first_tok = a.window > 0 ? max(0, pos - a.window + 1) : 0;
  const int first_blk = first_tok / kBlockTokens;
  const int per = ((nblocks - first_blk) + a.splits - 1) / a.splits;
  const int b0 = first_blk + split * per, b1 = min(nblocks, b0 + per);

  // query rows as MMA A fragments: lane holds Q[gid][64 j + 16 c .. + 16) for every j (rows >= G are zero)
  const float sm_scale = rsqrtf(static_cast<float>(D)) * a.k_descale[hkv] * 1.4426950408889634f;   // into the log2 domain
  uint32_t qa[NJ][8];
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
#pragma unroll
    for (int i = 0; i < 8; ++i) qa[j][i] = 0u;
    if (gid < G) {
      const __nv_bfloat16* qr = a.q + (static_cast<size_t>(hkv) * G + gid) * D + 64 * j + 16 * c;
      const uint4 v0 = *reinterpret_cast<const uint4*>(qr), v1 = *reinterpret_cast<const uint4*>(qr + 8);
      const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const __half2 h = __floats2half2_rn(BfLo(w[i]) * sm_scale, BfHi(w[i]) * sm_scale);
        qa[j][i] = *reinterpret_cast<const uint32_t*>(&h);
      }
    }
  }
  float m_run = -INFINITY, l_run = 0.f;          // of row gid (identical in the four lanes of a quad)
  float acc[8][DPL];
#pragma unroll
  for (int g = 0; g < 8; ++g)
#pragma unroll
    for (int d = 0; d < DPL; ++d) acc[g][d] = 0.f;

  for (int b = b0 + warp; b < b1; b += 8) {
    const int blk = a.block_table[b];
    const uint8_t* kb = a.cache + (static_cast<size_t>(blk) * a.Hkv + hkv) * 2 * kBlockTokens * D;
    const uint8_t* vb = kb + kBlockTokens * D;
    // ---- scores of the block's 16 tokens: two 8-token MMA tiles ----
    uint4 kraw[2][NJ];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int j = 0; j < NJ; ++j)
        kraw[nt][j] = __ldg(reinterpret_cast<const uint4*>(kb + (8 * nt + gid) * D + 64 * j + 16 * c));
    // V of the block: the lane's DPL bytes of each of the 16 token rows (issued now, used after the softmax)
    uint32_t vraw[16][(DPL + 3) / 4];
#pragma unroll
    for (int t = 0; t < 16; ++t) {
      if constexpr (DPL == 8) {
        const uint2 v = __ldg(reinterpret_cast<const uint2*>(vb + t * D + 8 * lane));
        vraw[t][0] = v.x; vraw[t][1] = v.y;
      } else if constexpr (DPL == 4) {
        vraw[t][0] = __ldg(reinterpret_cast<const uint32_t*>(vb + t * D + 4 * lane));
      } else {
        vraw[t][0] = __ldg(reinterpret_cast<const uint16_t*>(vb + t * D + 2 * lane));
      }
    }
    float sc[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        const uint32_t kw[4] = {kraw[nt][j].x, kraw[nt][j].y, kraw[nt][j].z, kraw[nt][j].w};
#pragma unroll
        for (int st = 0; st < 4; ++st) {        // four k-steps of 16 (permuted) dimensions out of the 16 loaded bytes
          const __half2 b0h = Fp8x2ToHalf2(static_cast<uint16_t>(kw[st] & 0xFFFFu));
          const __half2 b1h = Fp8x2ToHalf2(static_cast<uint16_t>(kw[st] >> 16));
          const uint32_t zero = 0u;
          asm volatile(
              "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
              : "+f"(sc[nt][0]), "+f"(sc[nt][1]), "+f"(sc[nt][2]), "+f"(sc[nt][3])
              : "r"(qa[j][2 * st]), "r"(zero), "r"(qa[j][2 * st + 1]), "r"(zero),
                "r"(*reinterpret_cast<const uint32_t*>(&b0h)), "r"(*reinterpret_cast<const uint32_t*>(&b1h)));
        }
      }
    }
    // ---- mask + online softmax of row gid over the 16 tokens (lane holds tokens 8 nt + 2 c, + 1) ----
    float s4[4];
    float mx = m_run;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int kp = b * kBlockTokens + 8 * nt + 2 * c + e;
        const bool ok = kp <= pos && kp >= first_tok;
        s4[nt * 2 + e] = ok ? sc[nt][e] : -INFINITY;
        mx = fmaxf(mx, s4[nt * 2 + e]);
      }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float alpha = (mx == -INFINITY) ? 1.f : exp2f(m_run - mx);
    float psum = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float p = (s4[i] == -INFINITY) ? 0.f : exp2f(s4[i] - mx);
      psum += p;
      const int tok = 8 * (i >> 1) + 2 * c + (i & 1);
      P2[tok * 8 + gid] = __float2half2_rn(p);
    }
    psum += __shfl_xor_sync(0xffffffffu, psum, 1);
    psum += __shfl_xor_sync(0xffffffffu, psum, 2);
    l_run = l_run * alpha + psum;
    m_run = mx;
    if (c == 0) alpha_s[gid] = alpha;
    __syncwarp();
    // ---- P V: every lane, its DPL dimensions, all rows ----
    {
      const float4 a0 = *reinterpret_cast<const float4*>(alpha_s), a1 = *reinterpret_cast<const float4*>(alpha_s + 4);
      const float al[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      __half2 hacc[8][(DPL + 1) / 2];
#pragma unroll
      for (int g = 0; g < 8; ++g)
#pragma unroll
        for (int d = 0; d < (DPL + 1) / 2; ++d) hacc[g][d] = __float2half2_rn(0.f);
#pragma unroll
      for (int t = 0; t < 16; ++t) {
        __half2 vh[(DPL + 1) / 2];
#pragma unroll
        for (int d = 0; d < (DPL + 1) / 2; ++d)
          vh[d] = Fp8x2ToHalf2(static_cast<uint16_t>((vraw[t][d / 2] >> (16 * (d & 1))) & 0xFFFFu));
        const uint4 p0 = *reinterpret_cast<const uint4*>(P2 + t * 8), p1 = *reinterpret_cast<const uint4*>(P2 + t * 8 + 4);
        const uint32_t pw[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const __half2 pg = *reinterpret_cast<const __half2*>(&pw[g]);
#pragma unroll
          for (int d = 0; d < (DPL + 1) / 2; ++d) hacc[g][d] = __hfma2(pg, vh[d], hacc[g][d]);
        }
      }
#pragma unroll
      for (int g = 0; g < 8; ++g)
#pragma unroll
        for (int d = 0; d < DPL; ++d) {
          const float add = (d & 1) ? __high2float(hacc[g][d / 2]) : __low2float(hacc[g][d / 2]);
          acc[g][d] = acc[g][d] * al[g] + add;
        }
    }
    __syncwarp();                                // the tile is rewritten by the next block
  }

  // ---- merge the eight warps: 4-7 into 0-3, 2-3 into 0-1, 1 into 0 (row statistics travel with the sums) ----
  // every lane needs (m, l) of all rows: publish the quad's values per warp first
  alpha_s[gid] = m_run;                          // all four lanes of a quad write the same value
  __syncwarp();
  float mrow[8], lrow[8];
  {
    const float4 a0 = *reinterpret_cast<const float4*>(alpha_s), a1 = *reinterpret_cast<const float4*>(alpha_s + 4);
    mrow[0] = a0.x; mrow[1] = a0.y; mrow[2] = a0.z; mrow[3] = a0.w; mrow[4] = a1.x; mrow[5] = a1.y; mrow[6] = a1.z; mrow[7] = a1.w;
  }
  __syncwarp();
  alpha_s[gid] = l_run;
  __syncwarp();
  {
    const float4 a0 = *reinterpret_cast<const float4*>(alpha_s), a1 = *reinterpret_cast<const float4*>(alpha_s + 4);
    lrow[0] = a0.x; lrow[1] = a0.y; lrow[2] = a0.z; lrow[3] = a0.w; lrow[4] = a1.x; lrow[5] = a1.y; lrow[6] = a1.z; lrow[7] = a1.w;
  }
  constexpr int MS = D + 2;                      // floats per row in the merge buffer: D sums, m, l
  for (int half = 4; half >= 1; half >>= 1) {
    __syncthreads();
    if (warp >= half && warp < 2 * half) {
      float* dst = merge + static_cast<size_t>(warp - half) * 8 * MS;
#pragma unroll
      for (int g = 0; g < 8; ++g) {
#pragma unroll
        for (int d = 0; d < DPL; ++d) dst[g * MS + DPL * lane + d] = acc[g][d];
        if (lane == 0) { dst[g * MS + D] = mrow[g]; dst[g * MS + D + 1] = lrow[g]; }
      }
    }
    __syncthreads();
    if (warp < half) {
      const float* src = merge + static_cast<size_t>(warp) * 8 * MS;
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        const float mo = src[g * MS + D], lo = src[g * MS + D + 1];
        const float mn = fmaxf(mrow[g], mo);
        const float wa = (mrow[g] == -INFINITY) ? 0.f : exp2f(mrow[g] - mn);
        const float wb = (mo == -INFINITY) ? 0.f : exp2f(mo - mn);
#pragma unroll
        for (int d = 0; d < DPL; ++d) acc[g][d] = acc[g][d] * wa + src[g * MS + DPL * lane + d] * wb;
        lrow[g] = lrow[g] * wa + lo * wb;
        mrow[g] = mn;
      }
    }
  }
  if (warp == 0) {
    const float vds = a.v_descale[hkv];
    const size_t base = (static_cast<size_t>(split) * a.Hkv + hkv) * G;
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      if (g < G) {
#pragma unroll
        for (int d = 0; d < DPL; ++d) a.part_acc[(base + g) * D + DPL * lane + d] = acc[g][d] * vds;
        if (lane == 0) {
          a.part_ml[(base + g) * 2] = mrow[g];
          a.part_ml[(base + g) * 2 + 1] = lrow[g];
        }
      }
    }
  }
}

template <int D>
int LaunchDecodeRow(const DecodeArgs& a, cudaStream_t s, int batch) {
  const size_t smem = 8 * (16 * 8 + 8) * 4 + static_cast<size_t>(4) * 8 * (D + 2) * 4;
  return LaunchPdl(DecodeRowKernel<D>, dim3(a.splits, a.Hkv, batch), dim3(256), smem, s, a);
}

// grid (G * D / 32, Hkv [, B]), 256 threads = 32 output columns x 8 groups of splits.  Every thread has all of its
// splits' partial sums in flight at once (8 loads for 64 splits), so the kernel is two dependent memory round trips
// (statistics, partial sums) whatever the number of heads: with three query heads per rank the one-CTA-per-head
// form took 19 us, longer than the attention itself.
constexpr int kCombineThreads = 256;
__global__ void __launch_bounds__(kCombineThreads)
CombineKernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
              const __nv_bfloat16* __restrict__ qg, __nv_bfloat16* __restrict__ out, int T, int Hq,
              int Hkv, int D, int splits, int gated, int batched) {
  PdlEnter();
  const int chunks = (D + 31) / 32;
  const int g = blockIdx.x / chunks, dchunk = blockIdx.x % chunks, hkv = blockIdx.y;
  const int lane = threadIdx.x & 31, sg = threadIdx.x >> 5;
  const int d = dchunk * 32 + lane;
  const int gqa = Hq / Hkv, G = gqa * T;
  if (batched) {
    const int b = blockIdx.z;
    const size_t per = static_cast<size_t>(splits) * Hkv * G;
    part_acc += b * per * D;
    part_ml += b * per * 2;
    qg += static_cast<size_t>(b) * Hq * 2 * D;
    out += static_cast<size_t>(b) * Hq * D;
  }
  __shared__ float wsm[kCombineThreads], lsm[kCombineThreads];
  __shared__ float red[8];
  __shared__ float nsum[8][32], dsum[8];
  float M = -INFINITY, num = 0.f, den = 0.f;
  for (int s0 = 0; s0 < splits; s0 += kCombineThreads) {     // one round for up to 256 splits
    const int ns = min(kCombineThreads, splits - s0);
    float m = -INFINITY, l = 0.f;
    if (static_cast<int>(threadIdx.x) < ns) {
      const size_t r = (static_cast<size_t>(s0 + threadIdx.x) * Hkv + hkv) * G + g;
      m = part_ml[r * 2];
      l = part_ml[r * 2 + 1];
    }
    float mx = WarpMax(m);
    __syncthreads();
    if (lane == 0) red[sg] = mx;
    __syncthreads();
    mx = red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) mx = fmaxf(mx, red[w]);
    const float Mn = fmaxf(M, mx);
    const float keep = (M == -INFINITY) ? 0.f : exp2f(M - Mn);
    {
      const float w = (m == -INFINITY) ? 0.f : exp2f(m - Mn);
      wsm[threadIdx.x] = w;                // threads past ns hold m = -inf: weight 0
      lsm[threadIdx.x] = w * l;
    }
    __syncthreads();
    num *= keep;
    den *= keep;
    M = Mn;
    const float* pa = part_acc + ((static_cast<size_t>(s0) * Hkv + hkv) * G + g) * D + d;
    const size_t stride = static_cast<size_t>(Hkv) * G * D;
    for (int sb = sg; sb < ns; sb += 64) {                    // 8 splits of this thread per pass, loads issued together
      float v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = (sb + 8 * i < ns && d < D) ? __ldcs(pa + static_cast<size_t>(sb + 8 * i) * stride) : 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (sb + 8 * i < ns) {
          num += wsm[sb + 8 * i] * v[i];
          den += lsm[sb + 8 * i];
        }
      }
    }
  }
  nsum[sg][lane] = num;
  if (lane == 0) dsum[sg] = den;
  __syncthreads();
  if (sg == 0 && d < D) {
    float n = 0.f, dn = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      n += nsum[w][lane];
      dn += dsum[w];
    }
    float o = dn > 0.f ? n / dn : 0.f;
    const int t = g / gqa, hq = hkv * gqa + g % gqa;
    if (gated) {
      const float gate = __bfloat162float(qg[(static_cast<size_t>(t) * Hq + hq) * 2 * D + D + d]);
      o *= Sigmoid(gate);
    }
    out[(static_cast<size_t>(t) * Hq + hq) * D + d] = __float2bfloat16(o);
  }
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

/* A/B switch: 1 (default) = one-token decode steps use the warp-autonomous kernel, 0 = the tiled kernel for every shape. */
void r4dxb_set_attn_decode_row(int on) { g_decode_row = on != 0; }

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
  if (T == 1 && G <= 8 && g_decode_row && (D == 256 || D == 128 || D == 64)) {
    e = D == 256 ? LaunchDecodeRow<256>(a, s, 1) : (D == 128 ? LaunchDecodeRow<128>(a, s, 1) : LaunchDecodeRow<64>(a, s, 1));
  } else if (G <= 8) e = LaunchDecode<8>(a, s);
  else if (G <= 16) e = LaunchDecode<16>(a, s);
  else if (G <= 32) e = LaunchDecode<32>(a, s);
  else if (G <= 64) e = LaunchDecode<64>(a, s);
  else return R4DXB_UNSUPPORTED;
  if (e) return e;
  return LaunchPdl(CombineKernel, dim3(G * ((D + 31) / 32), Hkv), dim3(kCombineThreads), 0, s, static_cast<const float*>(part_acc), static_cast<const float*>(part_ml),
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
  if (G <= 8 && g_decode_row && (D == 256 || D == 128 || D == 64)) {
    e = D == 256 ? LaunchDecodeRow<256>(a, s, B) : (D == 128 ? LaunchDecodeRow<128>(a, s, B) : LaunchDecodeRow<64>(a, s, B));
  } else if (G <= 8) e = LaunchDecode<8>(a, s, B);
  else if (G <= 16) e = LaunchDecode<16>(a, s, B);
  else if (G <= 32) e = LaunchDecode<32>(a, s, B);
  else e = LaunchDecode<64>(a, s, B);
  if (e) return e;
  CombineKernel<<<dim3(G * ((D + 31) / 32), Hkv, B), kCombineThreads, 0, s>>>(part_acc, part_ml, static_cast<const __nv_bfloat16*>(qg),
                                              static_cast<__nv_bfloat16*>(out), 1, Hq, Hkv, D, splits, gated, 1);
  return FinishLaunch();
}

}  // extern "C"
