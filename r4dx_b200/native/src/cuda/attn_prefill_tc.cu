// Causal GQA attention for a prefill chunk on the 5th-generation tensor cores: tcgen05.mma with the score
// tile S, the probability tile P and the output accumulator O all in tensor memory.
//
// One CTA = one query head x 128 consecutive query tokens.  It walks the visible keys in tiles of 64 tokens:
//     S = Q K^T   tcgen05.mma kind::f16, A = Q (shared memory, resident for the whole CTA), B = K tile; M 128, N 64,
//                 K = D in steps of 16; fp32 S in tensor memory (two buffers)
//     softmax     four warps, thread r owns query row r: tcgen05.ld S, running maximum in the log2 domain,
//                 P = 2^(S - m) rounded to fp16 and written back to tensor memory with tcgen05.st (thread = row =
//                 TMEM lane, so no shuffle and no shared memory is involved)
//     O += P V    tcgen05.mma with the A operand read from TENSOR MEMORY (the P tile) and B = V^T tile; M 128, N D,
//                 K = 64 tokens in steps of 16; fp32 O in tensor memory for the whole CTA
// The cache holds fp8 e4m3 rows in 16-token pages.  Twelve conversion warps (two groups, one per tile buffer, each
// loading a whole tile into registers before it waits for the tile's buffers) widen each K tile to fp16 in the
// canonical K-major 128-byte-swizzled layout, and write the V tile TRANSPOSED ([dimension][token]) so that V is a
// plain K-major B operand as well; Q is pre-multiplied by softmax scale x log2(e) x the K descale while it is
// converted, so scores need no further scaling.  The MMA issuer keeps one S tile ahead of the softmax
// (S_j+1 is issued before P_j V_j), conversion runs two tiles ahead.
//
// Rescaling of O when a row maximum grows is lazy: P is computed against the maximum in use, and only when some
// row's true maximum has moved more than 8 (a factor 256, harmless in fp16 / fp32) does the warp wait for the
// outstanding P V products, rescale its 32 rows of O in tensor memory and adopt the new maximum.
// Every wait is bounded; a wait that runs out sets the status word and the CTA unwinds (frees tensor memory).
//
// The reference's counterpart is a query-tiled WMMA kernel (reference:
// third_party/libr4d/r4d_attn_prefill_h256_gqa6.hip:112); nothing is shared with it.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace r4dxb {
namespace {

constexpr int kQRows = 128;
constexpr int kKvTile = 64;
constexpr int kPage = 16;
constexpr int kConvGroups = 2;            // conversion groups: group g owns the key tiles of buffer g (tiles g, g + 2, ...)
constexpr int kGroupWarps = 5;            // 4 + 1 + 10 = 15 warps: registers are granted per four warps, so 16 warps get 128 each
constexpr int kConvWarps = kConvGroups * kGroupWarps;
constexpr int kMmaWarp = 4;
constexpr int kThreads = (4 + 1 + kConvWarps) * 32;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kSCol = 256, kPCol = 384;          // S buffers: 256 + 64 b; P buffers: 384 + 32 b
constexpr float kRescaleStep = 8.f;

struct TcArgs {
  const __nv_bfloat16* q;      // [T, Hq, D] normed + roped
  const __nv_bfloat16* qg;     // [T, Hq, 2D] (gate in the upper half), may be null when !gated
  const uint8_t* cache;        // [page][Hkv][2][16][D] fp8
  const int* block_table;
  const float* k_descale;
  const float* v_descale;
  __nv_bfloat16* out;          // [T, Hq, D]
  int T, Hq, Hkv, pos0, gated, window;
  int* status;
};

struct Bars {
  uint64_t q_full, k_full[2], v_full[2], s_full[2], p_full[2], pv_done[2], o_final;
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ uint32_t Fp8x2Bits(uint32_t v16) {
  __half2_raw r = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(v16 & 0xFFFFu), __NV_E4M3);
  return *reinterpret_cast<uint32_t*>(&r);
}
// four e4m3 bytes of one word -> two half2 words (bytes 0-1, bytes 2-3), without shifts or masks
__device__ __forceinline__ void Fp8x4ToHalf(uint32_t w, uint32_t& lo, uint32_t& hi) {
  asm("{ .reg .b16 l, h; mov.b32 {l, h}, %2; cvt.rn.f16x2.e4m3x2 %0, l; cvt.rn.f16x2.e4m3x2 %1, h; }"
      : "=r"(lo), "=r"(hi) : "r"(w));
}
__device__ __forceinline__ float Exp2Approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// offset of 16-byte chunk c of row r inside a [rows][128 B] tile in the K-major 128-byte-swizzled UMMA layout
__device__ __forceinline__ int Sw128(int r, int c) { return (r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4); }

__device__ __forceinline__ void TmemStore32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

template <int D>
__global__ void __launch_bounds__(kThreads, 1) AttnPrefillTcKernel(TcArgs a) {
  constexpr int NS = D / 64;                          // 64-dimension slabs (one 128-byte swizzle row of fp16 each)
  constexpr int kQBytes = NS * kQRows * 128;
  constexpr int kKBytes = NS * kKvTile * 128;
  constexpr int kVBytes = D * 128;                    // V^T: one row per dimension, 64 tokens = 128 bytes
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  unsigned char* Qs = smem;
  unsigned char* Ks = Qs + kQBytes;                   // [2][kKBytes]
  unsigned char* Vs = Ks + 2 * kKBytes;               // [2][kVBytes]
  Bars* bar = reinterpret_cast<Bars*>(Vs + 2 * kVBytes);
  volatile int* abort_flag = &bar->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hq = blockIdx.y, hkv = hq / (a.Hq / a.Hkv);
  const int ntile_q = (a.T + kQRows - 1) / kQRows;
  const int qt = ntile_q - 1 - static_cast<int>(blockIdx.x);      // the tiles with the most keys start first
  const int q0 = qt * kQRows;
  const int rows = min(kQRows, a.T - q0);
  const int kv_limit = a.pos0 + a.T;                  // tokens present in the cache
  const int kv_end = a.pos0 + q0 + rows;              // first key position no row of this tile may see
  const int kv_first = a.window > 0 ? max(0, a.pos0 + q0 - a.window + 1) : 0;
  const int tile0 = kv_first / kKvTile;
  const int ntiles = (kv_end + kKvTile - 1) / kKvTile - tile0;

  if (threadIdx.x == 0) {
    ptx::MbarInit(&bar->q_full, kConvWarps);
    for (int b = 0; b < 2; ++b) {
      ptx::MbarInit(&bar->k_full[b], kGroupWarps);
      ptx::MbarInit(&bar->v_full[b], kGroupWarps);
      ptx::MbarInit(&bar->s_full[b], 1);
      ptx::MbarInit(&bar->p_full[b], 4);
      ptx::MbarInit(&bar->pv_done[b], 1);
    }
    ptx::MbarInit(&bar->o_final, 1);
    bar->abort_flag = 0;
    ptx::MbarFenceInit();
  }
  if (warp == kMmaWarp) {
    ptx::TmemAlloc(&bar->tmem_base, kTmemCols);
    ptx::TmemRelinquish();
  }
  ptx::TcFenceBefore();
  __syncthreads();
  ptx::TcFenceAfter();
  const uint32_t tbase = bar->tmem_base;

  if (warp > kMmaWarp) {
    // ---------------- conversion warps: Q once, then K and V^T of every key tile ----------------
    const int tid = threadIdx.x - (kMmaWarp + 1) * 32;          // 0 .. 383
    {
      const float scale = rsqrtf(static_cast<float>(D)) * 1.4426950408889634f * a.k_descale[hkv];
      for (int i = tid; i < kQRows * (D / 8); i += kConvWarps * 32) {   // all conversion warps share the Q tile
        const int r = i / (D / 8), ch = i % (D / 8);
        uint4 o = make_uint4(0u, 0u, 0u, 0u);
        if (r < rows) {
          const uint4 v = *reinterpret_cast<const uint4*>(a.q + (static_cast<size_t>(q0 + r) * a.Hq + hq) * D + ch * 8);
          const uint32_t w[4] = {v.x, v.y, v.z, v.w};
          uint32_t h[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const __half2 p = __floats2half2_rn(BfLo(w[j]) * scale, BfHi(w[j]) * scale);
            h[j] = *reinterpret_cast<const uint32_t*>(&p);
          }
          o = make_uint4(h[0], h[1], h[2], h[3]);
        }
        *reinterpret_cast<uint4*>(Qs + (ch >> 3) * (kQRows * 128) + Sw128(r, ch & 7)) = o;
      }
      ptx::FenceProxyAsyncShared();
      __syncwarp();
      if (lane == 0) ptx::MbarArrive(&bar->q_full);
    }
    // Key tiles: a group loads ALL raw fp8 bytes of its tile into registers first (page-table lookups and loads of
    // the whole tile in flight together), only then waits for the tile's shared-memory buffers, converts and stores.
    // Group g serves buffer g, i.e. every second tile: it then sees each completion of its buffers' barriers
    // exactly once and in order, which is what keeps a parity wait unambiguous (a group that ran two completions
    // ahead of a barrier would read an old phase as the one it is waiting for).
    const int grp = tid / (kGroupWarps * 32), gt = tid % (kGroupWarps * 32);
    constexpr int GT = kGroupWarps * 32;
    constexpr int KTOT = kKvTile * (D / 16), VTOT = 8 * (D / 4);
    constexpr int KI = (KTOT + GT - 1) / GT;          // 16-byte K items per thread and tile
    constexpr int VI = (VTOT + GT - 1) / GT;          // V items (8 tokens x 4 dimensions) per thread and tile
    // Item -> thread maps, fixed for the whole kernel (only the page of a token changes from tile to tile):
    //   K item i: token i / (D/16), 16-dimension chunk i % (D/16): consecutive lanes read consecutive 16 bytes of a row.
    //   V item i: token group tg = i % 8 (fastest), dimension quad dq = i / 8: the eight lanes of one quad write one
    //             whole 128-byte row of the transposed tile (no bank conflict); their loads are 16-byte segments.
    int k_src[KI], k_dst[KI], v_src[VI], v_dst[VI];
#pragma unroll
    for (int n = 0; n < KI; ++n) {
      const int i = gt + n * GT;
      const int tok = i / (D / 16), ch = i % (D / 16);
      k_src[n] = i < KTOT ? (tok << 16) | ((tok & 15) * D + ch * 16) : -1;          // token in the high half, byte offset inside the page low
      k_dst[n] = (ch >> 2) * (kKvTile * 128) + Sw128(tok, (ch & 3) * 2);              // the second chunk sits at dst ^ 16
    }
#pragma unroll
    for (int n = 0; n < VI; ++n) {
      const int i = gt + n * GT;
      const int tg = i % 8, dq = i / 8;
      v_src[n] = i < VTOT ? ((tg * 8) << 16) | (((tg * 8) & 15) * D + dq * 4) : -1;
      v_dst[n] = (dq * 4) | (tg << 16);
    }
    const size_t page_bytes = static_cast<size_t>(a.Hkv) * 2 * kPage * D;
    const uint8_t* cache_k = a.cache + static_cast<size_t>(hkv) * 2 * kPage * D;
    const uint8_t* cache_v = cache_k + kPage * D;
    bool ok = true;
    for (int j = grp; j < ntiles; j += kConvGroups) {
      const int b = j & 1;
      const int kv0 = (tile0 + j) * kKvTile;
      const uint32_t prev = static_cast<uint32_t>((j - 2) >> 1) & 1u;      // parity of the buffer's previous use
      const bool whole = kv0 + kKvTile <= kv_limit;                         // every token of the tile is in the cache
      uint4 kraw[KI];
      uint32_t vraw[VI][8];
#pragma unroll
      for (int n = 0; n < KI; ++n) {
        kraw[n] = make_uint4(0u, 0u, 0u, 0u);
        const int kp = kv0 + (k_src[n] >> 16);
        if (k_src[n] >= 0 && (whole || kp < kv_limit)) {
          const int page = a.block_table[kp >> 4];
          kraw[n] = __ldg(reinterpret_cast<const uint4*>(cache_k + page * page_bytes + (k_src[n] & 0xFFFF)));
        }
      }
#pragma unroll
      for (int n = 0; n < VI; ++n) {
        const int kp = kv0 + (v_src[n] >> 16);
#pragma unroll
        for (int tt = 0; tt < 8; ++tt) vraw[n][tt] = 0u;
        if (v_src[n] >= 0 && (whole || kp < kv_limit)) {
          const int page = a.block_table[kp >> 4];
          const uint8_t* vrow = cache_v + page * page_bytes + (v_src[n] & 0xFFFF);
          if (whole) {
#pragma unroll
            for (int tt = 0; tt < 8; ++tt) vraw[n][tt] = __ldg(reinterpret_cast<const uint32_t*>(vrow + tt * D));
          } else {
#pragma unroll
            for (int tt = 0; tt < 8; ++tt)
              if (kp + tt < kv_limit) vraw[n][tt] = __ldg(reinterpret_cast<const uint32_t*>(vrow + tt * D));
          }
        }
      }
      // ---- K tile: [64 tokens][D] fp8 -> fp16, K-major ----
      if (j >= 2 && ok) ok = ptx::WarpMbarWait(&bar->s_full[b], prev, abort_flag, 11);     // S_(j-2) has consumed the buffer
      if (ok) {
        unsigned char* kt = Ks + b * kKBytes;
#pragma unroll
        for (int n = 0; n < KI; ++n) {
          if (k_src[n] < 0) continue;
          uint4 lo, hi;
          Fp8x4ToHalf(kraw[n].x, lo.x, lo.y);
          Fp8x4ToHalf(kraw[n].y, lo.z, lo.w);
          Fp8x4ToHalf(kraw[n].z, hi.x, hi.y);
          Fp8x4ToHalf(kraw[n].w, hi.z, hi.w);
          *reinterpret_cast<uint4*>(kt + k_dst[n]) = lo;
          *reinterpret_cast<uint4*>(kt + (k_dst[n] ^ 16)) = hi;
        }
      }
      ptx::FenceProxyAsyncShared();
      __syncwarp();
      if (lane == 0) ptx::MbarArrive(&bar->k_full[b]);
      // ---- V tile, transposed: [D dimensions][64 tokens] fp16, K-major in the token index ----
      if (j >= 2 && ok) ok = ptx::WarpMbarWait(&bar->pv_done[b], prev, abort_flag, 12);    // P_(j-2) V_(j-2) has consumed it
      if (ok) {
        unsigned char* vt = Vs + b * kVBytes;
#pragma unroll
        for (int n = 0; n < VI; ++n) {
          if (v_src[n] < 0) continue;
          const int d0 = v_dst[n] & 0xFFFF, tg = v_dst[n] >> 16;
#pragma unroll
          for (int dd = 0; dd < 4; ++dd) {
            const uint32_t sel = static_cast<uint32_t>(dd) | (static_cast<uint32_t>(4 + dd) << 4);   // byte dd of both words
            const uint4 o = make_uint4(Fp8x2Bits(__byte_perm(vraw[n][0], vraw[n][1], sel)), Fp8x2Bits(__byte_perm(vraw[n][2], vraw[n][3], sel)),
                                       Fp8x2Bits(__byte_perm(vraw[n][4], vraw[n][5], sel)), Fp8x2Bits(__byte_perm(vraw[n][6], vraw[n][7], sel)));
            *reinterpret_cast<uint4*>(vt + Sw128(d0 + dd, tg)) = o;
          }
        }
      }
      ptx::FenceProxyAsyncShared();
      __syncwarp();
      if (lane == 0) ptx::MbarArrive(&bar->v_full[b]);
    }
  } else if (warp == kMmaWarp) {
    // ---------------- MMA issuer (one thread) ----------------
    if (lane == 0) {
      constexpr uint32_t idesc_s = ptx::UmmaInstrDescF16(128, kKvTile, false);
      constexpr uint32_t idesc_o = ptx::UmmaInstrDescF16(128, D, false);
      const uint32_t q_addr = ptx::SmemAddr(Qs);
      bool ok = ptx::MbarWait(&bar->q_full, 0, abort_flag, 1);
      auto issue_pv = [&](int j) {
        const int b = j & 1;
        const uint32_t ph = static_cast<uint32_t>(j >> 1) & 1u;
        ok = ok && ptx::MbarWait(&bar->p_full[b], ph, abort_flag, 3) && ptx::MbarWait(&bar->v_full[b], ph, abort_flag, 4);
        if (!ok) return;
        ptx::TcFenceAfter();
        const uint32_t v_addr = ptx::SmemAddr(Vs + b * kVBytes);
#pragma unroll
        for (int k = 0; k < kKvTile / 16; ++k)
          ptx::UmmaF16FromTmem(tbase, tbase + kPCol + b * 32 + k * 8, ptx::UmmaDescSw128(v_addr + k * 32), idesc_o,
                               (j > 0 || k > 0) ? 1u : 0u);
        ptx::UmmaCommit(&bar->pv_done[b]);
      };
      for (int j = 0; j < ntiles && ok; ++j) {
        const int b = j & 1;
        const uint32_t ph = static_cast<uint32_t>(j >> 1) & 1u;
        ok = ptx::MbarWait(&bar->k_full[b], ph, abort_flag, 2);
        // the softmax of tile j-2 has read S buffer b (it arrives on p_full after it)
        if (ok && j >= 2) ok = ptx::MbarWait(&bar->p_full[b], static_cast<uint32_t>((j - 2) >> 1) & 1u, abort_flag, 5);
        if (!ok) break;
        ptx::TcFenceAfter();
        const uint32_t k_addr = ptx::SmemAddr(Ks + b * kKBytes);
#pragma unroll
        for (int s = 0; s < NS; ++s)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            ptx::UmmaF16(tbase + kSCol + b * 64, ptx::UmmaDescSw128(q_addr + s * (kQRows * 128) + k * 32),
                         ptx::UmmaDescSw128(k_addr + s * (kKvTile * 128) + k * 32), idesc_s, (s > 0 || k > 0) ? 1u : 0u);
        ptx::UmmaCommit(&bar->s_full[b]);
        if (j >= 1) issue_pv(j - 1);
      }
      if (ok && ntiles > 0) issue_pv(ntiles - 1);
      if (ok) ptx::UmmaCommit(&bar->o_final);
    }
    __syncwarp();
  } else {
    // ---------------- softmax warps: thread = query row = TMEM lane ----------------
    const int r = warp * 32 + lane;
    const int qp = a.pos0 + q0 + r;                               // position of this row's query
    const uint32_t t_lane = tbase + (static_cast<uint32_t>(warp * 32) << 16);
    float m_used = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < ntiles; ++j) {
      const int b = j & 1;
      const uint32_t ph = static_cast<uint32_t>(j >> 1) & 1u;
      if (ok) ok = ptx::WarpMbarWait(&bar->s_full[b], ph, abort_flag, 6);
      if (!ok) continue;
      ptx::TcFenceAfter();
      uint32_t s0[32], s1[32];
      ptx::TmemLoad32x32(t_lane + kSCol + b * 64, s0);
      ptx::TmemLoad32x32(t_lane + kSCol + b * 64 + 32, s1);
      ptx::TmemLoadWait();
      const int kv0 = (tile0 + j) * kKvTile;
      // tiles that reach past the row's own position (or start before its window) need the mask
      const bool need_mask = (kv0 + kKvTile - 1 > a.pos0 + q0) || (a.window > 0 && kv0 < a.pos0 + q0 + kQRows - a.window);
      float mx = -INFINITY;
      if (need_mask) {
        const int lo = a.window > 0 ? qp - a.window : -1;         // visible: lo < kp <= qp
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const int k0 = kv0 + c, k1 = kv0 + 32 + c;
          if (!(k0 <= qp && k0 > lo)) s0[c] = 0xff800000u;        // -inf
          if (!(k1 <= qp && k1 > lo)) s1[c] = 0xff800000u;
        }
      }
#pragma unroll
      for (int c = 0; c < 32; ++c) mx = fmaxf(mx, fmaxf(__uint_as_float(s0[c]), __uint_as_float(s1[c])));
      // lazy rescale: adopt a new maximum only when some row of the warp has drifted by more than the step
      const bool drift = mx > m_used + kRescaleStep;
      if (__any_sync(0xffffffffu, drift)) {
        const float m_new = fmaxf(m_used, mx);
        if (j > 0) {
          // every P V issued so far must have landed before O is touched (products complete in order)
          ok = ptx::WarpMbarWait(&bar->pv_done[(j - 1) & 1], static_cast<uint32_t>((j - 1) >> 1) & 1u, abort_flag, 7);
          if (ok) {
            ptx::TcFenceAfter();
            const float f = (m_used == -INFINITY) ? 0.f : exp2f(m_used - m_new);
            l_run *= f;
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 32) {
              uint32_t o[32];
              ptx::TmemLoad32x32(t_lane + c0, o);
              ptx::TmemLoadWait();
#pragma unroll
              for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * f);
              TmemStore32x32(t_lane + c0, o);
            }
            ptx::TmemStoreWait();
          }
        }
        m_used = m_new;
      }
      if (!ok) continue;
      // P = 2^(S - m), fp16 pairs (k, k+1) per column
      uint32_t p[32];
      float sum = 0.f;
      const float mref = (m_used == -INFINITY) ? 0.f : m_used;
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const float e0 = Exp2Approx(__uint_as_float(s0[2 * c]) - mref), e1 = Exp2Approx(__uint_as_float(s0[2 * c + 1]) - mref);
        sum += e0 + e1;
        const __half2 h = __floats2half2_rn(e0, e1);
        p[c] = *reinterpret_cast<const uint32_t*>(&h);
      }
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const float e0 = Exp2Approx(__uint_as_float(s1[2 * c]) - mref), e1 = Exp2Approx(__uint_as_float(s1[2 * c + 1]) - mref);
        sum += e0 + e1;
        const __half2 h = __floats2half2_rn(e0, e1);
        p[16 + c] = *reinterpret_cast<const uint32_t*>(&h);
      }
      l_run += sum;
      // P buffer b was read by P_(j-2) V_(j-2)
      if (j >= 2) ok = ptx::WarpMbarWait(&bar->pv_done[b], static_cast<uint32_t>((j - 2) >> 1) & 1u, abort_flag, 8);
      if (!ok) continue;
      ptx::TcFenceAfter();
      TmemStore32x32(t_lane + kPCol + b * 32, p);
      ptx::TmemStoreWait();
      ptx::TcFenceBefore();
      __syncwarp();
      if (lane == 0) ptx::MbarArrive(&bar->p_full[b]);
    }
    // ---------------- epilogue: O / l, output gate, bf16 rows ----------------
    if (ok && ntiles > 0) ok = ptx::WarpMbarWait(&bar->o_final, 0, abort_flag, 9);
    if (ok) {
      ptx::TcFenceAfter();
      const float inv = (l_run > 0.f ? 1.f / l_run : 0.f) * a.v_descale[hkv];
      const bool live = r < rows && ntiles > 0;
      const size_t t = static_cast<size_t>(q0 + r);
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t o[32];
        ptx::TmemLoad32x32(t_lane + c0, o);
        ptx::TmemLoadWait();
        if (live) {
          uint32_t packed[16];
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            float x0 = __uint_as_float(o[2 * c]) * inv, x1 = __uint_as_float(o[2 * c + 1]) * inv;
            if (a.gated) {
              const uint32_t gv = *reinterpret_cast<const uint32_t*>(a.qg + (t * a.Hq + hq) * 2 * D + D + c0 + 2 * c);
              x0 *= Sigmoid(BfLo(gv));
              x1 *= Sigmoid(BfHi(gv));
            }
            packed[c] = PackBf16(x0, x1);
          }
          uint4* dst = reinterpret_cast<uint4*>(a.out + (t * a.Hq + hq) * D + c0);
#pragma unroll
          for (int v = 0; v < 4; ++v) dst[v] = make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
        }
      }
    }
  }

  // ---------------- teardown ----------------
  ptx::TcFenceBefore();
  __syncthreads();
  if (*abort_flag != 0) {
    if (threadIdx.x == 0 && a.status != nullptr) atomicCAS(a.status, 0, 600 + *abort_flag);
  }
  if (warp == kMmaWarp) {
    ptx::TcFenceAfter();
    ptx::TmemDealloc(tbase, kTmemCols);
  }
}

template <int D>
int LaunchTc(const TcArgs& a, cudaStream_t s) {
  constexpr int NS = D / 64;
  const size_t smem = static_cast<size_t>(NS) * kQRows * 128 + 2 * NS * kKvTile * 128 + 2 * D * 128 + sizeof(Bars) + 1024;
  auto kern = AttnPrefillTcKernel<D>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return static_cast<int>(e);
  dim3 grid((a.T + kQRows - 1) / kQRows, a.Hq);
  kern<<<grid, kThreads, smem, s>>>(a);
  return FinishLaunch();
}

}  // namespace
}  // namespace r4dxb

using namespace r4dxb;

/* Same contract as r4dxb_attn_prefill (flags bit 0: sigmoid output gate, bits 1..: sliding-window length), for head
   dimensions 128 and 256.  status: device word that receives 600 + role code if a bounded wait ran out. */
extern "C" int r4dxb_attn_prefill_tc(const void* q, const void* qg, const void* cache, const int* block_table,
                                     const float* k_descale, const float* v_descale, void* out, int T, int Hq, int Hkv, int D,
                                     int pos0, int flags, int* status, void* stream) {
  if (T < 1 || Hq % Hkv || (D != 256 && D != 128)) return R4DXB_BAD_ARG;
  TcArgs a;
  a.q = static_cast<const __nv_bfloat16*>(q);
  a.qg = static_cast<const __nv_bfloat16*>(qg);
  a.cache = static_cast<const uint8_t*>(cache);
  a.block_table = block_table;
  a.k_descale = k_descale;
  a.v_descale = v_descale;
  a.out = static_cast<__nv_bfloat16*>(out);
  a.T = T; a.Hq = Hq; a.Hkv = Hkv; a.pos0 = pos0; a.gated = flags & 1; a.window = flags >> 1;
  a.status = status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return D == 256 ? LaunchTc<256>(a, s) : LaunchTc<128>(a, s);
}
