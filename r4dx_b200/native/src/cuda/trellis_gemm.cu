// Trellis-decode GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), for T >= 16 rows.
//
//   Y[t, n] = bf16( svh[n] * H128( sum_k Q[n, k] * Xh[t, k] )[n] (+ residual[t, n]) )
//
// "Swap-AB": the decoded weight block is the UMMA A operand (M = 128 weight rows = the span of one
// output Hadamard), the activations are the B operand (N = TN tokens), so the fp32 accumulator
// sits in TMEM as [lane = weight row][column = token].  Weights are decoded exactly once per CTA
// and reused by all TN tokens of the tile.
//
// Warp roles (DW + 2 warps, DW = 4, 8 or 16 decode warps):
//   warps 0..DW-1  decode: packed words (shared memory) -> fp16 codes -> A tile in the canonical
//              K-major 128-byte-swizzled UMMA layout; later the epilogue (TMEM -> registers ->
//              shared transpose -> FWHT128 over the weight rows -> svh, residual -> bf16 rows).
//              The decode chain (shift, multiply, byte-sum) is dependent integer work at ~0.3 IPC
//              per warp, so several warps per scheduler are what keeps the tensor pipe fed.
//   warp DW    producer: TMA tile of Xh [TN x 64] (128B swizzle) + bulk copy of the slab's words
//   warp DW+1  MMA issuer: one elected thread issues 4 x tcgen05.mma (K = 16) per 64-wide K slab
//              and commits to the stage's "empty" barrier; it also owns the TMEM allocation.
// A dense mode (KB == 0) takes A from a plain fp16 [N, K] matrix instead of decoding: that is the
// bf16/fp16-layout linear and the bisecting aid for the tensor-core plumbing.
//
// The reference engine's counterparts are WMMA kernels whose decoded fragments are shared through
// LDS (reference: third_party/libr4d/r4d_gemm_trellis_nt_m256.hip:1-60); nothing is shared with them.
#include <cuda_fp8.h>

#include "sm100_ptx.cuh"
#include "trellis_decode.cuh"

namespace r4dxb {
namespace {

constexpr int kSlabK = 64;                 // K per pipeline stage = one 128-byte swizzle row of fp16
constexpr int kATileBytes = 128 * kSlabK * 2;   // 16 KiB

// Three rings, sized independently so that cheap data is prefetched deep and the big tile is not:
//   words (<= 5 KiB per slab, WST deep)  producer W -> decode warps
//   A     (16 KiB per slab, AST deep)    decode warps -> MMA
//   X     (TN x 128 B per slab, XST deep) producer X -> MMA
template <int KB, int TN, int F8 = 0>
struct GemmSmem {
  // a slab is one 128-byte swizzle row of K per operand row: 64 fp16 values (4 k-tiles of 16) or 128 e4m3 values (8 k-tiles)
  static constexpr int kKTiles = F8 ? 8 : 4;
  static constexpr int kWordsBytes = (KB == 0) ? 0 : kKTiles * 8 * 8 * KB * 4;   // k-tiles x 8 n-tiles x 8KB words
  static constexpr int kWordsSlot = ((kWordsBytes + 1023) / 1024) * 1024;
  static constexpr int kXTileBytes = TN * kSlabK * 2;
  static constexpr int WST = F8 ? 4 : 6;      // (8-bit slabs carry twice the words: four of them are as much K in flight as six 16-bit ones)
  static constexpr int AST = KB == 0 ? 4 : 3;
  static constexpr int XST = TN >= 512 ? 2 : (TN >= 256 ? 3 : 4);
  static constexpr int kABytes = AST * kATileBytes;
  static constexpr int kXBytes = XST * kXTileBytes;
  static constexpr int kEpiStride = 132;                                     // floats per staged token row
  static constexpr int kEpiBytes = 32 * kEpiStride * 4;                      // per group of four epilogue warps
  // the epilogue staging reuses the (by then drained) rings: it must hold one buffer per warp group
  static constexpr int kRingsRaw = kABytes + kXBytes + WST * kWordsSlot;
  static constexpr int kRing = kRingsRaw > 4 * kEpiBytes ? kRingsRaw : 4 * kEpiBytes;
  static constexpr int kBars = 2 * WST + 2 * AST + 2 * XST + 1;
  static constexpr int kTotal = kRing + 1024 /*alignment slack*/ + 512 /*barriers*/;
};

// Reduce-scatter epilogue (tensor-parallel prefill): instead of its own output tensor, the row-parallel product
// stores every partial row into the receive buffer of the rank that owns the row (rows are dealt out in
// contiguous blocks of rows_per_rank), over NVLink peer mappings, tile by tile as the epilogue produces them;
// one system-scope counter per owner collects the arrivals of every CTA on every rank.
struct RsArgs {
  __nv_bfloat16* recv[8];      // peer-mapped receive buffers, indexed by owner rank: [world(src)][rows_per_rank][N]
  unsigned* cnt[8];            // peer-mapped arrival counters, indexed by owner rank
  int world, rank, rows_per_rank;
};

// Plain linear modes of the same kernel (MODE 1: dense 16-bit A matrix, MODE 2: w4a16 group-quantised A): y = x W^T
// (+ bias) (+ residual) with no Hadamard epilogue; activations and a dense A may be bf16 instead of fp16, the result
// may be written as fp32 (vocabulary logits).  These are the tensor-core paths of the heads and of the dense towers for
// more than 8 rows (reference: third_party/libr4d/r4d_gemm_w4a16_nt_m64.hip:173 is the WMMA counterpart for w4a16).
__device__ __forceinline__ float GeluTanh(float v) {
  return 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
}
__device__ __forceinline__ float GeluErf(float v) { return 0.5f * v * (1.0f + erff(v * 0.7071067811865476f)); }

struct PlainArgs {
  const uint32_t* wsz;         // MODE 2: [N][K / group] (fp16 scale | fp16 -(1024 + zero) << 16)
  const __nv_bfloat16* bias;   // [N] or null
  int group;                   // MODE 2: quantisation group (32, 64 or 128)
  int bf16;                    // the 16-bit operands are bf16 (MODE 1 only)
  int out_f32;                 // y is fp32 [T, N] instead of bf16
  int act;                     // after the bias: 0 none, 1 tanh-GELU, 2 erf-GELU
  // MODE 3, grouped experts: the rows of xh are the (row, expert) pairs sorted by expert; a token tile is one expert's
  // next TN rows.  offsets [E + 1] and perm [pairs] come from the routing plan, tiles/ntiles from MoeTilesKernel.
  const int* g_offsets;
  const int* g_perm;           // sorted position -> pair id = output row
  const int* g_tiles;          // [2 * max_tiles]: (local expert, first sorted row)
  const int* g_ntiles;
  long long g_words;           // packed words per expert
  int g_max_tiles;             // grid height: an upper bound on the tile count
  // MODE 4, 8-bit operands: the decode warps emit e4m3 code values, the activations are e4m3 rows with one fp32 scale per
  // row (xh = scale * e4m3); K per slab is 128 and the products run at the 8-bit rate with half the activation bytes
  const float* x_scale;        // [T]
};

template <int KB, int TN, int DW, int MODE = 0>
__global__ void __launch_bounds__((DW + 3) * 32, 1)
TrellisGemmKernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_a,
                  const void* __restrict__ wsrc,
                  const __half* __restrict__ svh, __nv_bfloat16* __restrict__ y,
                  const __nv_bfloat16* __restrict__ residual, int T, int N, int K, int* __restrict__ status, RsArgs rs,
                  PlainArgs pl) {
  using S = GemmSmem<KB, TN, MODE == 4>;
  constexpr int kSlabElems = MODE == 4 ? 2 * kSlabK : kSlabK;      // K values per slab (one 128-byte row per operand row)
  constexpr int kKTiles = S::kKTiles;
  constexpr int WST = S::WST, AST = S::AST, XST = S::XST;
  extern __shared__ unsigned char smem_dyn[];
  // 1024-byte alignment: required by the swizzled UMMA / TMA tiles
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  unsigned char* a_ring = smem;
  unsigned char* x_ring = smem + S::kABytes;
  unsigned char* w_ring = smem + S::kABytes + S::kXBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::kRing);
  uint64_t* wfull = bars;                   // [WST] producer W -> decode
  uint64_t* wempty = wfull + WST;           // [WST] decode -> producer W
  uint64_t* afull = wempty + WST;           // [AST] decode -> MMA
  uint64_t* aempty = afull + AST;           // [AST] MMA -> decode
  uint64_t* xfull = aempty + AST;           // [XST] producer X -> MMA
  uint64_t* xempty = xfull + XST;           // [XST] MMA -> producer X
  uint64_t* accum = xempty + XST;           // [1]   MMA -> epilogue
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nb = blockIdx.x;                 // 128-row weight block
  int t0 = blockIdx.y * TN;                  // first token of the tile
  int t_end = T;                             // rows at and past t_end are not stored
  if constexpr (MODE == 3) {
    if (static_cast<int>(blockIdx.y) >= __ldg(pl.g_ntiles)) return;       // the whole CTA, before any barrier exists
    const int e = __ldg(pl.g_tiles + 2 * blockIdx.y);
    t0 = __ldg(pl.g_tiles + 2 * blockIdx.y + 1);
    t_end = __ldg(pl.g_offsets + e + 1);
    wsrc = static_cast<const uint32_t*>(wsrc) + static_cast<long long>(e) * pl.g_words;
    svh += static_cast<size_t>(e) * N;
  }
  const int slabs = (K + kSlabElems - 1) / kSlabElems;   // a ragged last slab only in the dense plain mode (TMA zero-fills X)
  constexpr uint32_t kTmemCols = TN < 32 ? 32 : TN;
  constexpr int kHalves = TN > 256 ? TN / 256 : 1;     // one MMA covers at most 256 token columns
  constexpr int kMmaN = TN > 256 ? 256 : TN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < WST; ++s) {
      ptx::MbarInit(&wfull[s], 1);
      ptx::MbarInit(&wempty[s], DW);
    }
    for (int s = 0; s < AST; ++s) {
      ptx::MbarInit(&afull[s], MODE == 1 ? 1 : DW);
      ptx::MbarInit(&aempty[s], 1);
    }
    for (int s = 0; s < XST; ++s) {
      ptx::MbarInit(&xfull[s], 1);
      ptx::MbarInit(&xempty[s], 1);
    }
    ptx::MbarInit(accum, 1);
    *abort_flag = 0;
    ptx::MbarFenceInit();
  }
  if (warp == DW + 1) {
    ptx::TmemAlloc(tmem_slot, kTmemCols);
    ptx::TmemRelinquish();
  }
  if (warp == DW && lane == 0) ptx::PrefetchTensorMap(&tmap_x);
  ptx::TcFenceBefore();
  __syncthreads();
  ptx::TcFenceAfter();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == DW) {
    // ---------------- producer X: TMA tiles of the transformed activations ----------------
    if (lane == 0) {
      for (int it = 0; it < slabs; ++it) {
        const int s = it % XST, round = it / XST;
        if (!ptx::MbarWait(&xempty[s], (round & 1) ^ 1, abort_flag, 1)) break;
        ptx::MbarArriveExpectTx(&xfull[s], S::kXTileBytes);
#pragma unroll
        for (int h = 0; h < kHalves; ++h)
          ptx::TmaLoad2D(x_ring + s * S::kXTileBytes + h * (kMmaN * kSlabK * 2), &tmap_x, &xfull[s], it * kSlabElems, t0 + h * kMmaN);
      }
    }
  } else if (warp == DW + 2) {
    // ---------------- producer W: packed words, prefetched WST slabs deep ----------------
    if (MODE == 1 && lane == 0) {
      // dense plain mode: the weight tile comes by TMA as well (rows and columns past the matrix read as zero)
      ptx::PrefetchTensorMap(&tmap_a);
      for (int it = 0; it < slabs; ++it) {
        const int s = it % AST, round = it / AST;
        if (!ptx::MbarWait(&aempty[s], (round & 1) ^ 1, abort_flag, 5)) break;
        ptx::MbarArriveExpectTx(&afull[s], kATileBytes);
        ptx::TmaLoad2D(a_ring + s * kATileBytes, &tmap_a, &afull[s], it * kSlabK, nb * 128);
      }
    }
    if (KB != 0 && lane == 0) {
      const size_t slab_words = kKTiles * 8 * 8 * (KB == 0 ? 1 : KB);
      const uint32_t* wbase = static_cast<const uint32_t*>(wsrc) + static_cast<size_t>(nb) * (K / 16) * 8 * 8 * (KB == 0 ? 1 : KB);
      for (int it = 0; it < slabs; ++it) {
        const int s = it % WST, round = it / WST;
        if (!ptx::MbarWait(&wempty[s], (round & 1) ^ 1, abort_flag, 7)) break;
        ptx::MbarArriveExpectTx(&wfull[s], S::kWordsBytes);
        ptx::BulkLoad(w_ring + s * S::kWordsSlot, wbase + static_cast<size_t>(it) * slab_words, S::kWordsBytes, &wfull[s]);
      }
    }
  } else if (warp == DW + 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc = MODE == 4 ? ptx::UmmaInstrDescE4m3(128, kMmaN) : ptx::UmmaInstrDescF16(128, kMmaN, MODE == 1 && pl.bf16 != 0);
      bool ok = true;
      for (int it = 0; it < slabs && ok; ++it) {
        const int sa = it % AST, ra = it / AST, sx = it % XST, rx = it / XST;
        ok = ptx::MbarWait(&xfull[sx], rx & 1, abort_flag, 2) && ptx::MbarWait(&afull[sa], ra & 1, abort_flag, 3);
        if (!ok) break;
        ptx::TcFenceAfter();
        const uint32_t a_addr = ptx::SmemAddr(a_ring + sa * kATileBytes), b_addr = ptx::SmemAddr(x_ring + sx * S::kXTileBytes);
#pragma unroll
        for (int h = 0; h < kHalves; ++h) {
#pragma unroll
          for (int k = 0; k < kSlabK / 16; ++k) {
            const uint64_t da = ptx::UmmaDescSw128(a_addr + k * 32);
            const uint64_t db = ptx::UmmaDescSw128(b_addr + h * (kMmaN * kSlabK * 2) + k * 32);
            if constexpr (MODE == 4) ptx::UmmaF8(tmem_base + h * kMmaN, da, db, idesc, (it > 0 || k > 0) ? 1u : 0u);
            else ptx::UmmaF16(tmem_base + h * kMmaN, da, db, idesc, (it > 0 || k > 0) ? 1u : 0u);
          }
        }
        ptx::UmmaCommit(&aempty[sa]);         // frees the A tile and the X tile once these MMAs have read them
        ptx::UmmaCommit(&xempty[sx]);
      }
      if (ok) ptx::UmmaCommit(accum);         // accumulator complete
    }
  } else {
    // ---------------- decode warps ----------------
    // a slab is 32 tiles (8 n-tiles x 4 k-tiles); warp w takes tiles w, w + DW, ...
    // lane slot: row (lane % 16) of the 16-row n-tile, K half (lane / 16) -> conflict-free 16-byte stores
    const int row_in_tile = lane & 15, khalf = lane >> 4;
    TrellisLane<(KB == 0 ? 4 : KB)> tl;
    tl.Init(2 * row_in_tile + khalf);
    bool ok = true;
    for (int it = 0; MODE != 1 && it < slabs && ok; ++it) {
      const int sa = it % AST, ra = it / AST, sw = it % WST, rw = it / WST;
      if (KB != 0) ok = ptx::MbarWait(&wfull[sw], rw & 1, abort_flag, 4);
      ok = ok && ptx::MbarWait(&aempty[sa], (ra & 1) ^ 1, abort_flag, 5);
      if (!ok) break;
      unsigned char* at = a_ring + sa * kATileBytes;
      if constexpr (MODE == 5) {
        // w8a16: a lane widens 32 consecutive k of one row (32 offset-binary bytes): a byte b becomes the fp16 1024 + b by
        // pairing it with 0x64; subtracting 1152 gives b - 128 exactly, the group scale is the only rounding
        for (int idx = warp; idx < 8; idx += DW) {
          const int r = idx * 16 + (lane >> 1), half = lane & 1;
          const size_t n = static_cast<size_t>(nb) * 128 + r;
          const int kbase = it * kSlabK + half * 32;
          const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(wsrc) + n * K + kbase);
          const uint4 q0 = __ldg(src), q1 = __ldg(src + 1);
          const __half sc = __ldg(reinterpret_cast<const __half*>(pl.wsz) + n * (K / pl.group) + kbase / pl.group);
          const __half2 sc2 = __half2half2(sc), off2 = __half2half2(__float2half(1152.0f));      // 1024 + 128
          const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t hb[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t w32 = qw[2 * c + (i >> 1)];
              const uint32_t b = __byte_perm(w32, 0x00000064u, (i & 1) ? 0x4342 : 0x4140);      // (1024 + b_lo, 1024 + b_hi)
              const __half2 v = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&b), off2), sc2);   // (b - 128) exactly, one rounding
              hb[i] = *reinterpret_cast<const uint32_t*>(&v);
            }
            const int chunk = half * 4 + c;
            *reinterpret_cast<uint4*>(at + (r >> 3) * 1024 + (r & 7) * 128 + ((chunk ^ (r & 7)) << 4)) = make_uint4(hb[0], hb[1], hb[2], hb[3]);
          }
        }
      } else if constexpr (MODE == 2) {
        // w4a16: a lane widens 32 consecutive k of one row (16 bytes of nibbles): nibble -> fp16 1024 + n by or-ing
        // 0x6400, the stored -(1024 + zero) makes n - zero exact, one fp16 multiply by the group scale
        for (int idx = warp; idx < 8; idx += DW) {
          const int r = idx * 16 + (lane >> 1), half = lane & 1;
          const size_t n = static_cast<size_t>(nb) * 128 + r;
          const int kbase = it * kSlabK + half * 32;
          const uint4 q = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint32_t*>(wsrc) + n * (K / 8) + kbase / 8));
          const uint32_t sz = __ldg(pl.wsz + n * (K / pl.group) + kbase / pl.group);
          const uint32_t scb = (sz & 0xFFFFu) | (sz << 16), nzb = (sz >> 16) | (sz & 0xFFFF0000u);
          const __half2 sc2 = *reinterpret_cast<const __half2*>(&scb), nz2 = *reinterpret_cast<const __half2*>(&nzb);
          const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
          for (int wi = 0; wi < 4; ++wi) {
            uint32_t hb[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t b = ((qw[wi] >> (4 * i)) & 0x000F000Fu) | 0x64006400u;       // (k + i, k + i + 4)
              const __half2 v = __hmul2(__hadd2(*reinterpret_cast<const __half2*>(&b), nz2), sc2);
              hb[i] = *reinterpret_cast<const uint32_t*>(&v);
            }
            uint4 packed;
            packed.x = __byte_perm(hb[0], hb[1], 0x5410); packed.y = __byte_perm(hb[2], hb[3], 0x5410);
            packed.z = __byte_perm(hb[0], hb[1], 0x7632); packed.w = __byte_perm(hb[2], hb[3], 0x7632);
            const int chunk = half * 4 + wi;
            *reinterpret_cast<uint4*>(at + (r >> 3) * 1024 + (r & 7) * 128 + ((chunk ^ (r & 7)) << 4)) = packed;
          }
        }
      } else if constexpr (MODE == 4) {
        // 8-bit operands: a slab is 8 k-tiles; a lane's 8 code values become 8 e4m3 bytes, the two K halves of a row share
        // one 16-byte swizzle chunk (chunk index = k-tile)
#pragma unroll 4
        for (int idx = warp; idx < 64; idx += DW) {
          const int j = idx & 7, kt = idx >> 3;
          const int r = j * 16 + row_in_tile;
          constexpr int NW = 8 * (KB == 0 ? 4 : KB);
          const uint32_t* tw = reinterpret_cast<const uint32_t*>(w_ring + sw * S::kWordsSlot) + (kt * 8 + j) * NW;
          uint32_t hi, lo;
          tl.Window(tw[tl.i0], tw[tl.i1], (KB == 4) ? 0u : tw[tl.i2], hi, lo);
          __half2 w[4];
          TrellisDecode8<(KB == 0 ? 4 : KB)>(hi, lo, w);
          uint2 packed;
          packed.x = static_cast<uint32_t>(__nv_cvt_halfraw2_to_fp8x2(*reinterpret_cast<__half2_raw*>(&w[0]), __NV_SATFINITE, __NV_E4M3)) |
                     (static_cast<uint32_t>(__nv_cvt_halfraw2_to_fp8x2(*reinterpret_cast<__half2_raw*>(&w[1]), __NV_SATFINITE, __NV_E4M3)) << 16);
          packed.y = static_cast<uint32_t>(__nv_cvt_halfraw2_to_fp8x2(*reinterpret_cast<__half2_raw*>(&w[2]), __NV_SATFINITE, __NV_E4M3)) |
                     (static_cast<uint32_t>(__nv_cvt_halfraw2_to_fp8x2(*reinterpret_cast<__half2_raw*>(&w[3]), __NV_SATFINITE, __NV_E4M3)) << 16);
          *reinterpret_cast<uint2*>(at + (r >> 3) * 1024 + (r & 7) * 128 + ((kt ^ (r & 7)) << 4) + khalf * 8) = packed;
        }
      } else {
#pragma unroll
      for (int idx = warp; idx < 32; idx += DW) {
        const int j = idx & 7;                             // n-tile inside the 128-row block
        const int kt = idx >> 3;
        const int r = j * 16 + row_in_tile;                // row inside the block
        uint4 packed;
        if (KB != 0) {
          constexpr int NW = 8 * (KB == 0 ? 4 : KB);
          const uint32_t* tw = reinterpret_cast<const uint32_t*>(w_ring + sw * S::kWordsSlot) + (kt * 8 + j) * NW;
          uint32_t hi, lo;
          tl.Window(tw[tl.i0], tw[tl.i1], (KB == 4) ? 0u : tw[tl.i2], hi, lo);
          __half2 w[4];
          TrellisDecode8<(KB == 0 ? 4 : KB)>(hi, lo, w);
          packed.x = *reinterpret_cast<uint32_t*>(&w[0]);
          packed.y = *reinterpret_cast<uint32_t*>(&w[1]);
          packed.z = *reinterpret_cast<uint32_t*>(&w[2]);
          packed.w = *reinterpret_cast<uint32_t*>(&w[3]);
        } else {
          const __half* dense = static_cast<const __half*>(wsrc);
          const int n = nb * 128 + r, k = it * kSlabK + kt * 16 + khalf * 8;
          if (MODE == 0 || (n < N && k < K))
            packed = __ldg(reinterpret_cast<const uint4*>(dense + static_cast<size_t>(n) * K + k));
          else
            packed = make_uint4(0u, 0u, 0u, 0u);
        }
        const int chunk = kt * 2 + khalf;                  // 16-byte chunk inside the 128-byte row
        *reinterpret_cast<uint4*>(at + (r >> 3) * 1024 + (r & 7) * 128 + ((chunk ^ (r & 7)) << 4)) = packed;
      }
      }
      ptx::FenceProxyAsyncShared();          // generic-proxy stores -> visible to the tensor core (async proxy)
      __syncwarp();
      if (lane == 0) {
        ptx::MbarArrive(&afull[sa]);
        if (KB != 0) ptx::MbarArrive(&wempty[sw]);
      }
    }

    // ---------------- epilogue (the decode warps: warp w reads TMEM lanes 32 (w % 4) .. +31) ----------------
    // groups of four warps take 32-column chunks round-robin; each group stages its chunk through its
    // own transpose buffer, which lives in the rings (every slot has drained by now)
    if (ok) ok = ptx::MbarWait(accum, 0, abort_flag, 6);
    ptx::TcFenceAfter();
    const float inv_sqrt = 0.08838834764831845f;
    constexpr int kGroups = DW / 4;
    const int q = warp & 3, grp = warp >> 2;
    float* epi = reinterpret_cast<float*>(smem + grp * S::kEpiBytes);
    constexpr int CW = TN < 32 ? 16 : 32;   // columns per TMEM load
    for (int c0 = grp * 32; c0 < TN; c0 += kGroups * 32) {
      if (ok) {
        uint32_t v[32];
        if constexpr (CW == 32) {
          ptx::TmemLoad32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + c0, v);
        } else {
          uint32_t v16[16];
          ptx::TmemLoad32x16(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + c0, v16);
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = v16[i];
        }
        ptx::TmemLoadWait();
#pragma unroll
        for (int c = 0; c < CW; ++c) epi[c * S::kEpiStride + q * 32 + lane] = __uint_as_float(v[c]);
      }
      asm volatile("bar.sync %0, 128;" ::"r"(1 + grp) : "memory");
      if (ok) {
        for (int c = q; c < CW; c += 4) {
          const int t = t0 + c0 + c;
          if (t < t_end && (MODE != 1 || nb * 128 + lane * 4 < N)) {
            const float4 p = *reinterpret_cast<const float4*>(epi + c * S::kEpiStride + lane * 4);
            float f[4] = {p.x, p.y, p.z, p.w};
            const int n = nb * 128 + lane * 4;
            float o0, o1, o2, o3;
            if constexpr (MODE == 0 || MODE == 3 || MODE == 4) {
              if constexpr (MODE == 4) {
                const float xs = __ldg(pl.x_scale + t);               // the row's activation scale
                f[0] *= xs; f[1] *= xs; f[2] *= xs; f[3] *= xs;
              }
              WarpFwht128(f);
              const uint2 sv = *reinterpret_cast<const uint2*>(svh + n);
              const __half2 s01 = *reinterpret_cast<const __half2*>(&sv.x), s23 = *reinterpret_cast<const __half2*>(&sv.y);
              o0 = f[0] * inv_sqrt * __low2float(s01); o1 = f[1] * inv_sqrt * __high2float(s01);
              o2 = f[2] * inv_sqrt * __low2float(s23); o3 = f[3] * inv_sqrt * __high2float(s23);
            } else {
              o0 = f[0]; o1 = f[1]; o2 = f[2]; o3 = f[3];
              if (pl.bias != nullptr) {
                const uint2 bv = *reinterpret_cast<const uint2*>(pl.bias + n);
                o0 += BfLo(bv.x); o1 += BfHi(bv.x); o2 += BfLo(bv.y); o3 += BfHi(bv.y);
              }
              if (pl.act == 1) {
                o0 = GeluTanh(o0); o1 = GeluTanh(o1); o2 = GeluTanh(o2); o3 = GeluTanh(o3);
              } else if (pl.act == 2) {
                o0 = GeluErf(o0); o1 = GeluErf(o1); o2 = GeluErf(o2); o3 = GeluErf(o3);
              }
            }
            if (residual != nullptr) {
              const uint2 rv = *reinterpret_cast<const uint2*>(residual + static_cast<size_t>(t) * N + n);
              o0 += BfLo(rv.x); o1 += BfHi(rv.x); o2 += BfLo(rv.y); o3 += BfHi(rv.y);
            }
            uint2 ov;
            ov.x = PackBf16(o0, o1);
            ov.y = PackBf16(o2, o3);
            if ((MODE == 1 || MODE == 2 || MODE == 5) && pl.out_f32) {
              *reinterpret_cast<float4*>(reinterpret_cast<float*>(y) + static_cast<size_t>(t) * N + n) = make_float4(o0, o1, o2, o3);
            } else if (rs.world > 0) {
              const int owner = t / rs.rows_per_rank, tl = t - owner * rs.rows_per_rank;
              *reinterpret_cast<uint2*>(rs.recv[owner] + (static_cast<size_t>(rs.rank) * rs.rows_per_rank + tl) * N + n) = ov;
            } else if (MODE == 3) {
              *reinterpret_cast<uint2*>(y + static_cast<size_t>(__ldg(pl.g_perm + t)) * N + n) = ov;
            } else {
              *reinterpret_cast<uint2*>(y + static_cast<size_t>(t) * N + n) = ov;
            }
          }
        }
      }
      asm volatile("bar.sync %0, 128;" ::"r"(1 + grp) : "memory");
    }
    if (rs.world > 0) {
      // every partial row of this tile is on its way: publish them, then count this CTA in at each owner it wrote to
      // (also when a wait ran out: the peers must not wait for a CTA that gave up; the status word tells the host)
      __threadfence_system();
      asm volatile("bar.sync 6, %0;" ::"r"(DW * 32) : "memory");
      if (threadIdx.x == 0) {
        const int t_last = min(t0 + TN, T) - 1;
        for (int o = t0 / rs.rows_per_rank; o <= t_last / rs.rows_per_rank; ++o) atomicAdd_system(rs.cnt[o], 1u);
      }
    }
  }

  // ---------------- teardown ----------------
  ptx::TcFenceBefore();
  __syncthreads();
  if (*abort_flag != 0) {
    // give copies that may still be in flight time to land before the shared memory goes away
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    if (threadIdx.x == 0) atomicExch(status, *abort_flag);
  }
  if (warp == DW + 1) ptx::TmemDealloc(tmem_base, kTmemCols);
}

// ---- input transform: Xh = fp16(H128(suh * x)) -------------------------------------------------------
// one warp per 128-block; producer variants fold the preceding elementwise op into the transform
// (reference: src/kernels/src/trellis_transform.hip:84-486 fuses the same producers).
//   mode 0: x = in[t, k]                      (in: [T, K])
//   mode 1: x = silu(in[t, k]) * in[t, K + k] (in: [T, 2K] fused gate|up rows); mode 2: the same with a tanh-GELU gate
__global__ void TrellisInputKernel(const __nv_bfloat16* __restrict__ in, const __half* __restrict__ suh,
                                   __half* __restrict__ out, int T, int K, int mode) {
  const int lane = threadIdx.x & 31;
  const int blocks_per_row = K / 128;
  const long long item = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= static_cast<long long>(T) * blocks_per_row) return;
  const int t = static_cast<int>(item / blocks_per_row), b = static_cast<int>(item % blocks_per_row);
  const int k = b * 128 + lane * 4;
  float v[4];
  if (mode == 0) {
    const uint2 xv = *reinterpret_cast<const uint2*>(in + static_cast<size_t>(t) * K + k);
    v[0] = BfLo(xv.x); v[1] = BfHi(xv.x); v[2] = BfLo(xv.y); v[3] = BfHi(xv.y);
  } else {
    const uint2 g = *reinterpret_cast<const uint2*>(in + static_cast<size_t>(t) * 2 * K + k);
    const uint2 u = *reinterpret_cast<const uint2*>(in + static_cast<size_t>(t) * 2 * K + K + k);
    // the product is rounded to bf16 exactly like the unfused silu_mul kernel rounds it
    const int act = mode == 2 ? 1 : 0;
    const uint32_t p01 = PackBf16(GateAct(BfLo(g.x), act) * BfLo(u.x), GateAct(BfHi(g.x), act) * BfHi(u.x));
    const uint32_t p23 = PackBf16(GateAct(BfLo(g.y), act) * BfLo(u.y), GateAct(BfHi(g.y), act) * BfHi(u.y));
    v[0] = BfLo(p01); v[1] = BfHi(p01); v[2] = BfLo(p23); v[3] = BfHi(p23);
  }
  const uint2 sv = *reinterpret_cast<const uint2*>(suh + k);
  const __half2 s01 = *reinterpret_cast<const __half2*>(&sv.x), s23 = *reinterpret_cast<const __half2*>(&sv.y);
  v[0] *= __low2float(s01); v[1] *= __high2float(s01); v[2] *= __low2float(s23); v[3] *= __high2float(s23);
  WarpFwht128(v);
  const float inv_sqrt = 0.08838834764831845f;
  __half2 o01 = __floats2half2_rn(v[0] * inv_sqrt, v[1] * inv_sqrt), o23 = __floats2half2_rn(v[2] * inv_sqrt, v[3] * inv_sqrt);
  uint2 ov;
  ov.x = *reinterpret_cast<uint32_t*>(&o01);
  ov.y = *reinterpret_cast<uint32_t*>(&o23);
  *reinterpret_cast<uint2*>(out + static_cast<size_t>(t) * K + k) = ov;
}

// ---- grouped experts: tile list and per-expert input transform ---------------------------------------
// One block.  Expert e with n_e planned rows gets ceil(n_e / tn) tiles; tiles are written in expert order.
__global__ void MoeTilesKernel(const int* __restrict__ offsets, int E, int tn, int* __restrict__ tiles,
                               int* __restrict__ ntiles, int max_tiles) {
  __shared__ int scan[1024];
  const int e = threadIdx.x;
  const int n = e < E ? offsets[e + 1] - offsets[e] : 0;
  const int c = (n + tn - 1) / tn;
  scan[e] = c;
  __syncthreads();
  for (int d = 1; d < 1024; d <<= 1) {
    const int v = e >= d ? scan[e - d] : 0;
    __syncthreads();
    scan[e] += v;
    __syncthreads();
  }
  const int base = scan[e] - c;
  if (e < E) {
    const int o = offsets[e];
    for (int j = 0; j < c && base + j < max_tiles; ++j) {
      tiles[2 * (base + j)] = e;
      tiles[2 * (base + j) + 1] = o + j * tn;
    }
  }
  if (e == 1023) *ntiles = min(scan[1023], max_tiles);
}

// xh[p] = fp16(H128(suh[e(p)] * act(in[perm[p] / xdiv]))) for every planned pair p (sorted by expert); one warp per
// 128-block.  The expert of a sorted position is found by bisection of the offsets.
__global__ void TrellisInputGroupedKernel(const __nv_bfloat16* __restrict__ in, const __half* __restrict__ suh,
                                          __half* __restrict__ out, const int* __restrict__ offsets,
                                          const int* __restrict__ perm, int E, int P, int K, int xdiv, int mode) {
  const int lane = threadIdx.x & 31;
  const int blocks_per_row = K / 128;
  const long long item = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= static_cast<long long>(P) * blocks_per_row) return;
  const int p = static_cast<int>(item / blocks_per_row), b = static_cast<int>(item % blocks_per_row);
  if (p >= __ldg(offsets + E)) return;
  int lo = 0, hi = E;                                  // largest e with offsets[e] <= p
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (__ldg(offsets + mid) <= p) lo = mid; else hi = mid;
  }
  const int t = __ldg(perm + p) / xdiv;
  const int k = b * 128 + lane * 4;
  float v[4];
  if (mode == 0) {
    const uint2 xv = *reinterpret_cast<const uint2*>(in + static_cast<size_t>(t) * K + k);
    v[0] = BfLo(xv.x); v[1] = BfHi(xv.x); v[2] = BfLo(xv.y); v[3] = BfHi(xv.y);
  } else {
    const uint2 g = *reinterpret_cast<const uint2*>(in + static_cast<size_t>(t) * 2 * K + k);
    const uint2 u = *reinterpret_cast<const uint2*>(in + static_cast<size_t>(t) * 2 * K + K + k);
    const int act = mode == 2 ? 1 : 0;
    const uint32_t p01 = PackBf16(GateAct(BfLo(g.x), act) * BfLo(u.x), GateAct(BfHi(g.x), act) * BfHi(u.x));
    const uint32_t p23 = PackBf16(GateAct(BfLo(g.y), act) * BfLo(u.y), GateAct(BfHi(g.y), act) * BfHi(u.y));
    v[0] = BfLo(p01); v[1] = BfHi(p01); v[2] = BfLo(p23); v[3] = BfHi(p23);
  }
  const uint2 sv = *reinterpret_cast<const uint2*>(suh + static_cast<size_t>(lo) * K + k);
  const __half2 s01 = *reinterpret_cast<const __half2*>(&sv.x), s23 = *reinterpret_cast<const __half2*>(&sv.y);
  v[0] *= __low2float(s01); v[1] *= __high2float(s01); v[2] *= __low2float(s23); v[3] *= __high2float(s23);
  WarpFwht128(v);
  const float inv_sqrt = 0.08838834764831845f;
  __half2 o01 = __floats2half2_rn(v[0] * inv_sqrt, v[1] * inv_sqrt), o23 = __floats2half2_rn(v[2] * inv_sqrt, v[3] * inv_sqrt);
  uint2 ov;
  ov.x = *reinterpret_cast<uint32_t*>(&o01);
  ov.y = *reinterpret_cast<uint32_t*>(&o23);
  *reinterpret_cast<uint2*>(out + static_cast<size_t>(p) * K + k) = ov;
}

// ---- 8-bit activations: xq = e4m3(xh / scale), scale = rowmax |xh| / 448, one CTA per row ---------------------------
__global__ void __launch_bounds__(256) QuantizeRowsE4m3Kernel(const __half* __restrict__ xh, uint8_t* __restrict__ xq,
                                                              float* __restrict__ scale, int K) {
  __shared__ float red[32];
  const __half* row = xh + static_cast<size_t>(blockIdx.x) * K;
  float amax = 0.f;
  for (int k = threadIdx.x * 8; k < K; k += 256 * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(row + k);
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) amax = fmaxf(amax, fmaxf(fabsf(__low2float(h[i])), fabsf(__high2float(h[i]))));
  }
  amax = WarpMax(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) amax = fmaxf(amax, red[w]);
  const float sc = amax > 0.f ? amax * (1.0f / 448.0f) : 1.0f;
  const float inv = 1.0f / sc;
  if (threadIdx.x == 0) scale[blockIdx.x] = sc;
  uint8_t* out = xq + static_cast<size_t>(blockIdx.x) * K;
  for (int k = threadIdx.x * 8; k < K; k += 256 * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(row + k);
    const __half2* h = reinterpret_cast<const __half2*>(&v);
    uint32_t o[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float2 a = __half22float2(h[2 * i]), b = __half22float2(h[2 * i + 1]);
      const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a.x * inv, a.y * inv), __NV_SATFINITE, __NV_E4M3);
      const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(b.x * inv, b.y * inv), __NV_SATFINITE, __NV_E4M3);
      o[i] = lo | (hi << 16);
    }
    *reinterpret_cast<uint2*>(out + k) = make_uint2(o[0], o[1]);
  }
}

int g_decode_warps = 16;
int g_grouped_decode_warps = 0;      // 0: by tile size

template <int KB, int TN, int DW, int MODE = 0>
int LaunchGemm(const void* wsrc, const void* svh, const void* xh, void* y, const void* residual, int T, int N, int K,
               int* status, cudaStream_t stream, const RsArgs& rs, const PlainArgs& pl = PlainArgs{}) {
  using S = GemmSmem<KB, TN, MODE == 4>;
  static_assert(S::kTotal <= 227 * 1024, "shared memory budget");
  static_assert(S::kBars * 8 + 16 <= 512, "barrier block");
  CUtensorMap tmap;
  const int rc = MODE == 4 ? MakeTensorMap2D8(&tmap, xh, static_cast<uint64_t>(T), static_cast<uint64_t>(K), TN > 256 ? 256 : TN, 128)
                           : MakeTensorMap2D16(&tmap, xh, static_cast<uint64_t>(T), static_cast<uint64_t>(K), TN > 256 ? 256 : TN, kSlabK,
                                               MODE == 1 && pl.bf16 != 0);
  if (rc) return rc;
  CUtensorMap tmap_a = tmap;
  if (MODE == 1) {
    const int ra = MakeTensorMap2D16(&tmap_a, wsrc, static_cast<uint64_t>(N), static_cast<uint64_t>(K), 128, kSlabK, pl.bf16 != 0);
    if (ra) return ra;
  }
  auto kern = TrellisGemmKernel<KB, TN, DW, MODE>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal);
  if (e != cudaSuccess) return static_cast<int>(e);
  dim3 grid((N + 127) / 128, MODE == 3 ? pl.g_max_tiles : (T + TN - 1) / TN);
  kern<<<grid, (DW + 3) * 32, S::kTotal, stream>>>(tmap, tmap_a, wsrc, static_cast<const __half*>(svh),
                                                   static_cast<__nv_bfloat16*>(y),
                                                   static_cast<const __nv_bfloat16*>(residual), T, N, K, status, rs, pl);
  return FinishLaunch();
}

template <int KB>
int LaunchGrouped(const void* w, const void* svh, const void* xh, void* y, int P, int N, int K, int tn, int* status,
                  cudaStream_t s, const PlainArgs& pl) {
  const RsArgs rs = {};
  // measured on the 512-expert block: 1745 -> 1308 us at 2048 rows (tile 64), but 4178 -> 4519 us at 8192 rows (tile 128)
  const int dw = g_grouped_decode_warps ? g_grouped_decode_warps : (tn <= 64 ? 8 : 16);
  if (dw == 8) {
    // eight decode warps: 352 threads per CTA, so two CTAs share an SM and one tile's prologue and epilogue overlap the
    // other's main loop (an expert tile has little K: the fixed part of a CTA is most of its time)
    switch (tn) {
      case 16: return LaunchGemm<KB, 16, 8, 3>(w, svh, xh, y, nullptr, P, N, K, status, s, rs, pl);
      case 32: return LaunchGemm<KB, 32, 8, 3>(w, svh, xh, y, nullptr, P, N, K, status, s, rs, pl);
      case 64: return LaunchGemm<KB, 64, 8, 3>(w, svh, xh, y, nullptr, P, N, K, status, s, rs, pl);
      case 128: return LaunchGemm<KB, 128, 8, 3>(w, svh, xh, y, nullptr, P, N, K, status, s, rs, pl);
      default: return R4DXB_BAD_ARG;
    }
  }
  switch (tn) {
    case 16: return LaunchGemm<KB, 16, 16, 3>(w, svh, xh, y, nullptr, P, N, K, status, s, rs, pl);
    case 32: return LaunchGemm<KB, 32, 16, 3>(w, svh, xh, y, nullptr, P, N, K, status, s, rs, pl);
    case 64: return LaunchGemm<KB, 64, 16, 3>(w, svh, xh, y, nullptr, P, N, K, status, s, rs, pl);
    case 128: return LaunchGemm<KB, 128, 16, 3>(w, svh, xh, y, nullptr, P, N, K, status, s, rs, pl);
    case 256: return LaunchGemm<KB, 256, 16, 3>(w, svh, xh, y, nullptr, P, N, K, status, s, rs, pl);
    default: return R4DXB_BAD_ARG;
  }
}

template <int MODE>
int LaunchPlain(const void* w, const void* xh, void* y, const void* residual, int T, int N, int K, int tn, int* status,
                cudaStream_t s, const PlainArgs& pl) {
  const RsArgs rs = {};
  switch (tn) {
    case 16: return LaunchGemm<0, 16, 8, MODE>(w, nullptr, xh, y, residual, T, N, K, status, s, rs, pl);
    case 32: return LaunchGemm<0, 32, 8, MODE>(w, nullptr, xh, y, residual, T, N, K, status, s, rs, pl);
    case 64: return LaunchGemm<0, 64, 8, MODE>(w, nullptr, xh, y, residual, T, N, K, status, s, rs, pl);
    case 128: return LaunchGemm<0, 128, 8, MODE>(w, nullptr, xh, y, residual, T, N, K, status, s, rs, pl);
    case 256: return LaunchGemm<0, 256, 8, MODE>(w, nullptr, xh, y, residual, T, N, K, status, s, rs, pl);
    case 512: return LaunchGemm<0, 512, 8, MODE>(w, nullptr, xh, y, residual, T, N, K, status, s, rs, pl);
    default: return R4DXB_BAD_ARG;
  }
}

template <int KB, int DW>
int LaunchGemmTN(const void* wsrc, const void* svh, const void* xh, void* y, const void* residual, int T, int N, int K,
                 int tn, int* status, cudaStream_t s, const RsArgs& rs) {
  switch (tn) {
    case 16: return LaunchGemm<KB, 16, DW>(wsrc, svh, xh, y, residual, T, N, K, status, s, rs);
    case 32: return LaunchGemm<KB, 32, DW>(wsrc, svh, xh, y, residual, T, N, K, status, s, rs);
    case 64: return LaunchGemm<KB, 64, DW>(wsrc, svh, xh, y, residual, T, N, K, status, s, rs);
    case 128: return LaunchGemm<KB, 128, DW>(wsrc, svh, xh, y, residual, T, N, K, status, s, rs);
    case 256: return LaunchGemm<KB, 256, DW>(wsrc, svh, xh, y, residual, T, N, K, status, s, rs);
    case 512: return LaunchGemm<KB, 512, DW>(wsrc, svh, xh, y, residual, T, N, K, status, s, rs);
    default: return R4DXB_BAD_ARG;
  }
}

template <int KB>
int LaunchGemmDW(const void* wsrc, const void* svh, const void* xh, void* y, const void* residual, int T, int N, int K,
                 int tn, int* status, cudaStream_t s, const RsArgs& rs) {
  switch (g_decode_warps) {
    case 4: return LaunchGemmTN<KB, 4>(wsrc, svh, xh, y, residual, T, N, K, tn, status, s, rs);
    case 8: return LaunchGemmTN<KB, 8>(wsrc, svh, xh, y, residual, T, N, K, tn, status, s, rs);
    default: return LaunchGemmTN<KB, 16>(wsrc, svh, xh, y, residual, T, N, K, tn, status, s, rs);
  }
}

}  // namespace
}  // namespace r4dxb

using namespace r4dxb;

extern "C" {

int r4dxb_trellis_input(const void* in, const void* suh, void* out, int T, int K, int mode, void* stream) {
  if (T < 1 || K % 128 || mode < 0 || mode > 2) return R4DXB_BAD_ARG;
  const long long items = static_cast<long long>(T) * (K / 128);
  const int warps_per_cta = 8;
  TrellisInputKernel<<<static_cast<unsigned>((items + warps_per_cta - 1) / warps_per_cta), warps_per_cta * 32, 0,
                       static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(in),
                                                            static_cast<const __half*>(suh), static_cast<__half*>(out), T, K, mode);
  return FinishLaunch();
}

/* y[T, N] (bf16) from xh[T, K] (fp16, already input-transformed).  kb = 0: `w` is a dense fp16 [N, K]
 * matrix (svh still applies; pass ones and set hadamard-free weights accordingly); kb in {3,4,5}: packed
 * trellis words.  tn = token tile (16/32/64/128/256/512).  status: device int, set non-zero if a bounded wait
 * inside the kernel ran out. */
/* decode warps per CTA of the tensor-core GEMM (4, 8 or 16): a tuning and A/B-measurement switch */
void r4dxb_set_gemm_decode_warps(int n) {
  g_decode_warps = (n == 4 || n == 8) ? n : 16;
  g_grouped_decode_warps = n == 8 ? 8 : (n == 16 ? 16 : 0);
}

int r4dxb_trellis_gemm(const void* w, const void* svh, const void* xh, void* y, const void* residual, int T, int N, int K,
                       int kb, int tn, int* status, void* stream) {
  if (T < 1 || N % 128 || K % 128) return R4DXB_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  RsArgs rs = {};
  switch (kb) {
    case 0: return LaunchGemmDW<0>(w, svh, xh, y, residual, T, N, K, tn, status, s, rs);
    case 3: return LaunchGemmDW<3>(w, svh, xh, y, residual, T, N, K, tn, status, s, rs);
    case 4: return LaunchGemmDW<4>(w, svh, xh, y, residual, T, N, K, tn, status, s, rs);
    case 5: return LaunchGemmDW<5>(w, svh, xh, y, residual, T, N, K, tn, status, s, rs);
    default: return R4DXB_BAD_ARG;
  }
}

/* Plain linear on the tensor cores, any number of rows: y[T, N] = x[T, K] W^T (+ bias) (+ residual).
 * kind 0: W is a dense 16-bit [N, K] matrix (bf16 != 0: W and x are bf16, else fp16), N a multiple of 4 and K of 8;
 * kind 1: W is w4a16 (wq nibbles [N][K/8] + wsz [N][K/group]), x is fp16, N and K multiples of 128;
 * kind 2: W is w8a16 (offset-binary bytes [N][K] + fp16 scales [N][K/group] passed as wsz), x is fp16, N and K multiples of 128.
 * out_f32: y is fp32 instead of bf16.  act (low byte of out_f32 >> 8): 0 none, 1 tanh-GELU, 2 erf-GELU after the bias. */
int r4dxb_linear_tc(const void* w, const void* wsz, int kind, int group, int bf16, const void* x, void* y, int out_f32,
                    const void* bias, const void* residual, int T, int N, int K, int tn, int* status, void* stream) {
  if (T < 1 || N < 4 || K < 8 || kind < 0 || kind > 2) return R4DXB_BAD_ARG;
  if (kind == 0 && (N % 4 || K % 8)) return R4DXB_BAD_ARG;
  if (kind >= 1 && (N % 128 || K % 128 || wsz == nullptr || (group != 32 && group != 64 && group != 128) || bf16))
    return R4DXB_BAD_ARG;
  PlainArgs pl = {};
  pl.wsz = static_cast<const uint32_t*>(wsz);
  pl.bias = static_cast<const __nv_bfloat16*>(bias);
  pl.group = group;
  pl.bf16 = bf16;
  pl.out_f32 = out_f32 & 1;
  pl.act = (out_f32 >> 8) & 0xFF;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (kind == 2) return LaunchPlain<5>(w, x, y, residual, T, N, K, tn, status, s, pl);
  return kind == 0 ? LaunchPlain<1>(w, x, y, residual, T, N, K, tn, status, s, pl)
                   : LaunchPlain<2>(w, x, y, residual, T, N, K, tn, status, s, pl);
}

/* 8-bit prefill product: rows of fp16 transformed activations -> e4m3 rows + one fp32 scale per row, then the trellis GEMM
 * with e4m3 code values and e4m3 activations on tcgen05.mma kind::f8f6f4 (fp32 accumulate, the row scale applied in the
 * epilogue).  K a multiple of 128; token tiles 128 / 256 / 512. */
int r4dxb_quantize_rows_e4m3(const void* xh, void* xq, float* scale, int T, int K, void* stream) {
  if (T < 1 || K < 8 || K % 8) return R4DXB_BAD_ARG;
  QuantizeRowsE4m3Kernel<<<T, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __half*>(xh), static_cast<uint8_t*>(xq), scale, K);
  return FinishLaunch();
}

int r4dxb_trellis_gemm_f8(const void* w, const void* svh, const void* xq, const float* x_scale, void* y, const void* residual,
                          int T, int N, int K, int kb, int tn, int* status, void* stream) {
  if (T < 1 || N % 128 || K % 128 || x_scale == nullptr) return R4DXB_BAD_ARG;
  const RsArgs rs = {};
  PlainArgs pl = {};
  pl.x_scale = x_scale;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define R4DXB_F8(KBV, TNV) if (kb == KBV && tn == TNV) return LaunchGemm<KBV, TNV, 16, 4>(w, svh, xq, y, residual, T, N, K, status, s, rs, pl);
  R4DXB_F8(3, 128) R4DXB_F8(3, 256) R4DXB_F8(3, 512) R4DXB_F8(4, 128) R4DXB_F8(4, 256) R4DXB_F8(4, 512)
  R4DXB_F8(5, 128) R4DXB_F8(5, 256) R4DXB_F8(5, 512)
#undef R4DXB_F8
  return R4DXB_BAD_ARG;
}

/* Grouped experts on the tensor cores (prefill and wide batches of the mixture-of-experts block).
 * r4dxb_moe_tiles: tile list of the routing plan for token tiles of tn rows (E <= 1024 local experts).
 * r4dxb_trellis_input_grouped: xh[p] = fp16(H128(suh[e(p)] * act(in[perm[p] / xdiv]))) for the planned pairs in expert order.
 * r4dxb_trellis_gemm_grouped: y[perm[p]] = svh[e] * H128(xh[p] Q_e^T); max_tiles >= P / tn + E bounds the grid. */
int r4dxb_moe_tiles(const int* offsets, int E, int tn, int* tiles, int* ntiles, int max_tiles, void* stream) {
  if (E < 1 || E > 1024 || tn < 1 || max_tiles < 1) return R4DXB_BAD_ARG;
  MoeTilesKernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(offsets, E, tn, tiles, ntiles, max_tiles);
  return FinishLaunch();
}

int r4dxb_trellis_input_grouped(const void* in, const void* suh, void* out, const int* offsets, const int* perm, int E, int P,
                                int K, int xdiv, int mode, void* stream) {
  if (P < 1 || K % 128 || xdiv < 1 || mode < 0 || mode > 2) return R4DXB_BAD_ARG;
  const long long items = static_cast<long long>(P) * (K / 128);
  TrellisInputGroupedKernel<<<static_cast<unsigned>((items + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(in), static_cast<const __half*>(suh), static_cast<__half*>(out), offsets, perm, E, P, K,
      xdiv, mode);
  return FinishLaunch();
}

int r4dxb_trellis_gemm_grouped(const void* words, const void* svh, const void* xh, void* y, const int* offsets, const int* perm,
                               const int* tiles, const int* ntiles, int max_tiles, int P, int E, int N, int K, int kb, int tn,
                               int* status, void* stream) {
  if (P < 1 || E < 1 || N % 128 || K % 128 || max_tiles < 1 || max_tiles > 65535) return R4DXB_BAD_ARG;
  PlainArgs pl = {};
  pl.g_offsets = offsets;
  pl.g_perm = perm;
  pl.g_tiles = tiles;
  pl.g_ntiles = ntiles;
  pl.g_words = static_cast<long long>(N / 16) * (K / 16) * 8 * kb;
  pl.g_max_tiles = max_tiles;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (kb) {
    case 3: return LaunchGrouped<3>(words, svh, xh, y, P, N, K, tn, status, s, pl);
    case 4: return LaunchGrouped<4>(words, svh, xh, y, P, N, K, tn, status, s, pl);
    case 5: return LaunchGrouped<5>(words, svh, xh, y, P, N, K, tn, status, s, pl);
    default: return R4DXB_BAD_ARG;
  }
}

/* Row-parallel product with the reduce-scatter in its epilogue: partial row t goes to rank t / rows_per_rank, into
 * recv[owner] + (rank * rows_per_rank + t % rows_per_rank) * N (bf16), and every CTA adds 1 to cnt[owner] for each
 * owner its token tile touches, after its rows are visible at system scope.  recv / cnt: `world` peer-mapped pointers. */
int r4dxb_trellis_gemm_rs(const void* w, const void* svh, const void* xh, int T, int N, int K, int kb, int tn, int* status,
                          void* const* recv, void* const* cnt, int world, int rank, int rows_per_rank, void* stream) {
  if (T < 1 || N % 128 || K % 128 || world < 2 || world > 8 || rank < 0 || rank >= world || rows_per_rank < 1 ||
      static_cast<long long>(rows_per_rank) * world < T)
    return R4DXB_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  RsArgs rs = {};
  for (int p = 0; p < world; ++p) {
    rs.recv[p] = static_cast<__nv_bfloat16*>(recv[p]);
    rs.cnt[p] = static_cast<unsigned*>(cnt[p]);
  }
  rs.world = world; rs.rank = rank; rs.rows_per_rank = rows_per_rank;
  switch (kb) {
    case 3: return LaunchGemmDW<3>(w, svh, xh, nullptr, nullptr, T, N, K, tn, status, s, rs);
    case 4: return LaunchGemmDW<4>(w, svh, xh, nullptr, nullptr, T, N, K, tn, status, s, rs);
    case 5: return LaunchGemmDW<5>(w, svh, xh, nullptr, nullptr, T, N, K, tn, status, s, rs);
    default: return R4DXB_BAD_ARG;
  }
}

}  // extern "C"
