// Trellis weight-streaming product for T <= 8 activation rows on the 5th-generation tensor cores, with the
// decoded weights going register -> tensor memory and never touching shared memory.
//
//   y[t, n] = bf16( svh[n] * H128( sum_k Q[n, k] * xh[t, k] )[n] (+ residual[t, n]) ),  xh = H128(suh (.) act(x))
//
// Why this is not the CUDA-core kernel of trellis_gemv.cu.  A code value is  Q = c * scale + bias  with
// c = 1024 + bytesum(state * 0x83DCD12D), an integer that fp16 holds exactly, so
//     sum_k Q[n, k] x[k]  =  scale * sum_k c[n, k] x[k]  +  bias * sum_k x[k].
// The decode therefore stops at c (extract, multiply, byte sum, pack two to a register): no scale/bias FMA and
// no multiply-accumulate on the CUDA cores, ~4 lane-instructions per weight instead of ~7.  The contraction
// runs as tcgen05.mma kind::f16 (M = 128 output rows, N = 8 activation rows, K = 16 per instruction):
//   * A lives in TENSOR MEMORY: thread r of a decode warpgroup owns row r of the 128-row block, decodes the 16
//     states of its row of a 16x16 tile and writes them as 8 half2 columns of its TMEM lane with one tcgen05.st;
//   * B is the transformed activation slice itself, written once by the prologue into shared memory in the
//     K-major core-matrix layout (8 rows x 16 bytes), so no per-stage operand staging exists at all;
//   * D (128 x 8, fp32) accumulates in tensor memory, in four tiles taken in turn; products c * x are exact in
//     fp32 and the epilogue applies  scale * D + bias * sum_k x[k]  (the row sums come from the prologue, added
//     in a fixed order).
// Against the definition of the format (each code value rounded to fp16 once) the value used here is the
// unrounded c * scale + bias, i.e. at most half an fp16 ulp away.
//
// (An int8 variant - the four hash bytes as unsigned 8-bit K' = 4K operand, activations split into two signed
// bytes - decodes in ~3 instructions per weight but needs twice the MMA instructions; at the measured ~50 clocks
// per M = 128 instruction with A in tensor memory it is capped near 20 weights per clock and SM, below this one.)
//
// Around that core the kernel keeps the structure of the CUDA-core version: one CTA per (128-row block, K
// slice), `ksplit` CTAs of a cluster reduced over distributed shared memory in rank order, bulk-copy stage ring
// for the packed words, RMSNorm / gated-MLP prologues, residual and tensor-parallel all-reduce epilogues,
// programmatic dependent launch.  Roles: warps 0-7 decode (two warpgroups; warp w owns TMEM lanes 32 (w % 4)..;
// group g takes k-tiles 4g .. 4g+3 of every 128-wide K block) and issue their group's MMAs in turn, warp 8
// streams the words.  (A dedicated MMA-issuing warp was tried first: next to sixteen busy decode warps every step
// of its dependent chain of barrier and tcgen05 instructions took ~300 clocks, and it became the bottleneck.)
//
// Tensor memory is allocated BEFORE the kernel lets its dependents launch: a dependent CTA that took the columns
// first and then sat in griddepcontrol.wait would block this grid's allocation for ever.
//
// The reference engine has no counterpart of this scheme; the job is that of its input-transform + WMMA GEMM for
// M <= 8 (reference: third_party/libr4d/r4d_gemm_trellis_nt_m64.hip:30-90,216).
#include <cooperative_groups.h>

#include "sm100_ptx.cuh"
#include "tp_push.cuh"
#include "r4dxb_trellis.h"

namespace cg = cooperative_groups;

namespace r4dxb {
namespace {

constexpr int kDecodeWarps = 8;
constexpr int kProducerWarp = 8;
constexpr int kThreads = 288;
constexpr int kMaxStages = 6;
constexpr uint32_t kTmemCols = 256;        // D: kAccs tiles of 8 columns from column 0; A: kACol + 64 * (K block % 3)
constexpr int kAccs = 8;                   // accumulator tiles: four per decode group, taken in turn (MMAs chained on one tile serialise)
constexpr int kABufs = 3;                  // A buffers of 64 columns (one 128-wide K block each), shared by the two groups
constexpr uint32_t kACol = 64;

struct Ctl {                               // control block at the start of dynamic shared memory
  uint64_t full[kMaxStages], empty[kMaxStages];
  uint64_t a_full[kABufs], a_empty[kABufs];
  uint64_t d_full, red_bar;
  uint32_t tmem_base;
  int abort_flag;
  float rnorm[8];
  float sx[8];
};
constexpr int kCtlBytes = 512;
static_assert(sizeof(Ctl) <= kCtlBytes, "control block");

struct MmaArgs {
  const uint32_t* words;
  const __half* suh;
  const __half* svh;
  const __nv_bfloat16* x;
  __nv_bfloat16* y;
  const __nv_bfloat16* residual;
  const __nv_bfloat16* norm_w;
  float eps;
  int T, N, K, kblocks_per_cta, stages;
  int act;
  int* status;                             // set to 500 + role code when a bounded wait inside the CTA ran out
};


// ---- decode: 16 consecutive states of one tile row out of a 96-bit window ------------------------------------
// The row rl of a tile holds positions 16 rl .. 16 rl + 15; its last state ends at stream bit E = 16 KB (rl + 1).
// x2:x1:x0 is the 96-bit big-endian window that ends at E (bit 0 of x0 = stream bit E - 1).
template <int KB>
struct RowWindow {
  int i0, i1, i2, i3;
  int off;
  __device__ __forceinline__ void Init(int rl) {
    constexpr int R = 256 * KB, NW = 8 * KB;
    int b0 = 16 * KB * (rl + 1) - 96;
    if (b0 < 0) b0 += R;
    i0 = b0 >> 5;
    off = b0 & 31;
    i1 = (i0 + 1) % NW;
    i2 = (i0 + 2) % NW;
    i3 = (i0 + 3) % NW;
  }
  __device__ __forceinline__ void Load(const uint32_t* tw, uint32_t& x2, uint32_t& x1, uint32_t& x0) const {
    if constexpr (KB == 4) {               // the window is word aligned for every row
      x2 = tw[i0];
      const uint2 v = *reinterpret_cast<const uint2*>(tw + i1);     // i1 = 2 rl: 8-byte aligned
      x1 = v.x;
      x0 = v.y;
    } else {
      const uint32_t a = tw[i0], b = tw[i1], c = tw[i2], d = tw[i3];
      x2 = __funnelshift_l(b, a, off);
      x1 = __funnelshift_l(c, b, off);
      x0 = __funnelshift_l(d, c, off);
    }
  }
};

template <int KB, int J>
__device__ __forceinline__ uint32_t RowState(uint32_t x2, uint32_t x1, uint32_t x0) {
  constexpr int sh = KB * (15 - J);
  constexpr int q = sh >> 5, r = sh & 31;
  const uint32_t lo = q == 0 ? x0 : (q == 1 ? x1 : x2);
  const uint32_t hi = q == 0 ? x1 : x2;
  if constexpr (r == 0) return lo & 0xFFFFu;
  else if constexpr (r == 16) return lo >> 16;
  else if constexpr (r < 16) return (lo >> r) & 0xFFFFu;
  else return __funnelshift_r(lo, hi, r) & 0xFFFFu;
}

// c = 1024 + bytesum(state * MUL) as fp16 bits: 0x6400 is 1024.0 and one unit in the last place is 1 there
__device__ __forceinline__ uint32_t CodeBits(uint32_t state) {
  return __dp4a(state * R4DXB_TRELLIS_MUL, 0x01010101u, 0x6400u);
}
__device__ __forceinline__ uint32_t Pack2(uint32_t s_even, uint32_t s_odd) {
  return __byte_perm(CodeBits(s_even), CodeBits(s_odd), 0x5410);
}

// 16 code values of one tile row as 8 half2 registers (k, k+1 pairs).
template <int KB>
__device__ __forceinline__ void DecodeRow16(uint32_t x2, uint32_t x1, uint32_t x0, uint32_t (&h)[8]) {
  if constexpr (KB == 4) {
    // States sit on nibble boundaries.  With the window also shifted by 4, 16 and 20 bits every state is two whole
    // bytes of some 32-bit word, and one byte permute (with a zero register) extracts it: 22 ALU instructions
    // for 16 states instead of 28 shift-and-mask pairs.
    const uint32_t y0 = __funnelshift_r(x0, x1, 16), y1 = __funnelshift_r(x1, x2, 16);    // bits 16.., 48..
    const uint32_t z0 = __funnelshift_r(x0, x1, 4), z1 = __funnelshift_r(x1, x2, 4);      // bits 4.., 36..
    const uint32_t u0 = __funnelshift_r(x0, x1, 20), u1 = __funnelshift_r(x1, x2, 20);    // bits 20.., 52..
    auto b01 = [](uint32_t w) { return __byte_perm(w, 0u, 0x4410); };   // bytes 0-1
    auto b12 = [](uint32_t w) { return __byte_perm(w, 0u, 0x4421); };   // bytes 1-2
    auto b23 = [](uint32_t w) { return __byte_perm(w, 0u, 0x4432); };   // bytes 2-3
    // position j has shift 4 (15 - j) from the end of the window
    h[7] = Pack2(b01(z0), b01(x0));      // j = 14 (sh 4), 15 (sh 0)
    h[6] = Pack2(b12(z0), b12(x0));      // j = 12 (sh 12), 13 (sh 8)
    h[5] = Pack2(b01(u0), b01(y0));      // j = 10 (sh 20), 11 (sh 16)
    h[4] = Pack2(b12(u0), b12(y0));      // j = 8 (sh 28), 9 (sh 24)
    h[3] = Pack2(b01(z1), b01(x1));      // j = 6 (sh 36), 7 (sh 32)
    h[2] = Pack2(b12(z1), b12(x1));      // j = 4 (sh 44), 5 (sh 40)
    h[1] = Pack2(b01(u1), b01(y1));      // j = 2 (sh 52), 3 (sh 48)
    h[0] = Pack2(b12(u1), b12(y1));      // j = 0 (sh 60), 1 (sh 56)
    (void)b23;
  } else {
#define R4DXB_H(P) h[P] = Pack2(RowState<KB, 2 * P>(x2, x1, x0), RowState<KB, 2 * P + 1>(x2, x1, x0));
    R4DXB_H(0) R4DXB_H(1) R4DXB_H(2) R4DXB_H(3) R4DXB_H(4) R4DXB_H(5) R4DXB_H(6) R4DXB_H(7)
#undef R4DXB_H
  }
}

template <int KB, int TMAX, int PRO, bool kTp>
__global__ void __launch_bounds__(kThreads, 2)
TrellisGemvMmaKernel(MmaArgs a, TpPush tp) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  cg::cluster_group cluster = cg::this_cluster();
  const int ksplit = gridDim.x;
  const int krank = blockIdx.x;            // == rank inside the cluster
  const int nb = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nstage = a.kblocks_per_cta;    // 128-wide K blocks of this CTA
  const int kslice = nstage * 128;
  const int k_begin = krank * kslice;
  const int T = a.T, N = a.N, K = a.K;
  constexpr int NW = 8 * KB;
  constexpr int kStageBytes = 8 * 8 * NW * 4;     // 8 k-tiles x 8 n-tiles

  Ctl* ctl = reinterpret_cast<Ctl*>(smem_raw);
  float* part = reinterpret_cast<float*>(smem_raw + kCtlBytes);                        // [ksplit][TMAX][128] (cluster rank 0)
  float* bsum = part + ksplit * TMAX * 128;                                            // [TMAX][nstage] sums of xs per K block
  // B operand: xs[t][k] as fp16 in K-major core matrices: 8 consecutive k of 8 rows = 128 contiguous bytes
  unsigned char* xs = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(bsum + TMAX * nstage) + 127) & ~uintptr_t(127));   // [kslice / 8][8 rows][8 halfs]
  unsigned char* wst = xs + static_cast<size_t>(kslice) * 16;                          // [stages][kStageBytes]
  volatile int* abort_flag = &ctl->abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < a.stages; ++s) {
      ptx::MbarInit(&ctl->full[s], 1);
      ptx::MbarInit(&ctl->empty[s], 4);           // the four warps of the group that decodes the block
    }
    for (int c = 0; c < kABufs; ++c) {
      ptx::MbarInit(&ctl->a_full[c], 4);
      ptx::MbarInit(&ctl->a_empty[c], 4);         // one commit per issuing warp
    }
    ptx::MbarInit(&ctl->d_full, 8);
    ptx::MbarInit(&ctl->red_bar, ksplit * 4);
    ctl->abort_flag = 0;
    ptx::MbarFenceInit();
  }
  __syncthreads();
  if (ksplit > 1) asm volatile("barrier.cluster.arrive.release;" ::: "memory");

  // the weight stream depends on nothing: fill the ring before anything can block
  const unsigned char* wsrc = reinterpret_cast<const unsigned char*>(a.words) +
                              (static_cast<size_t>(nb) * (K / 128) + static_cast<size_t>(krank) * nstage) * kStageBytes;
  if (warp == kProducerWarp) {
    if (lane == 0) {
      for (int it = 0; it < a.stages; ++it) {
        ptx::MbarArriveExpectTx(&ctl->full[it], kStageBytes);
        ptx::BulkLoad(wst + static_cast<size_t>(it) * kStageBytes, wsrc + static_cast<size_t>(it) * kStageBytes, kStageBytes,
                      &ctl->full[it]);
      }
    }
    __syncwarp();
    ptx::TmemAlloc(&ctl->tmem_base, kTmemCols);
    ptx::TmemRelinquish();
  }
  ptx::TcFenceBefore();
  __syncthreads();
  ptx::TcFenceAfter();
  const uint32_t tbase = ctl->tmem_base;
  // tensor memory is ours: the next kernel in the stream may begin its own launch and weight prefetch
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == kProducerWarp) {
    // ---------------- producer: the rest of this CTA's words through the stage ring ----------------
    if (lane == 0) {
      int s = 0;
      uint32_t phase = 0;          // parity of the first release of stage s
      for (int it = a.stages; it < nstage; ++it) {
        if (!ptx::MbarWait(&ctl->empty[s], phase, abort_flag, 1)) break;
        ptx::MbarArriveExpectTx(&ctl->full[s], kStageBytes);
        ptx::BulkLoad(wst + static_cast<size_t>(s) * kStageBytes, wsrc + static_cast<size_t>(it) * kStageBytes, kStageBytes,
                      &ctl->full[s]);
        if (++s == a.stages) { s = 0; phase ^= 1u; }
      }
    }
    __syncwarp();
  } else {
    // ---------------- prologue (decode warps): xs = fp16(H128(suh * act(x))) for this K slice ----------------
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if constexpr (PRO == 1) {
      float* part_ss = part;              // [TMAX][8] partial sums; the split-K partials that live here come much later
      const int kw = (K / 8 + 7) & ~7;
      const int k_lo = warp * kw, k_hi = min(K, k_lo + kw);
#pragma unroll
      for (int t = 0; t < TMAX; ++t) {
        float ss = 0.f;
        if (t < T) {
          const __nv_bfloat16* row = a.x + static_cast<size_t>(t) * K;
          for (int k = k_lo + lane * 8; k < k_hi; k += 256) {
            const uint4 v = *reinterpret_cast<const uint4*>(row + k);
            ss += BfLo(v.x) * BfLo(v.x) + BfHi(v.x) * BfHi(v.x) + BfLo(v.y) * BfLo(v.y) + BfHi(v.y) * BfHi(v.y) +
                  BfLo(v.z) * BfLo(v.z) + BfHi(v.z) * BfHi(v.z) + BfLo(v.w) * BfLo(v.w) + BfHi(v.w) * BfHi(v.w);
          }
          ss = WarpSum(ss);
        }
        if (lane == 0) part_ss[t * 8 + warp] = ss;
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (threadIdx.x < TMAX) {
        float ss = 0.f;
#pragma unroll
        for (int w8 = 0; w8 < 8; ++w8) ss += part_ss[threadIdx.x * 8 + w8];
        ctl->rnorm[threadIdx.x] = rsqrtf(ss / K + a.eps);
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");
    }
    const float inv_sqrt = 0.08838834764831845f;   // 1 / sqrt(128)
    for (int item = warp; item < nstage * TMAX; item += kDecodeWarps) {
      const int t = item / nstage, b = item % nstage;
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      const int k = k_begin + b * 128 + lane * 4;
      if (t < T) {
        if constexpr (PRO == 2) {
          const uint2 g = *reinterpret_cast<const uint2*>(a.x + static_cast<size_t>(t) * 2 * K + k);
          const uint2 u = *reinterpret_cast<const uint2*>(a.x + static_cast<size_t>(t) * 2 * K + K + k);
          const uint32_t p01 = PackBf16(GateAct(BfLo(g.x), a.act) * BfLo(u.x), GateAct(BfHi(g.x), a.act) * BfHi(u.x));
          const uint32_t p23 = PackBf16(GateAct(BfLo(g.y), a.act) * BfLo(u.y), GateAct(BfHi(g.y), a.act) * BfHi(u.y));
          v[0] = BfLo(p01); v[1] = BfHi(p01); v[2] = BfLo(p23); v[3] = BfHi(p23);
        } else {
          const uint2 xv = *reinterpret_cast<const uint2*>(a.x + static_cast<size_t>(t) * K + k);
          v[0] = BfLo(xv.x); v[1] = BfHi(xv.x); v[2] = BfLo(xv.y); v[3] = BfHi(xv.y);
          if constexpr (PRO == 1) {
            const uint2 wv = *reinterpret_cast<const uint2*>(a.norm_w + k);
            const float r = ctl->rnorm[t];
            // same rounding point as the standalone norm kernel: the normalised row is a bf16 tensor
            const uint32_t p01 = PackBf16(v[0] * r * (1.f + BfLo(wv.x)), v[1] * r * (1.f + BfHi(wv.x)));
            const uint32_t p23 = PackBf16(v[2] * r * (1.f + BfLo(wv.y)), v[3] * r * (1.f + BfHi(wv.y)));
            v[0] = BfLo(p01); v[1] = BfHi(p01); v[2] = BfLo(p23); v[3] = BfHi(p23);
          }
        }
        const uint2 sv = *reinterpret_cast<const uint2*>(a.suh + k);
        const __half2 s01 = *reinterpret_cast<const __half2*>(&sv.x), s23 = *reinterpret_cast<const __half2*>(&sv.y);
        v[0] *= __low2float(s01); v[1] *= __high2float(s01); v[2] *= __low2float(s23); v[3] *= __high2float(s23);
      }
      WarpFwht128(v);
      const __half2 o01 = __floats2half2_rn(v[0] * inv_sqrt, v[1] * inv_sqrt);
      const __half2 o23 = __floats2half2_rn(v[2] * inv_sqrt, v[3] * inv_sqrt);
      uint2 ov;
      ov.x = *reinterpret_cast<const uint32_t*>(&o01);
      ov.y = *reinterpret_cast<const uint32_t*>(&o23);
      // core matrix (b * 16 + lane / 2), row t, 8-byte half (lane & 1)
      *reinterpret_cast<uint2*>(xs + (b * 16 + (lane >> 1)) * 128 + t * 16 + (lane & 1) * 8) = ov;
      // sum of the block's (rounded) values, for the bias term of the code
      const float bs = WarpSum(__low2float(o01) + __high2float(o01) + __low2float(o23) + __high2float(o23));
      if (lane == 0) bsum[t * nstage + b] = bs;
    }
    ptx::FenceProxyAsyncShared();                  // xs is read by the tensor core (async proxy)
    asm volatile("bar.sync 1, 256;" ::: "memory");
    if (warp < TMAX) {                             // fixed order: the row sum does not depend on timing
      float sacc = 0.f;
      for (int b = lane; b < nstage; b += 32) sacc += bsum[warp * nstage + b];
      sacc = WarpSum(sacc);
      if (lane == 0) ctl->sx[warp] = sacc;
    }

    // ---------------- main loop: decode rows into tensor memory, issue the block's MMAs ----------------
    // The two warpgroups take the 128-wide K blocks alternately; a block goes into A buffer (block % 3), so a
    // buffer is refilled three blocks after the MMAs that read it were issued and nobody ever waits for them.
    const int wg = warp >> 2, w4 = warp & 3;
    const int r = w4 * 32 + lane;                 // output row inside the 128-row block = TMEM lane
    const int ntile = r >> 4, rl = r & 15;
    RowWindow<KB> rw;
    rw.Init(rl);
    const uint32_t t_lane = tbase + (static_cast<uint32_t>(w4 * 32) << 16);
    constexpr uint32_t idesc = ptx::UmmaInstrDescF16(128, 8, false);
    const uint64_t bdesc0 = ptx::UmmaDescNoSwizzle(ptx::SmemAddr(xs), 128, 128);
    bool ok = true;
    for (int it = wg; it < nstage; it += 2) {
      const int s = it % a.stages, buf = it % kABufs;
      const uint32_t sphase = static_cast<uint32_t>(it / a.stages) & 1u;       // parity of this fill of stage s
      const uint32_t use_par = static_cast<uint32_t>(it / kABufs) & 1u;        // parity of this use of the A buffer
      if (ok) ok = ptx::WarpMbarWait(&ctl->full[s], sphase, abort_flag, 2);
      // the buffer's columns are free once the MMAs that read their previous contents have finished
      if (ok) ok = ptx::WarpMbarWait(&ctl->a_empty[buf], use_par ^ 1u, abort_flag, 5);
      if (ok) {
        ptx::TcFenceAfter();
        const uint32_t* sw = reinterpret_cast<const uint32_t*>(wst + static_cast<size_t>(s) * kStageBytes) + ntile * NW;
        const uint32_t acol = t_lane + kACol + buf * 64;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          uint32_t x2, x1, x0;
          rw.Load(sw + kk * 8 * NW, x2, x1, x0);
          uint32_t h[8];
          DecodeRow16<KB>(x2, x1, x0, h);
          ptx::TmemStore32x8(acol + kk * 8, h);
        }
      }
      __syncwarp();
      if (lane == 0) ptx::MbarArrive(&ctl->empty[s]);        // this warp has read the block's words
      ptx::TmemStoreWait();
      ptx::TcFenceBefore();
      __syncwarp();
      if (lane == 0) ptx::MbarArrive(&ctl->a_full[buf]);
      if (lane == 0 && ok) {
        // every warp issues the MMAs of two of the block's eight k-tiles once all four warps' rows are in: the
        // issue cost (~50 clocks per instruction) is spread evenly instead of making one warp late for the next block
        if (ptx::MbarWait(&ctl->a_full[buf], use_par, abort_flag, 4)) {
          ptx::TcFenceAfter();
          const uint64_t bdesc = bdesc0 + static_cast<uint64_t>(((it * 16 + w4 * 4) * 128) >> 4);
#pragma unroll
          for (int i = 0; i < 2; ++i)
            ptx::UmmaF16FromTmem(tbase + (wg * 4 + w4) * 8, tbase + kACol + buf * 64 + (w4 * 2 + i) * 8,
                                 bdesc + static_cast<uint64_t>((i * 2 * 128) >> 4), idesc, (it >= 2 || i >= 1) ? 1u : 0u);
          ptx::UmmaCommit(&ctl->a_empty[buf]);
          if (it + 2 >= nstage) ptx::UmmaCommit(&ctl->d_full);      // this group's last block
        }
      }
      __syncwarp();
    }
    if (wg >= nstage && lane == 0) ptx::MbarArrive(&ctl->d_full);   // a one-block slice: group 1 has nothing to add

    // ---------------- accumulators -> fp32 partial rows -> cluster rank 0 ----------------
    if (ksplit > 1) asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
    if (wg == 0) {
      const bool dok = ptx::WarpMbarWait(&ctl->d_full, 0, abort_flag, 6);
      ptx::TcFenceAfter();
      uint32_t d[32], d1[32];
      ptx::TmemLoad32x32(t_lane, d);               // eight accumulator tiles of 8 columns
      ptx::TmemLoad32x32(t_lane + 32, d1);
      ptx::TmemLoadWait();
      asm volatile("bar.sync 4, 128;" ::: "memory");         // the row sums written by warps 0..TMAX-1 before their main loop
      float* dst = ksplit > 1 ? cluster.map_shared_rank(part, 0) : part;
      dst += krank * TMAX * 128;
      const float kScale = __half2float(__ushort_as_half(R4DXB_TRELLIS_SCALE_F16));
      const float kBias = __half2float(__ushort_as_half(R4DXB_TRELLIS_BIAS_F16));
#pragma unroll
      for (int t = 0; t < TMAX; ++t) {
        const float g0 = (__uint_as_float(d[t]) + __uint_as_float(d[8 + t])) + (__uint_as_float(d[16 + t]) + __uint_as_float(d[24 + t]));
        const float g1 = (__uint_as_float(d1[t]) + __uint_as_float(d1[8 + t])) + (__uint_as_float(d1[16 + t]) + __uint_as_float(d1[24 + t]));
        const float dsum = nstage > 1 ? g0 + g1 : g0;          // a one-block slice never touches the second group's tiles
        dst[t * 128 + r] = (dok && t < T) ? fmaf(kScale, dsum, kBias * ctl->sx[t]) : 0.f;
      }
      __syncwarp();
      if (lane == 0) {
        uint32_t remote_bar;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_bar) : "r"(ptx::SmemAddr(&ctl->red_bar)), "r"(0));
        asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar) : "memory");
      }
    }
  }
  if (warp >= kDecodeWarps) {
    __syncwarp();
    if (ksplit > 1) asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
  }

  // ---------------- epilogue (cluster rank 0) ----------------
  if (krank == 0 && warp < kDecodeWarps) {
    {
      bool landed = false;
      for (int i = 0; i < ptx::kSpinLimit && !landed; ++i) {
        uint32_t okw;
        asm volatile(
            "{ .reg .pred p; mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
            : "=r"(okw) : "r"(ptx::SmemAddr(&ctl->red_bar)), "r"(0) : "memory");
        landed = okw != 0;
        if (!landed && (i & 63) == 63 && *abort_flag) break;
      }
      if (!landed && lane == 0) *abort_flag = 7;
    }
    const float inv_sqrt = 0.08838834764831845f;
    float o[4] = {0.f, 0.f, 0.f, 0.f};
    const int t = warp;              // warp t finishes row t (T <= 8 = decode warps)
    const int n = nb * 128 + lane * 4;
    if (t < T) {
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      for (int rk = 0; rk < ksplit; ++rk) {       // fixed order: the result does not depend on timing
        const float4 p = *reinterpret_cast<const float4*>(part + (rk * TMAX + t) * 128 + lane * 4);
        v[0] += p.x; v[1] += p.y; v[2] += p.z; v[3] += p.w;
      }
      WarpFwht128(v);
      const uint2 sv = *reinterpret_cast<const uint2*>(a.svh + n);
      const __half2 s01 = *reinterpret_cast<const __half2*>(&sv.x), s23 = *reinterpret_cast<const __half2*>(&sv.y);
      o[0] = v[0] * inv_sqrt * __low2float(s01); o[1] = v[1] * inv_sqrt * __high2float(s01);
      o[2] = v[2] * inv_sqrt * __low2float(s23); o[3] = v[3] * inv_sqrt * __high2float(s23);
    }
    if constexpr (kTp) {
      const unsigned seq = tp.block_seq[nb] + 1;     // written only by this CTA, after the barrier below
      if (t < T) TpAllReduceRow(tp, seq, t, N, n, o);
      asm volatile("bar.sync 2, 256;" ::: "memory");
      if (threadIdx.x == 0) tp.block_seq[nb] = seq;
    }
    if (t < T) {
      if (a.residual != nullptr) {
        const uint2 rv = *reinterpret_cast<const uint2*>(a.residual + static_cast<size_t>(t) * N + n);
        o[0] += BfLo(rv.x); o[1] += BfHi(rv.x); o[2] += BfLo(rv.y); o[3] += BfHi(rv.y);
      }
      uint2 ov;
      ov.x = PackBf16(o[0], o[1]);
      ov.y = PackBf16(o[2], o[3]);
      *reinterpret_cast<uint2*>(a.y + static_cast<size_t>(t) * N + n) = ov;
    }
  }

  // ---------------- release tensor memory ----------------
  ptx::TcFenceBefore();
  __syncthreads();
  if (warp == kProducerWarp) {
    ptx::TcFenceAfter();
    ptx::TmemDealloc(tbase, kTmemCols);
  }
  if (threadIdx.x == 0 && ctl->abort_flag != 0 && a.status != nullptr) atomicCAS(a.status, 0, 500 + ctl->abort_flag);
}

size_t SmemBytes(int tmax, int kslice, int stages, int kb, int ksplit) {
  return kCtlBytes + static_cast<size_t>(ksplit) * tmax * 128 * 4 + static_cast<size_t>(tmax) * (kslice / 128) * 4 + 128 +
         static_cast<size_t>(kslice) * 16 + static_cast<size_t>(stages) * 8 * 8 * 8 * kb * 4;
}

template <int KB, int TMAX, int PRO, bool kTp>
int Launch(MmaArgs a, int ksplit, cudaStream_t stream, const TpPush& tp) {
  a.kblocks_per_cta = a.K / 128 / ksplit;
  const int kslice = a.kblocks_per_cta * 128;
  // ring depth: everything in flight for short slices, otherwise as many stages (up to 6) as keep two CTAs on an SM
  int stages = a.kblocks_per_cta < kMaxStages ? a.kblocks_per_cta : kMaxStages;
  while (stages > 2 && SmemBytes(TMAX, kslice, stages, KB, ksplit) > 112 * 1024) --stages;
  a.stages = stages;
  const size_t smem = SmemBytes(TMAX, kslice, stages, KB, ksplit);
  if (smem > 220 * 1024) return R4DXB_TOO_LARGE;
  auto kern = TrellisGemvMmaKernel<KB, TMAX, PRO, kTp>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ksplit, a.N / 128, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = ksplit;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_use_pdl ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, a, tp);
  ++g_launch_count;
  return static_cast<int>(e);
}

template <int KB, int PRO, bool kTp>
int LaunchT(const MmaArgs& a, int ksplit, cudaStream_t stream, const TpPush& tp) {
  if (a.T == 1) return Launch<KB, 1, PRO, kTp>(a, ksplit, stream, tp);
  if (a.T == 2) return Launch<KB, 2, PRO, kTp>(a, ksplit, stream, tp);
  if (a.T <= 4) return Launch<KB, 4, PRO, kTp>(a, ksplit, stream, tp);
  return Launch<KB, 8, PRO, kTp>(a, ksplit, stream, tp);
}

template <bool kTp>
int LaunchAll(const MmaArgs& a, int kb, int prologue, int ksplit, cudaStream_t s, const TpPush& tp) {
#define R4DXB_CASE(KBV, PROV) \
  if (kb == KBV && prologue == PROV) return LaunchT<KBV, PROV, kTp>(a, ksplit, s, tp);
  R4DXB_CASE(3, 0) R4DXB_CASE(3, 1) R4DXB_CASE(3, 2)
  R4DXB_CASE(4, 0) R4DXB_CASE(4, 1) R4DXB_CASE(4, 2)
  R4DXB_CASE(5, 0) R4DXB_CASE(5, 1) R4DXB_CASE(5, 2)
#undef R4DXB_CASE
  return R4DXB_BAD_ARG;
}

int CheckArgs(int T, int N, int K, int ksplit) {
  if (T < 1 || T > 8 || N % 128 || K % 128) return R4DXB_BAD_ARG;
  if (ksplit != 1 && ksplit != 2 && ksplit != 4 && ksplit != 8) return R4DXB_BAD_ARG;
  if ((K / 128) % ksplit) return R4DXB_BAD_ARG;
  if (K / ksplit > 6144) return R4DXB_TOO_LARGE;       // the activation slice (16 bytes per k) must fit beside the weight ring
  return 0;
}

}  // namespace
}  // namespace r4dxb

using namespace r4dxb;

extern "C" {

// Same contract as r4dxb_trellis_gemv_ex, on the tensor-memory path.  `status`: device word that receives
// 500 + role code if a bounded wait inside a CTA ran out (may be null).
int r4dxb_trellis_gemv_mma(const void* words, const void* suh, const void* svh, const void* x, void* y,
                           const void* residual, const void* norm_w, float eps, int prologue, int T, int N, int K, int kb,
                           int ksplit, int* status, void* stream) {
  if (int rc = CheckArgs(T, N, K, ksplit)) return rc;
  if (prologue == 1 && (norm_w == nullptr || K % 8)) return R4DXB_BAD_ARG;
  MmaArgs a = {};
  a.words = static_cast<const uint32_t*>(words);
  a.suh = static_cast<const __half*>(suh);
  a.svh = static_cast<const __half*>(svh);
  a.x = static_cast<const __nv_bfloat16*>(x);
  a.y = static_cast<__nv_bfloat16*>(y);
  a.residual = static_cast<const __nv_bfloat16*>(residual);
  a.norm_w = static_cast<const __nv_bfloat16*>(norm_w);
  a.eps = eps;
  a.T = T; a.N = N; a.K = K;
  a.status = status;
  if (prologue == 3) { prologue = 2; a.act = 1; }      // GeGLU: the gated prologue with a tanh-GELU gate
  TpPush none = {};
  return LaunchAll<false>(a, kb, prologue, ksplit, static_cast<cudaStream_t>(stream), none);
}

// Row-parallel product + all-reduce + residual in one kernel on the tensor-memory path; the collective's
// arguments are those of r4dxb_trellis_gemv_allreduce (the wait status of the collective is `tp_status`).
int r4dxb_trellis_gemv_mma_allreduce(const void* words, const void* suh, const void* svh, const void* x, void* y,
                                     const void* residual, int prologue, int T, int N, int K, int kb, int ksplit,
                                     void* const* recv, void* block_seq, int* tp_status, int world, int rank,
                                     int spin_limit, int* status, void* stream) {
  if (int rc = CheckArgs(T, N, K, ksplit)) return rc;
  if (world < 2 || world > kMaxWorld || rank < 0 || rank >= world || prologue == 1) return R4DXB_BAD_ARG;
  MmaArgs a = {};
  a.words = static_cast<const uint32_t*>(words);
  a.suh = static_cast<const __half*>(suh);
  a.svh = static_cast<const __half*>(svh);
  a.x = static_cast<const __nv_bfloat16*>(x);
  a.y = static_cast<__nv_bfloat16*>(y);
  a.residual = static_cast<const __nv_bfloat16*>(residual);
  a.T = T; a.N = N; a.K = K;
  a.status = status;
  if (prologue == 3) { prologue = 2; a.act = 1; }
  TpPush tp = {};
  for (int p = 0; p < world; ++p) tp.recv[p] = static_cast<float2*>(recv[p]);
  tp.block_seq = static_cast<unsigned*>(block_seq);
  tp.status = tp_status;
  tp.world = world;
  tp.rank = rank;
  tp.spin_limit = spin_limit;
  return LaunchAll<true>(a, kb, prologue, ksplit, static_cast<cudaStream_t>(stream), tp);
}

}  // extern "C"
