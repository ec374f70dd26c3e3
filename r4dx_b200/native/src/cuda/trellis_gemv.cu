// Trellis-decode weight-streaming GEMM for T <= 8 activation rows (decode and speculative verify).
//
//   y[t, n] = bf16( svh[n] * H128( sum_k Q[n, k] * xh[t, k] )[n] (+ residual[t, n]) )
//   xh = fp16( H128(suh (.) act(x)) )
//
// One CTA owns a 128-row block of N (the span of one output Hadamard) and a K slice; `ksplit` CTAs of
// one thread-block cluster share a row block and are reduced through distributed shared memory in
// rank order (deterministic, no atomics, no global scratch).
//
// Weight stream: a producer warp moves the CTA's packed words global -> shared with bulk async
// copies (one 128-K stage = 8 k-tiles x 8 n-tiles, a single contiguous run thanks to the
// [N/128][K/16][8][words] order) through a ring of mbarrier-guarded stages, so the whole slice of a
// small matrix is in flight at once and a large one keeps tens of KB per SM in flight without
// spending registers.  Eight consumer warps (warp j = n-tile j) decode from shared memory: every
// lane turns 8 consecutive K codes of one row into fp16 and multiplies them with the staged
// activations.
//
// Programmatic dependent launch hides launch and prefetch latency: the kernel lets its successor
// start early and itself waits for its predecessor (griddepcontrol.wait) only before touching
// activations -- the weight stream, which depends on no other kernel, is already in flight by then.
//
// Prologue modes fold the producer of the activations into this kernel:
//   0  x is the activation                       [T, K]
//   1  x is the residual stream, act = RMSNorm   x * rsqrt(mean x^2 + eps) * (1 + w), rounded to bf16
//   2  x is fused [gate | up] rows [T, 2K], act = bf16(silu(gate) * up)
// so a decoder layer needs no separate norm / SwiGLU launches.
//
// The tensor-parallel variant finishes a row-parallel linear with the all-reduce inside the kernel
// (see TpPush).  The reference engine uses an input-transform kernel + a WMMA GEMM with a ticket-based
// split-K finish + a host-mailbox all-reduce kernel for the same job
// (reference: third_party/libr4d/r4d_gemm_trellis_nt_m64.hip:30-90,216; src/kernels/src/r4dx_tp_kernels.hip:235-311).
#include <cooperative_groups.h>

#include "sm100_ptx.cuh"
#include "tp_push.cuh"
#include "trellis_decode.cuh"

namespace cg = cooperative_groups;

namespace r4dxb {

bool g_use_pdl = true;       // shared with the small decode kernels (common.cuh: LaunchPdl)

namespace {

constexpr int kConsumerWarps = 8;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
struct GemvArgs {
  const uint32_t* words;
  const __half* suh;
  const __half* svh;
  const __nv_bfloat16* x;
  __nv_bfloat16* y;
  const __nv_bfloat16* residual;
  const __nv_bfloat16* norm_w;     // prologue mode 1
  float eps;
  int T, N, K, kblocks_per_cta, stages;
  // grouped (mixture-of-experts) mode: blockIdx.z = local expert; the expert's rows come from a
  // device-side plan, so no routing decision is ever read back by the host
  const int* g_offsets;            // [experts + 1] into g_perm
  const int* g_perm;               // pair indices sorted by expert; output row = pair
  int g_in_div;                    // input row = pair / g_in_div (top-k pairs share a token row) or pair (1)
  int g_pass;                      // which group of TMAX rows of each expert this launch handles
  // expert-parallel input (optional): rows arrive from peers; g_seq = device call counter (this call is
  // *g_seq + 1, its parity selects the buffer half), g_ready[par][row] == call number once a row landed
  const unsigned* g_seq;
  const unsigned* g_ready;
  long long g_x_par_stride;        // elements between the two halves of x
  long long g_ready_par_stride;
  int g_spin_limit;
  int* g_status;
  long long g_words_stride;        // words between consecutive experts
  // compact grid (optional): blockIdx.z runs over the call's (row, slot) pairs instead of every local expert; the CTAs of
  // the first pair in an expert's list run that expert, the others leave.  A decode step touches 10 of 512 experts: the
  // full grid spent most of the kernel's time launching CTAs that return at once.
  const int* g_pair_ids;           // [pairs] global expert id of each pair (the router's output)
  int g_e_begin, g_experts;
  int act;                         // gate activation of the fused gated-MLP prologue (GateAct)
  // sibling mode: up to kMaxSiblings weights that read the same activations through the same prologue (q / k / v,
  // the GDN qkv / z pair) share one launch; blockIdx.y runs over the row blocks of all of them back to back
  int nsib;
  struct Sibling {
    const uint32_t* words;
    const __half* suh;
    const __half* svh;
    __nv_bfloat16* y;
    int N, nb_end;                 // row blocks [previous nb_end, nb_end) belong to this sibling
  } sib[3];
};
constexpr int kMaxSiblings = 3;

template <int KB, int TMAX, int PRO, bool kTp, bool kGrouped = false>
__global__ void __launch_bounds__(kThreads)
TrellisGemvKernel(GemvArgs a, TpPush tp) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  cg::cluster_group cluster = cg::this_cluster();
  const int ksplit = gridDim.x;
  const int krank = blockIdx.x;            // == rank inside the cluster
  int nb = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // the weight this CTA serves: the launch's only one, or one of the siblings (kernel parameters stay read-only)
  const uint32_t* w_words = a.words;
  const __half* w_suh = a.suh;
  const __half* w_svh = a.svh;
  __nv_bfloat16* w_y = a.y;
  int N = a.N;
  if (!kGrouped && !kTp && a.nsib > 0) {
    int sidx = 0;
    while (sidx + 1 < a.nsib && nb >= a.sib[sidx].nb_end) ++sidx;
    if (sidx > 0) nb -= a.sib[sidx - 1].nb_end;
    w_words = a.sib[sidx].words; w_suh = a.sib[sidx].suh; w_svh = a.sib[sidx].svh; w_y = a.sib[sidx].y; N = a.sib[sidx].N;
  }
  // K blocks are dealt out as evenly as the count allows (17 blocks over 4 CTAs: 4, 4, 4, 5); shared memory is laid
  // out for the longest slice
  const int kslice = a.kblocks_per_cta * 128;
  const int kblocks_total = a.K / 128;
  const int kb_lo = krank * kblocks_total / ksplit;
  const int my_blocks = (krank + 1) * kblocks_total / ksplit - kb_lo;
  const int k_begin = kb_lo * 128;
  int T = a.T;
  const int K = a.K;
  int g_base = 0;
  if constexpr (kGrouped) {
    // this launch handles rows [g_pass * TMAX, +TMAX) of every expert's list
    int e = blockIdx.z;
    if (a.g_pair_ids != nullptr) {
      e = a.g_pair_ids[blockIdx.z] - a.g_e_begin;
      if (e < 0 || e >= a.g_experts) return;                                   // (uniform over the cluster, like the exit below)
      if (a.g_perm[a.g_offsets[e]] != static_cast<int>(blockIdx.z)) return;   // not the first pair of its expert
    }
    g_base = a.g_offsets[e] + a.g_pass * TMAX;
    const int left = a.g_offsets[e + 1] - g_base;
    if (left <= 0) return;         // uniform over the cluster: every CTA of it leaves before any barrier
    T = left < TMAX ? left : TMAX;
    if (a.g_seq != nullptr) {
      const unsigned call = *a.g_seq + 1;
      a.x += static_cast<size_t>(call & 1) * a.g_x_par_stride;
      if (a.g_ready != nullptr) a.g_ready += static_cast<size_t>(call & 1) * a.g_ready_par_stride;
    }
    w_words += static_cast<size_t>(e) * a.g_words_stride;
    w_suh += static_cast<size_t>(e) * K;
    w_svh += static_cast<size_t>(e) * N;
  }
  constexpr int NW = 8 * KB;
  constexpr int kStageBytes = 8 * 8 * NW * 4;     // 8 k-tiles x 8 n-tiles
  auto in_row = [&](int t) -> size_t {
    if constexpr (kGrouped) return static_cast<size_t>(a.g_perm[g_base + t] / a.g_in_div);
    else return static_cast<size_t>(t);
  };
  auto out_row = [&](int t) -> size_t {
    if constexpr (kGrouped) return static_cast<size_t>(a.g_perm[g_base + t]);
    else return static_cast<size_t>(t);
  };

  float* part = reinterpret_cast<float*>(smem_raw);                                  // [ksplit][TMAX][128] (used on cluster rank 0)
  float* rnorm = part + ksplit * TMAX * 128;                                          // [8] per-row rsqrt
  uint64_t* full = reinterpret_cast<uint64_t*>(rnorm + 8);                            // [8]
  uint64_t* empty = full + 8;                                                         // [8]
  uint64_t* red_bar = empty + 8;                                                      // [1] split-K partials have landed
  volatile int* abort_flag = reinterpret_cast<volatile int*>(red_bar + 1);
  __half* xs = reinterpret_cast<__half*>(smem_raw + ksplit * TMAX * 128 * 4 + 32 + 128 + 16);   // [TMAX][kslice]
  unsigned char* wst = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(xs + static_cast<size_t>(TMAX) * kslice) + 127) & ~uintptr_t(127));   // [stages][kStageBytes]

  if (threadIdx.x == 0) {
    for (int s = 0; s < a.stages; ++s) {
      ptx::MbarInit(&full[s], 1);
      ptx::MbarInit(&empty[s], kConsumerWarps);
    }
    ptx::MbarInit(red_bar, ksplit * kConsumerWarps);
    *abort_flag = 0;
    ptx::MbarFenceInit();
  }
  __syncthreads();
  // Cluster rendezvous, split in two: arrive now, wait only just before the first remote write, so
  // the weight stream and the prologue overlap with it.  It guarantees that rank 0's reduction
  // barrier is initialised before any peer CTA touches it.
  if (ksplit > 1) asm volatile("barrier.cluster.arrive.release;" ::: "memory");
  // let the next kernel in the stream begin its own launch and weight prefetch
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == kConsumerWarps) {
    // ---------------- producer: stream this CTA's words through the stage ring ----------------
    if (lane == 0) {
      const unsigned char* src = reinterpret_cast<const unsigned char*>(w_words) +
                                 (static_cast<size_t>(nb) * (K / 128) + static_cast<size_t>(kb_lo)) * kStageBytes;
      int s = 0;
      uint32_t phase = 1;          // parity to wait for on the "empty" barrier of stage s (fresh barriers pass parity 1)
      for (int it = 0; it < my_blocks; ++it) {
        if (!ptx::MbarWait(&empty[s], phase, abort_flag, 1)) break;
        ptx::MbarArriveExpectTx(&full[s], kStageBytes);
        ptx::BulkLoad(wst + static_cast<size_t>(s) * kStageBytes, src + static_cast<size_t>(it) * kStageBytes, kStageBytes, &full[s]);
        if (++s == a.stages) { s = 0; phase ^= 1u; }
      }
    }
  } else {
    // ---------------- prologue (consumer warps): xs = fp16(H128(suh * act(x))) for this K slice ----------------
    // everything before this point touched only weights; activations come from the previous kernel
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if constexpr (kGrouped) {
      if (a.g_ready != nullptr) {
        // rows are stored by peer GPUs: wait (bounded) for the flag of every row this launch reads
        const unsigned call = *a.g_seq + 1;
        if (warp < T && lane == 0) {
          const unsigned* f = a.g_ready + in_row(warp);
          bool got = TpStatusNow(a.g_status) != 0;       // sticky: after one timeout nobody waits again
          for (int i = 0; i < a.g_spin_limit && !got; ++i) {
            unsigned v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
            if (v == call) { got = true; break; }
            if (i > 64) __nanosleep(32);
          }
          if (!got) atomicCAS(a.g_status, 0, 400 + static_cast<int>(in_row(warp) % 1000));
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
      }
    }
    if constexpr (PRO == 1) {
      // RMSNorm statistics need the whole row, not just this CTA's slice.  All eight consumer warps share every
      // row (an eighth of K each) so that the reduction is a couple of loads deep instead of K / 256.
      float* part_ss = part;              // [TMAX][8] partial sums; the split-K partials that live here come much later
      const int kw = (K / 8 + 7) & ~7;    // columns per warp, a multiple of 8
      const int k_lo = warp * kw, k_hi = min(K, k_lo + kw);
#pragma unroll
      for (int t = 0; t < TMAX; ++t) {
        float ss = 0.f;
        if (t < T) {
          const __nv_bfloat16* row = a.x + in_row(t) * K;
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
        rnorm[threadIdx.x] = rsqrtf(ss / K + a.eps);
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");
    }
    const float inv_sqrt = 0.08838834764831845f;   // 1 / sqrt(128)
    for (int item = warp; item < my_blocks * TMAX; item += kConsumerWarps) {
      const int t = item / my_blocks, b = item % my_blocks;
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      const int k = k_begin + b * 128 + lane * 4;
      if (t < T) {
        if constexpr (PRO == 2) {
          const uint2 g = *reinterpret_cast<const uint2*>(a.x + in_row(t) * 2 * K + k);
          const uint2 u = *reinterpret_cast<const uint2*>(a.x + in_row(t) * 2 * K + K + k);
          const uint32_t p01 = PackBf16(GateAct(BfLo(g.x), a.act) * BfLo(u.x), GateAct(BfHi(g.x), a.act) * BfHi(u.x));
          const uint32_t p23 = PackBf16(GateAct(BfLo(g.y), a.act) * BfLo(u.y), GateAct(BfHi(g.y), a.act) * BfHi(u.y));
          v[0] = BfLo(p01); v[1] = BfHi(p01); v[2] = BfLo(p23); v[3] = BfHi(p23);
        } else {
          // (peer-written rows must not come from a stale L1 line)
          const uint2 xv = kGrouped ? __ldcg(reinterpret_cast<const uint2*>(a.x + in_row(t) * K + k))
                                    : *reinterpret_cast<const uint2*>(a.x + in_row(t) * K + k);
          v[0] = BfLo(xv.x); v[1] = BfHi(xv.x); v[2] = BfLo(xv.y); v[3] = BfHi(xv.y);
          if constexpr (PRO == 1) {
            const uint2 wv = *reinterpret_cast<const uint2*>(a.norm_w + k);
            const float r = rnorm[t];
            // same rounding point as the standalone norm kernel: the normalised row is a bf16 tensor
            const uint32_t p01 = PackBf16(v[0] * r * (1.f + BfLo(wv.x)), v[1] * r * (1.f + BfHi(wv.x)));
            const uint32_t p23 = PackBf16(v[2] * r * (1.f + BfLo(wv.y)), v[3] * r * (1.f + BfHi(wv.y)));
            v[0] = BfLo(p01); v[1] = BfHi(p01); v[2] = BfLo(p23); v[3] = BfHi(p23);
          }
        }
        const uint2 sv = *reinterpret_cast<const uint2*>(w_suh + k);
        const __half2 s01 = *reinterpret_cast<const __half2*>(&sv.x), s23 = *reinterpret_cast<const __half2*>(&sv.y);
        v[0] *= __low2float(s01); v[1] *= __high2float(s01); v[2] *= __low2float(s23); v[3] *= __high2float(s23);
      }
      WarpFwht128(v);
      __half2 o01 = __floats2half2_rn(v[0] * inv_sqrt, v[1] * inv_sqrt);
      __half2 o23 = __floats2half2_rn(v[2] * inv_sqrt, v[3] * inv_sqrt);
      uint2 ov;
      ov.x = *reinterpret_cast<uint32_t*>(&o01);
      ov.y = *reinterpret_cast<uint32_t*>(&o23);
      *reinterpret_cast<uint2*>(xs + static_cast<size_t>(t) * kslice + b * 128 + lane * 4) = ov;
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");

    // ---------------- main loop: warp = n-tile, lane = (row, k half) ----------------
    TrellisLane<KB> tl;
    tl.Init(lane);
    float acc[TMAX];
#pragma unroll
    for (int t = 0; t < TMAX; ++t) acc[t] = 0.f;
    const int khalf = (lane & 1) * 8;
    bool ok = true;
    // stage index and barrier parity advance by counting: a division by the run-time ring depth per 128-wide
    // K block would cost as much as decoding a dozen weights
    int s = 0;
    uint32_t phase = 0;
    for (int it = 0; it < my_blocks && ok; ++it) {
      ok = ptx::MbarWait(&full[s], phase, abort_flag, 2);
      if (!ok) break;
      const uint32_t* sw = reinterpret_cast<const uint32_t*>(wst + static_cast<size_t>(s) * kStageBytes) + warp * NW;
      __half2 hacc[TMAX];
#pragma unroll
      for (int t = 0; t < TMAX; ++t) hacc[t] = __float2half2_rn(0.f);
#pragma unroll
      for (int kt = 0; kt < 8; ++kt) {
        const uint32_t* tw = sw + kt * 8 * NW;
        uint32_t hi, lo;
        tl.Window(tw[tl.i0], tw[tl.i1], (KB == 4) ? 0u : tw[tl.i2], hi, lo);
        __half2 w[4];
        TrellisDecode8<KB>(hi, lo, w);
        const int kk = it * 128 + kt * 16 + khalf;
#pragma unroll
        for (int t = 0; t < TMAX; ++t) {
          // grouped launches are compiled for the widest expert but most experts hold one or two rows:
          // skip the rows this CTA does not have (T is uniform over the CTA)
          if (kGrouped && TMAX > 2 && t >= T) break;
          const uint4 xv = *reinterpret_cast<const uint4*>(xs + static_cast<size_t>(t) * kslice + kk);
          __half2 h = __hfma2(w[0], *reinterpret_cast<const __half2*>(&xv.x), hacc[t]);
          h = __hfma2(w[1], *reinterpret_cast<const __half2*>(&xv.y), h);
          h = __hfma2(w[2], *reinterpret_cast<const __half2*>(&xv.z), h);
          hacc[t] = __hfma2(w[3], *reinterpret_cast<const __half2*>(&xv.w), h);
        }
        if (kt == 3 || kt == 7) {       // fold the fp16 partials into fp32 every 32 products per half
#pragma unroll
          for (int t = 0; t < TMAX; ++t) {
            acc[t] += __low2float(hacc[t]) + __high2float(hacc[t]);
            hacc[t] = __float2half2_rn(0.f);
          }
        }
      }
      __syncwarp();
      if (lane == 0) ptx::MbarArrive(&empty[s]);
      if (++s == a.stages) { s = 0; phase ^= 1u; }
    }
    // hand the partial rows to cluster rank 0: distributed-shared-memory stores + one remote
    // mbarrier arrival per warp; only rank 0 waits, the other CTAs are done
    __syncwarp();
    if (ksplit > 1) asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
    float* dst = ksplit > 1 ? cluster.map_shared_rank(part, 0) : part;
    dst += krank * TMAX * 128;
#pragma unroll
    for (int t = 0; t < TMAX; ++t) {
      acc[t] += __shfl_xor_sync(0xffffffffu, acc[t], 1);
      if ((lane & 1) == 0) dst[t * 128 + warp * 16 + (lane >> 1)] = acc[t];
    }
    __syncwarp();
    if (lane == 0) {
      uint32_t remote_bar;
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_bar) : "r"(ptx::SmemAddr(red_bar)), "r"(0));
      asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar) : "memory");
    }
  }
  if (warp == kConsumerWarps) {
    // lane 0 may still be feeding the ring while the other lanes are already here: reconverge first,
    // and use the per-thread (non-.aligned) form of the barrier
    __syncwarp();
    if (ksplit > 1) asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
  }

  // ---------------- epilogue (cluster rank 0) ----------------
  if (krank == 0 && warp < kConsumerWarps) {
    {
      // wait (bounded) until every consumer warp of every CTA of the cluster has delivered its partial rows
      bool landed = false;
      for (int i = 0; i < ptx::kSpinLimit && !landed; ++i) {
        uint32_t okw;
        asm volatile(
            "{ .reg .pred p; mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
            : "=r"(okw) : "r"(ptx::SmemAddr(red_bar)), "r"(0) : "memory");
        landed = okw != 0;
      }
      // a split-K hand-off that never completes leaves a code in whichever status word this launch was given
      if (!landed && lane == 0) {
        if constexpr (kTp) atomicCAS(tp.status, 0, 390);
        if constexpr (kGrouped) { if (a.g_status != nullptr) atomicCAS(a.g_status, 0, 390); }
      }
    }
    const float inv_sqrt = 0.08838834764831845f;
    float o[4] = {0.f, 0.f, 0.f, 0.f};
    const int t = warp;              // warp t finishes row t (T <= 8 = consumer warps)
    const int n = nb * 128 + lane * 4;
    if (t < T) {
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      for (int r = 0; r < ksplit; ++r) {       // fixed order: the result does not depend on timing
        const float4 p = *reinterpret_cast<const float4*>(part + (r * TMAX + t) * 128 + lane * 4);
        v[0] += p.x; v[1] += p.y; v[2] += p.z; v[3] += p.w;
      }
      WarpFwht128(v);
      const uint2 sv = *reinterpret_cast<const uint2*>(w_svh + n);
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
        const uint2 rv = *reinterpret_cast<const uint2*>(a.residual + out_row(t) * N + n);
        o[0] += BfLo(rv.x); o[1] += BfHi(rv.x); o[2] += BfLo(rv.y); o[3] += BfHi(rv.y);
      }
      uint2 ov;
      ov.x = PackBf16(o[0], o[1]);
      ov.y = PackBf16(o[2], o[3]);
      if constexpr (kGrouped) {
        if (tp.ep_P > 0) {
          const unsigned call = *a.g_seq + 1;
          const size_t gp = out_row(t);
          const int dest = static_cast<int>(gp / tp.ep_P);
          const size_t slot = static_cast<size_t>(call & 1) * tp.ep_P + gp % tp.ep_P;
          *reinterpret_cast<uint2*>(tp.ep_y[dest] + slot * N + n) = ov;
          __threadfence_system();
          __syncwarp();
          if (lane == 0) atomicAdd_system(tp.ep_cnt[dest] + slot, 1u);
        } else {
          *reinterpret_cast<uint2*>(w_y + out_row(t) * N + n) = ov;
        }
      } else {
        *reinterpret_cast<uint2*>(w_y + out_row(t) * N + n) = ov;
      }
    }
  }
}

size_t SmemBytes(int tmax, int kslice, int stages, int kb, int ksplit) {
  return static_cast<size_t>(ksplit) * tmax * 128 * 4 + 32 + 128 + 16 + static_cast<size_t>(tmax) * kslice * 2 + 128 +
         static_cast<size_t>(stages) * 8 * 8 * 8 * kb * 4;
}

template <int KB, int TMAX, int PRO, bool kTp>
int Launch(GemvArgs a, int ksplit, cudaStream_t stream, const TpPush& tp) {
  a.kblocks_per_cta = (a.K / 128 + ksplit - 1) / ksplit;       // the longest slice
  const int kslice = a.kblocks_per_cta * 128;
  // ring depth: everything in flight for short slices, otherwise up to 6 stages (48-60 KiB)
  a.stages = a.kblocks_per_cta < 6 ? a.kblocks_per_cta : 6;
  const size_t smem = SmemBytes(TMAX, kslice, a.stages, KB, ksplit);
  if (smem > 220 * 1024) return R4DXB_TOO_LARGE;
  auto kern = TrellisGemvKernel<KB, TMAX, PRO, kTp>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ksplit, a.nsib > 0 ? a.sib[a.nsib - 1].nb_end : a.N / 128, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = ksplit;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  // programmatic dependent launch: this kernel may start while its predecessor drains (it waits
  // on-device before reading activations)
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_use_pdl ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, a, tp);
  ++g_launch_count;
  return static_cast<int>(e);
}

template <int KB, int TMAX, int PRO>
int LaunchGrouped(GemvArgs a, int ksplit, int experts, cudaStream_t stream, const TpPush& ep) {
  a.kblocks_per_cta = (a.K / 128 + ksplit - 1) / ksplit;
  const int kslice = a.kblocks_per_cta * 128;
  a.stages = a.kblocks_per_cta < 6 ? a.kblocks_per_cta : 6;
  const size_t smem = SmemBytes(TMAX, kslice, a.stages, KB, ksplit);
  if (smem > 220 * 1024) return R4DXB_TOO_LARGE;
  auto kern = TrellisGemvKernel<KB, TMAX, PRO, false, true>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ksplit, a.N / 128, experts);       // (experts = the pair count when the grid is compact)
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
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, a, ep);
  ++g_launch_count;
  return static_cast<int>(e);
}

template <int KB, int PRO, bool kTp>
int LaunchT(const GemvArgs& a, int ksplit, cudaStream_t stream, const TpPush& tp) {
  if (a.T == 1) return Launch<KB, 1, PRO, kTp>(a, ksplit, stream, tp);
  if (a.T == 2) return Launch<KB, 2, PRO, kTp>(a, ksplit, stream, tp);
  if (a.T <= 4) return Launch<KB, 4, PRO, kTp>(a, ksplit, stream, tp);
  return Launch<KB, 8, PRO, kTp>(a, ksplit, stream, tp);
}

template <bool kTp>
int LaunchAll(const GemvArgs& a, int kb, int prologue, int ksplit, cudaStream_t s, const TpPush& tp) {
#define R4DXB_CASE(KBV, PROV) \
  if (kb == KBV && prologue == PROV) return LaunchT<KBV, PROV, kTp>(a, ksplit, s, tp);
  R4DXB_CASE(3, 0) R4DXB_CASE(3, 1) R4DXB_CASE(3, 2)
  R4DXB_CASE(4, 0) R4DXB_CASE(4, 1) R4DXB_CASE(4, 2)
  R4DXB_CASE(5, 0) R4DXB_CASE(5, 1) R4DXB_CASE(5, 2)
#undef R4DXB_CASE
  return R4DXB_BAD_ARG;
}

GemvArgs MakeArgs(const void* words, const void* suh, const void* svh, const void* x, void* y, const void* residual,
                  const void* norm_w, float eps, int T, int N, int K) {
  GemvArgs a = {};
  a.words = static_cast<const uint32_t*>(words);
  a.suh = static_cast<const __half*>(suh);
  a.svh = static_cast<const __half*>(svh);
  a.x = static_cast<const __nv_bfloat16*>(x);
  a.y = static_cast<__nv_bfloat16*>(y);
  a.residual = static_cast<const __nv_bfloat16*>(residual);
  a.norm_w = static_cast<const __nv_bfloat16*>(norm_w);
  a.eps = eps;
  a.T = T; a.N = N; a.K = K;
  a.g_in_div = 1;
  return a;
}

int CheckArgs(int T, int N, int K, int ksplit) {
  if (T < 1 || T > 8 || N % 128 || K % 128) return R4DXB_BAD_ARG;
  if (ksplit != 1 && ksplit != 2 && ksplit != 4 && ksplit != 8) return R4DXB_BAD_ARG;
  if (K / 128 < ksplit) return R4DXB_BAD_ARG;       // every CTA of the cluster needs at least one K block
  return 0;
}

}  // namespace
}  // namespace r4dxb

using namespace r4dxb;

extern "C" {

/* A/B switch for programmatic dependent launch (default on). */
void r4dxb_set_pdl(int on) { g_use_pdl = on != 0; }

int r4dxb_trellis_gemv_ex(const void* words, const void* suh, const void* svh, const void* x, void* y,
                          const void* residual, const void* norm_w, float eps, int prologue, int T, int N, int K, int kb,
                          int ksplit, void* stream) {
  if (int rc = CheckArgs(T, N, K, ksplit)) return rc;
  if (prologue == 1 && (norm_w == nullptr || K % 8)) return R4DXB_BAD_ARG;
  GemvArgs a = MakeArgs(words, suh, svh, x, y, residual, norm_w, eps, T, N, K);
  if (prologue == 3) { prologue = 2; a.act = 1; }      // GeGLU: the SwiGLU prologue with a tanh-GELU gate
  TpPush none = {};
  return LaunchAll<false>(a, kb, prologue, ksplit, static_cast<cudaStream_t>(stream), none);
}

/* Sibling projections in one launch: `count` (2 or 3) trellis weights of the same K and bit width that read the same
 * rows x through the same prologue; weight i writes y[i] [T, n[i]].  No residual, no all-reduce. */
int r4dxb_trellis_gemv_siblings(int count, const void* const* words, const void* const* suh, const void* const* svh,
                                void* const* y, const int* n, const void* x, const void* norm_w, float eps, int prologue, int T,
                                int K, int kb, int ksplit, void* stream) {
  if (count < 2 || count > kMaxSiblings) return R4DXB_BAD_ARG;
  for (int i = 0; i < count; ++i)
    if (int rc = CheckArgs(T, n[i], K, ksplit)) return rc;
  if (prologue == 1 && (norm_w == nullptr || K % 8)) return R4DXB_BAD_ARG;
  GemvArgs a = MakeArgs(words[0], suh[0], svh[0], x, y[0], nullptr, norm_w, eps, T, n[0], K);
  if (prologue == 3) { prologue = 2; a.act = 1; }
  a.nsib = count;
  int end = 0;
  for (int i = 0; i < count; ++i) {
    end += n[i] / 128;
    a.sib[i].words = static_cast<const uint32_t*>(words[i]);
    a.sib[i].suh = static_cast<const __half*>(suh[i]);
    a.sib[i].svh = static_cast<const __half*>(svh[i]);
    a.sib[i].y = static_cast<__nv_bfloat16*>(y[i]);
    a.sib[i].N = n[i];
    a.sib[i].nb_end = end;
  }
  TpPush none = {};
  return LaunchAll<false>(a, kb, prologue, ksplit, static_cast<cudaStream_t>(stream), none);
}

int r4dxb_trellis_gemv(const void* words, const void* suh, const void* svh, const void* x, void* y,
                       const void* residual, int T, int N, int K, int kb, int ksplit, void* stream) {
  return r4dxb_trellis_gemv_ex(words, suh, svh, x, y, residual, nullptr, 0.f, 0, T, N, K, kb, ksplit, stream);
}

// Grouped expert linear: one launch covers every local expert (grid.z); expert e multiplies the rows
// perm[offsets[e] + pass*tmax ...] (at most tmax of them) by its own weights.  words / suh / svh hold
// the experts back to back.  Input row of a pair = pair / in_div; output row = pair.  prologue 0 or 2.
int r4dxb_trellis_gemv_grouped_ep(const void* words, const void* suh, const void* svh, const void* x, void* y,
                                  const int* offsets, const int* perm, int in_div, int pass, int tmax, int prologue,
                                  int experts, int N, int K, int kb, int ksplit,
                                  const void* seq_ptr, const void* ready, long long x_par_stride, long long ready_par_stride,
                                  void* const* ep_y, void* const* ep_cnt, int ep_P, int world, int spin_limit, int* status,
                                  void* stream) {
  if (int rc = CheckArgs(1, N, K, ksplit)) return rc;
  if (experts < 1 || experts > 65535 || in_div < 1 || (prologue != 0 && prologue != 2) || world > kMaxWorld) return R4DXB_BAD_ARG;
  GemvArgs a = MakeArgs(words, suh, svh, x, y, nullptr, nullptr, 0.f, tmax, N, K);
  a.g_offsets = offsets;
  a.g_perm = perm;
  a.g_in_div = in_div;
  a.g_pass = pass;
  a.g_words_stride = static_cast<long long>(N / 16) * (K / 16) * 8 * kb;
  a.g_seq = static_cast<const unsigned*>(seq_ptr);
  a.g_ready = static_cast<const unsigned*>(ready);
  a.g_x_par_stride = x_par_stride;
  a.g_ready_par_stride = ready_par_stride;
  a.g_spin_limit = spin_limit;
  a.g_status = status;
  TpPush ep = {};
  if (ep_y != nullptr) {
    for (int p = 0; p < world; ++p) {
      ep.ep_y[p] = static_cast<__nv_bfloat16*>(ep_y[p]);
      ep.ep_cnt[p] = static_cast<unsigned*>(ep_cnt[p]);
    }
    ep.ep_P = ep_P;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define R4DXB_G(KBV, TM, PROV) \
  if (kb == KBV && tmax == TM && prologue == PROV) return LaunchGrouped<KBV, TM, PROV>(a, ksplit, experts, s, ep);
  R4DXB_G(3, 2, 0) R4DXB_G(3, 2, 2) R4DXB_G(3, 8, 0) R4DXB_G(3, 8, 2)
  R4DXB_G(4, 2, 0) R4DXB_G(4, 2, 2) R4DXB_G(4, 8, 0) R4DXB_G(4, 8, 2)
  R4DXB_G(5, 2, 0) R4DXB_G(5, 2, 2) R4DXB_G(5, 8, 0) R4DXB_G(5, 8, 2)
#undef R4DXB_G
  return R4DXB_BAD_ARG;
}

/* The grouped product over a compact grid: pair_ids [pairs] are the routed expert ids of the call's (row, slot) pairs;
 * only experts that some pair names get CTAs (a decode step: 10 of 512).  Same results as the full grid. */
int r4dxb_trellis_gemv_grouped_pairs(const void* words, const void* suh, const void* svh, const void* x, void* y,
                                     const int* offsets, const int* perm, const int* pair_ids, int pairs, int e_begin,
                                     int in_div, int pass, int tmax, int prologue, int experts, int N, int K, int kb, int ksplit,
                                     void* stream) {
  if (int rc = CheckArgs(1, N, K, ksplit)) return rc;
  if (experts < 1 || pairs < 1 || pairs > 65535 || in_div < 1 || (prologue != 0 && prologue != 2) || pair_ids == nullptr)
    return R4DXB_BAD_ARG;
  GemvArgs a = MakeArgs(words, suh, svh, x, y, nullptr, nullptr, 0.f, tmax, N, K);
  a.g_offsets = offsets;
  a.g_perm = perm;
  a.g_in_div = in_div;
  a.g_pass = pass;
  a.g_words_stride = static_cast<long long>(N / 16) * (K / 16) * 8 * kb;
  a.g_pair_ids = pair_ids;
  a.g_e_begin = e_begin;
  a.g_experts = experts;
  const TpPush ep = {};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define R4DXB_G(KBV, TM, PROV) \
  if (kb == KBV && tmax == TM && prologue == PROV) return LaunchGrouped<KBV, TM, PROV>(a, ksplit, pairs, s, ep);
  R4DXB_G(3, 2, 0) R4DXB_G(3, 2, 2) R4DXB_G(3, 8, 0) R4DXB_G(3, 8, 2)
  R4DXB_G(4, 2, 0) R4DXB_G(4, 2, 2) R4DXB_G(4, 8, 0) R4DXB_G(4, 8, 2)
  R4DXB_G(5, 2, 0) R4DXB_G(5, 2, 2) R4DXB_G(5, 8, 0) R4DXB_G(5, 8, 2)
#undef R4DXB_G
  return R4DXB_BAD_ARG;
}

int r4dxb_trellis_gemv_grouped(const void* words, const void* suh, const void* svh, const void* x, void* y,
                               const int* offsets, const int* perm, int in_div, int pass, int tmax, int prologue,
                               int experts, int N, int K, int kb, int ksplit, void* stream) {
  return r4dxb_trellis_gemv_grouped_ep(words, suh, svh, x, y, offsets, perm, in_div, pass, tmax, prologue, experts, N, K, kb,
                                       ksplit, nullptr, nullptr, 0, 0, nullptr, nullptr, 0, 0, 0, nullptr, stream);
}

// Row-parallel linear + all-reduce + residual in one kernel (see TpPush).  recv: `world` peer-mapped
// pointers (index = rank), each [2][world][8][N] (value, seq) pairs, zero-initialised; block_seq
// ([N/128] u32, zero-initialised) and status: this rank's own memory.  spin_limit bounds every wait.
int r4dxb_trellis_gemv_allreduce(const void* words, const void* suh, const void* svh, const void* x, void* y,
                                 const void* residual, int prologue, int T, int N, int K, int kb, int ksplit,
                                 void* const* recv, void* block_seq, int* status, int world, int rank, int spin_limit,
                                 void* stream) {
  if (int rc = CheckArgs(T, N, K, ksplit)) return rc;
  if (world < 2 || world > kMaxWorld || rank < 0 || rank >= world || prologue == 1) return R4DXB_BAD_ARG;
  GemvArgs a = MakeArgs(words, suh, svh, x, y, residual, nullptr, 0.f, T, N, K);
  if (prologue == 3) { prologue = 2; a.act = 1; }
  TpPush tp = {};
  for (int p = 0; p < world; ++p) tp.recv[p] = static_cast<float2*>(recv[p]);
  tp.block_seq = static_cast<unsigned*>(block_seq);
  tp.status = status;
  tp.world = world;
  tp.rank = rank;
  tp.spin_limit = spin_limit;
  return LaunchAll<true>(a, kb, prologue, ksplit, static_cast<cudaStream_t>(stream), tp);
}

}  // extern "C"
