// Trellis-decode weight-streaming GEMM for T <= 8 activation rows (decode and speculative verify).
//
//   y[t, n] = bf16( svh[n] * H128( sum_k Q[n, k] * xh[t, k] )[n] ) (+ residual[t, n])
//   xh = fp16( H128(suh (.) x) )
//
// One CTA owns a 128-row block of N (the span of one output Hadamard) and a K slice; `ksplit`
// CTAs of one thread-block cluster share a row block and are reduced through distributed shared
// memory in rank order (deterministic, no atomics, no global scratch).  Warp j of the CTA streams
// n-tile j (16 rows): every lane decodes 8 consecutive K codes of one row per tile and multiplies
// them with the staged activations.  The input Hadamard runs in the prologue from global x, the
// output Hadamard + svh + residual in the epilogue, so a layer's linear is a single launch.
//
// The reference engine splits this over an input-transform kernel and a WMMA GEMM with a
// ticket-based split-K finish (reference: third_party/libr4d/r4d_gemm_trellis_nt_m64.hip:30-90,216).
#include <cooperative_groups.h>

#include "trellis_decode.cuh"

namespace cg = cooperative_groups;

namespace r4dxb {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;
constexpr int kMaxWorld = 8;

// Tensor-parallel epilogue: the all-reduce of a row-parallel linear, issued from the GEMV kernel.
// Every rank's CTA for block nb pushes its fp32 partial (T x 128) into each peer's receive slot
// with plain stores over NVLink, releases a per-(block, source) flag at system scope, waits
// (bounded) for the other ranks' flags of the same block, sums the partials in rank order -- the
// same order on every rank, so all ranks hold identical bits -- adds the residual and writes bf16.
// Receive slots are double-buffered by the call parity of a per-block sequence counter that lives
// in device memory (so a captured graph can be replayed).
struct TpPush {
  float* recv[kMaxWorld];          // recv[p]: rank p's receive buffer [2][world][8][N] (peer-mapped)
  unsigned* flags[kMaxWorld];      // flags[p]: rank p's flags [N/128][world]
  unsigned* block_seq;             // local [N/128] call counters
  int* status;                     // local: set non-zero when a wait ran out
  int world, rank, spin_limit;
};

__device__ __forceinline__ void StoreReleaseSys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned LoadAcquireSys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

template <int KB, int TMAX, bool kTp>
__global__ void __launch_bounds__(kThreads)
TrellisGemvKernel(const uint32_t* __restrict__ words, const __half* __restrict__ suh, const __half* __restrict__ svh,
                  const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                  const __nv_bfloat16* __restrict__ residual, int T, int N, int K, int kblocks_per_cta, TpPush tp) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  cg::cluster_group cluster = cg::this_cluster();
  const int ksplit = gridDim.x;
  const int krank = blockIdx.x;            // == rank inside the cluster
  const int nb = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int kslice = kblocks_per_cta * 128;
  const int k_begin = krank * kslice;

  float* part = reinterpret_cast<float*>(smem_raw);                       // [TMAX][128]
  __half* xs = reinterpret_cast<__half*>(smem_raw + TMAX * 128 * 4);       // [TMAX][kslice]

  // ---- prologue: xs = fp16(H128(suh * x)) for this CTA's K slice -------------------------------
  {
    const float inv_sqrt = 0.08838834764831845f;   // 1 / sqrt(128)
    for (int item = warp; item < kblocks_per_cta * TMAX; item += kThreads / 32) {
      const int t = item / kblocks_per_cta, b = item % kblocks_per_cta;
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      const int k = k_begin + b * 128 + lane * 4;
      if (t < T) {
        const uint2 xv = *reinterpret_cast<const uint2*>(x + static_cast<size_t>(t) * K + k);
        const uint2 sv = *reinterpret_cast<const uint2*>(suh + k);
        const __half2 s01 = *reinterpret_cast<const __half2*>(&sv.x), s23 = *reinterpret_cast<const __half2*>(&sv.y);
        v[0] = BfLo(xv.x) * __low2float(s01);
        v[1] = BfHi(xv.x) * __high2float(s01);
        v[2] = BfLo(xv.y) * __low2float(s23);
        v[3] = BfHi(xv.y) * __high2float(s23);
      }
      WarpFwht128(v);
      __half2 o01 = __floats2half2_rn(v[0] * inv_sqrt, v[1] * inv_sqrt);
      __half2 o23 = __floats2half2_rn(v[2] * inv_sqrt, v[3] * inv_sqrt);
      uint2 ov;
      ov.x = *reinterpret_cast<uint32_t*>(&o01);
      ov.y = *reinterpret_cast<uint32_t*>(&o23);
      *reinterpret_cast<uint2*>(xs + static_cast<size_t>(t) * kslice + b * 128 + lane * 4) = ov;
    }
  }
  __syncthreads();

  // ---- main loop: warp = n-tile, lane = (row, k half) ------------------------------------------
  constexpr int NW = 8 * KB;
  TrellisLane<KB> tl;
  tl.Init(lane);
  const int tiles_k = K / 16;
  const int kt_begin = k_begin / 16, kt_count = kslice / 16;
  // tile (nb, tk, warp) starts at ((nb * tiles_k + tk) * 8 + warp) * NW
  const uint32_t* wp = words + (static_cast<size_t>(nb) * tiles_k + kt_begin) * 8 * NW + warp * NW;
  constexpr size_t kTileStride = 8 * NW;   // words between consecutive k-tiles of the same n-tile

  float acc[TMAX];
#pragma unroll
  for (int t = 0; t < TMAX; ++t) acc[t] = 0.f;

  uint32_t cur[kUnroll][3], nxt[kUnroll][3];
  auto load = [&](uint32_t (&dst)[kUnroll][3], int kt) {
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint32_t* p = wp + static_cast<size_t>(kt + u) * kTileStride;
      dst[u][0] = __ldg(p + tl.i0);
      dst[u][1] = __ldg(p + tl.i1);
      if constexpr (KB != 4) dst[u][2] = __ldg(p + tl.i2); else dst[u][2] = 0;
    }
  };
  load(cur, 0);
  const int khalf = (lane & 1) * 8;
  for (int kt = 0; kt < kt_count; kt += kUnroll) {
    if (kt + kUnroll < kt_count) load(nxt, kt + kUnroll);
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      uint32_t hi, lo;
      tl.Window(cur[u][0], cur[u][1], cur[u][2], hi, lo);
      __half2 w[4];
      TrellisDecode8<KB>(hi, lo, w);
      const int kk = (kt + u) * 16 + khalf;
#pragma unroll
      for (int t = 0; t < TMAX; ++t) {
        const uint4 xv = *reinterpret_cast<const uint4*>(xs + static_cast<size_t>(t) * kslice + kk);
        __half2 s = __hmul2(w[0], *reinterpret_cast<const __half2*>(&xv.x));
        s = __hfma2(w[1], *reinterpret_cast<const __half2*>(&xv.y), s);
        s = __hfma2(w[2], *reinterpret_cast<const __half2*>(&xv.z), s);
        s = __hfma2(w[3], *reinterpret_cast<const __half2*>(&xv.w), s);
        acc[t] += __low2float(s) + __high2float(s);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      cur[u][0] = nxt[u][0]; cur[u][1] = nxt[u][1]; cur[u][2] = nxt[u][2];
    }
  }

  // ---- epilogue ---------------------------------------------------------------------------------
#pragma unroll
  for (int t = 0; t < TMAX; ++t) {
    acc[t] += __shfl_xor_sync(0xffffffffu, acc[t], 1);
    if ((lane & 1) == 0) part[t * 128 + warp * 16 + (lane >> 1)] = acc[t];
  }
  cluster.sync();   // every CTA's partial block is complete and visible cluster-wide
  if (krank == 0) {
    const float inv_sqrt = 0.08838834764831845f;
    float o[4] = {0.f, 0.f, 0.f, 0.f};
    const int t = warp;              // warp t finishes row t (T <= 8 = warps per CTA)
    const int n = nb * 128 + lane * 4;
    if (t < T) {
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      for (int r = 0; r < ksplit; ++r) {       // fixed order: the result does not depend on timing
        const float* rp = cluster.map_shared_rank(part, r);
        const float4 p = *reinterpret_cast<const float4*>(rp + t * 128 + lane * 4);
        v[0] += p.x; v[1] += p.y; v[2] += p.z; v[3] += p.w;
      }
      WarpFwht128(v);
      const uint2 sv = *reinterpret_cast<const uint2*>(svh + n);
      const __half2 s01 = *reinterpret_cast<const __half2*>(&sv.x), s23 = *reinterpret_cast<const __half2*>(&sv.y);
      o[0] = v[0] * inv_sqrt * __low2float(s01); o[1] = v[1] * inv_sqrt * __high2float(s01);
      o[2] = v[2] * inv_sqrt * __low2float(s23); o[3] = v[3] * inv_sqrt * __high2float(s23);
    }
    if constexpr (kTp) {
      __shared__ unsigned s_seq;
      __shared__ int s_fail;
      if (threadIdx.x == 0) { s_seq = tp.block_seq[nb] + 1; s_fail = 0; }
      __syncthreads();
      const unsigned seq = s_seq;
      const size_t slot_elems = static_cast<size_t>(tp.world) * 8 * N;
      const size_t my_off = (seq & 1) * slot_elems + (static_cast<size_t>(tp.rank) * 8 + t) * N + n;
      if (t < T) {
        for (int p = 0; p < tp.world; ++p)
          if (p != tp.rank) *reinterpret_cast<float4*>(tp.recv[p] + my_off) = make_float4(o[0], o[1], o[2], o[3]);
        __threadfence_system();
      }
      __syncthreads();
      if (threadIdx.x < tp.world && threadIdx.x != tp.rank) {
        StoreReleaseSys(tp.flags[threadIdx.x] + nb * tp.world + tp.rank, seq);
        // wait for the same block from that rank
        const unsigned* f = tp.flags[tp.rank] + nb * tp.world + threadIdx.x;
        bool ok = false;
        for (int i = 0; i < tp.spin_limit; ++i) {
          if (static_cast<int>(LoadAcquireSys(f) - seq) >= 0) { ok = true; break; }
          if (i > 64) __nanosleep(64);
        }
        if (!ok) { s_fail = 1; atomicExch(tp.status, 100 + static_cast<int>(threadIdx.x)); }
      }
      __syncthreads();
      if (t < T && !s_fail) {
        float a4[4] = {0.f, 0.f, 0.f, 0.f};
        const float* mine = tp.recv[tp.rank] + (seq & 1) * slot_elems;
        for (int r = 0; r < tp.world; ++r) {     // rank order, identical on every rank
          if (r == tp.rank) {
            a4[0] += o[0]; a4[1] += o[1]; a4[2] += o[2]; a4[3] += o[3];
          } else {
            const float4 p = __ldcg(reinterpret_cast<const float4*>(mine + (static_cast<size_t>(r) * 8 + t) * N + n));   // L2, never a stale L1 line
            a4[0] += p.x; a4[1] += p.y; a4[2] += p.z; a4[3] += p.w;
          }
        }
        o[0] = a4[0]; o[1] = a4[1]; o[2] = a4[2]; o[3] = a4[3];
      }
      if (threadIdx.x == 0) tp.block_seq[nb] = seq;
    }
    if (t < T) {
      if (residual != nullptr) {
        const uint2 rv = *reinterpret_cast<const uint2*>(residual + static_cast<size_t>(t) * N + n);
        o[0] += BfLo(rv.x); o[1] += BfHi(rv.x); o[2] += BfLo(rv.y); o[3] += BfHi(rv.y);
      }
      uint2 ov;
      ov.x = PackBf16(o[0], o[1]);
      ov.y = PackBf16(o[2], o[3]);
      *reinterpret_cast<uint2*>(y + static_cast<size_t>(t) * N + n) = ov;
    }
  }
  cluster.sync();   // peers keep their shared memory alive until rank 0 has read it
}

template <int KB, int TMAX, bool kTp>
int Launch(const void* words, const void* suh, const void* svh, const void* x, void* y, const void* residual, int T,
           int N, int K, int ksplit, cudaStream_t stream, const TpPush& tp) {
  const int kblocks = K / 128 / ksplit;
  const size_t smem = static_cast<size_t>(TMAX) * 128 * 4 + static_cast<size_t>(TMAX) * kblocks * 128 * 2;
  if (smem > 200 * 1024) return R4DXB_TOO_LARGE;
  auto kern = TrellisGemvKernel<KB, TMAX, kTp>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ksplit, N / 128, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = ksplit;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, static_cast<const uint32_t*>(words), static_cast<const __half*>(suh),
                                     static_cast<const __half*>(svh), static_cast<const __nv_bfloat16*>(x),
                                     static_cast<__nv_bfloat16*>(y), static_cast<const __nv_bfloat16*>(residual), T, N, K,
                                     kblocks, tp);
  ++g_launch_count;
  return static_cast<int>(e);
}

template <int KB, bool kTp>
int LaunchT(const void* words, const void* suh, const void* svh, const void* x, void* y, const void* residual, int T,
            int N, int K, int ksplit, cudaStream_t stream, const TpPush& tp) {
  if (T == 1) return Launch<KB, 1, kTp>(words, suh, svh, x, y, residual, T, N, K, ksplit, stream, tp);
  if (T == 2) return Launch<KB, 2, kTp>(words, suh, svh, x, y, residual, T, N, K, ksplit, stream, tp);
  if (T <= 4) return Launch<KB, 4, kTp>(words, suh, svh, x, y, residual, T, N, K, ksplit, stream, tp);
  return Launch<KB, 8, kTp>(words, suh, svh, x, y, residual, T, N, K, ksplit, stream, tp);
}

}  // namespace
}  // namespace r4dxb

extern "C" int r4dxb_trellis_gemv(const void* words, const void* suh, const void* svh, const void* x, void* y,
                                  const void* residual, int T, int N, int K, int kb, int ksplit, void* stream) {
  using namespace r4dxb;
  if (T < 1 || T > 8 || N % 128 || K % 128) return R4DXB_BAD_ARG;
  if (ksplit != 1 && ksplit != 2 && ksplit != 4 && ksplit != 8) return R4DXB_BAD_ARG;
  if ((K / 128) % ksplit) return R4DXB_BAD_ARG;
  if (((K / 128 / ksplit) * 8) % kUnroll) return R4DXB_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  TpPush none = {};
  switch (kb) {
    case 3: return LaunchT<3, false>(words, suh, svh, x, y, residual, T, N, K, ksplit, s, none);
    case 4: return LaunchT<4, false>(words, suh, svh, x, y, residual, T, N, K, ksplit, s, none);
    case 5: return LaunchT<5, false>(words, suh, svh, x, y, residual, T, N, K, ksplit, s, none);
    default: return R4DXB_BAD_ARG;
  }
}

// Row-parallel linear + all-reduce in one kernel (see TpPush).  recv / flags: `world` peer-mapped
// pointers (index = rank); block_seq, status: this rank's own memory.  spin_limit bounds every wait.
extern "C" int r4dxb_trellis_gemv_allreduce(const void* words, const void* suh, const void* svh, const void* x, void* y,
                                            const void* residual, int T, int N, int K, int kb, int ksplit,
                                            void* const* recv, void* const* flags, void* block_seq, int* status,
                                            int world, int rank, int spin_limit, void* stream) {
  using namespace r4dxb;
  if (T < 1 || T > 8 || N % 128 || K % 128 || world < 2 || world > kMaxWorld || rank < 0 || rank >= world) return R4DXB_BAD_ARG;
  if (ksplit != 1 && ksplit != 2 && ksplit != 4 && ksplit != 8) return R4DXB_BAD_ARG;
  if ((K / 128) % ksplit) return R4DXB_BAD_ARG;
  TpPush tp = {};
  for (int p = 0; p < world; ++p) {
    tp.recv[p] = static_cast<float*>(recv[p]);
    tp.flags[p] = static_cast<unsigned*>(flags[p]);
  }
  tp.block_seq = static_cast<unsigned*>(block_seq);
  tp.status = status;
  tp.world = world;
  tp.rank = rank;
  tp.spin_limit = spin_limit;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (kb) {
    case 3: return LaunchT<3, true>(words, suh, svh, x, y, residual, T, N, K, ksplit, s, tp);
    case 4: return LaunchT<4, true>(words, suh, svh, x, y, residual, T, N, K, ksplit, s, tp);
    case 5: return LaunchT<5, true>(words, suh, svh, x, y, residual, T, N, K, ksplit, s, tp);
    default: return R4DXB_BAD_ARG;
  }
}
