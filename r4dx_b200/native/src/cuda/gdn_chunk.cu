// Chunked (WY-form) gated delta rule for long prefill chunks, D = 128, 64 tokens per chunk.
//
// With gamma_i the running product of the decay inside a chunk and S0 the state before it, the 64
// rank-one updates of the chunk collapse to
//   (I + A) U = beta V - (beta gamma K) S0^T,   A_ij = beta_i (gamma_i / gamma_j) (k_i . k_j), j < i
//   O   = diag(gamma) Q S0^T + P U,             P_ij = (gamma_i / gamma_j) (q_i . k_j),       j <= i
//   S64 = gamma_64 S0 + U^T diag(gamma_64 / gamma) K
// so the work splits in two kernels:
//   phase A (grid chunks x heads, no dependence on the state): A and P in fp32, then the triangular
//           solve for U~ = (I + A)^-1 beta V and W = (I + A)^-1 beta gamma K by forward substitution,
//           one right-hand-side column per thread with the 64 unknowns in registers;
//   phase B (grid heads x 4 row blocks of the state, sequential over chunks): U = U~ - W S0^T,
//           O, and the state update as TF32 tensor-core products (mma.sync m16n8k8, fp32
//           accumulate) out of shared memory; W, Q, P and K stream through two cp.async slots, each
//           fetched one product ahead of its use.  The fp32 state block lives in shared memory for
//           the whole sequence.
// The per-token recurrence (gdn_prefill.cu) stays as the reference path and for D = 64
// (reference: third_party/libr4d/r4d_gdn_chunk_scan_k128_v128_c64_bf16.hip:1-60 runs the same
// algebra in bf16 on its matrix cores).
#include <cuda_pipeline.h>

#include "common.cuh"

namespace r4dxb {
namespace {

constexpr int kC = 64;            // tokens per chunk
constexpr int kD = 128;           // key and value head width
constexpr int kLdK = kD + 4;      // phase A: row stride of k / q (conflict-free 16-byte row reads)
constexpr int kLdA = kC + 4;

struct PhaseASmem {
  float ks[kC][kLdK];
  float qs[kC][kLdK];
  float As[kC][kLdA];
  float G[kC];
  float B[kC];
};

__device__ __forceinline__ float Dot4(const float4& a, const float4& b, float acc) {
  acc = fmaf(a.x, b.x, acc);
  acc = fmaf(a.y, b.y, acc);
  acc = fmaf(a.z, b.z, acc);
  return fmaf(a.w, b.w, acc);
}

// grid (chunks, H), 256 threads
__global__ void __launch_bounds__(256) GdnChunkPrepKernel(const float* __restrict__ q, const float* __restrict__ k,
                                                          const float* __restrict__ v, const float* __restrict__ eg,
                                                          const float* __restrict__ beta, float* __restrict__ ws_ut,
                                                          float* __restrict__ ws_w, float* __restrict__ ws_p,
                                                          float* __restrict__ ws_g, int T, int H, int Hk) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  PhaseASmem& sm = *reinterpret_cast<PhaseASmem*>(smem_raw);
  const int c = blockIdx.x, h = blockIdx.y, hk = h / (H / Hk);
  const int t0 = c * kC, tid = threadIdx.x;
  const size_t ch = static_cast<size_t>(c) * H + h;

  for (int i = tid; i < kC * kD / 4; i += 256) {
    const int row = i / (kD / 4), off = (i % (kD / 4)) * 4;
    const int t = t0 + row;
    float4 kv = make_float4(0.f, 0.f, 0.f, 0.f), qv = kv;
    if (t < T) {
      kv = *reinterpret_cast<const float4*>(k + (static_cast<size_t>(t) * Hk + hk) * kD + off);
      qv = *reinterpret_cast<const float4*>(q + (static_cast<size_t>(t) * Hk + hk) * kD + off);
    }
    *reinterpret_cast<float4*>(&sm.ks[row][off]) = kv;
    *reinterpret_cast<float4*>(&sm.qs[row][off]) = qv;
  }
  if (tid < kC) {
    const int t = t0 + tid;
    // rows past the end are identity steps: decay 1, beta 0
    sm.B[tid] = t < T ? beta[static_cast<size_t>(t) * H + h] : 0.f;
    sm.G[tid] = t < T ? fmaxf(logf(eg[static_cast<size_t>(t) * H + h]), -80.f) : 0.f;
  }
  __syncthreads();
  if (tid == 0) {
    float acc = 0.f;
    for (int i = 0; i < kC; ++i) {
      acc += sm.G[i];
      sm.G[i] = acc;
    }
  }
  __syncthreads();
  if (tid < kC) ws_g[ch * kC + tid] = sm.G[tid];

  // ---- k.k and q.k for the lower triangle: thread (ty, tx) owns rows ty + 16 rr, columns tx + 16 cc ----
  {
    const int ty = tid >> 4, tx = tid & 15;
    float kk[4][4], qk[4][4];
#pragma unroll
    for (int rr = 0; rr < 4; ++rr)
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) kk[rr][cc] = qk[rr][cc] = 0.f;
    for (int kq = 0; kq < kD; kq += 4) {
      float4 kr[4], qr[4], kc[4];
#pragma unroll
      for (int rr = 0; rr < 4; ++rr) {
        kr[rr] = *reinterpret_cast<const float4*>(&sm.ks[ty + 16 * rr][kq]);
        qr[rr] = *reinterpret_cast<const float4*>(&sm.qs[ty + 16 * rr][kq]);
        kc[rr] = *reinterpret_cast<const float4*>(&sm.ks[tx + 16 * rr][kq]);
      }
#pragma unroll
      for (int rr = 0; rr < 4; ++rr)
#pragma unroll
        for (int cc = 0; cc < 4; ++cc)
          if (cc <= rr) {      // 16-wide column blocks right of the row block are entirely above the diagonal
            kk[rr][cc] = Dot4(kr[rr], kc[cc], kk[rr][cc]);
            qk[rr][cc] = Dot4(qr[rr], kc[cc], qk[rr][cc]);
          }
    }
#pragma unroll
    for (int rr = 0; rr < 4; ++rr)
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        const int i = ty + 16 * rr, j = tx + 16 * cc;
        const float decay = j <= i ? expf(sm.G[i] - sm.G[j]) : 0.f;
        sm.As[i][j] = j < i ? sm.B[i] * decay * kk[rr][cc] : 0.f;
        ws_p[(ch * kC + i) * kC + j] = decay * qk[rr][cc];
      }
  }
  __syncthreads();

  // ---- forward substitution: thread = one right-hand-side column (128 of beta V, 128 of beta gamma K) ----
  {
    const bool is_u = tid < kD;
    const int col = is_u ? tid : tid - kD;
    float* dst = (is_u ? ws_ut : ws_w) + ch * kC * kD + col;
    float x[kC];
#pragma unroll
    for (int i = 0; i < kC; ++i) {
      float rhs;
      if (is_u) {
        const int t = t0 + i;
        rhs = t < T ? sm.B[i] * v[(static_cast<size_t>(t) * H + h) * kD + col] : 0.f;
      } else {
        rhs = sm.B[i] * expf(sm.G[i]) * sm.ks[i][col];
      }
      float acc0 = rhs, acc1 = 0.f;
#pragma unroll
      for (int j = 0; j + 3 < i; j += 4) {
        const float4 a = *reinterpret_cast<const float4*>(&sm.As[i][j]);
        acc0 = fmaf(-a.x, x[j], acc0);
        acc1 = fmaf(-a.y, x[j + 1], acc1);
        acc0 = fmaf(-a.z, x[j + 2], acc0);
        acc1 = fmaf(-a.w, x[j + 3], acc1);
      }
#pragma unroll
      for (int j = (i / 4) * 4; j < i; ++j) acc0 = fmaf(-sm.As[i][j], x[j], acc0);
      x[i] = acc0 + acc1;
      dst[static_cast<size_t>(i) * kD] = x[i];
    }
  }
}

// ---------------------------------------- phase B ----------------------------------------
constexpr int kLd = kD + 8;       // W / Q / K / state rows: conflict-free 8-byte fragment reads and strided scalar reads
constexpr int kLdP = kC + 4;      // P rows: conflict-free scalar fragment reads
constexpr int kLdU = 32 + 8;      // U rows (this CTA's 32 value columns)
constexpr int kSlotFloats = kC * kLd;

struct PhaseBSmem {
  float slot[2][kSlotFloats];
  float S[32][kLd];
  float U[2][kC][kLdU];
  float G[2][kC];
  float eG[kC];
  float fG[kC];
};

__device__ __forceinline__ uint32_t Tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}

__device__ __forceinline__ void MmaTf32(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// acc[nt] += A[m0 .. m0+16, 0 .. 128) * S[n0 + 8 nt .. +8, 0 .. 128)^T, both row-major along the contraction.
// Inside every block of 8 contraction columns the hardware index t maps to column 2t and t + 4 to 2t + 1, so
// that one 8-byte load feeds two fragment registers; A and B use the same map, so the product is unchanged.
template <int NT>
__device__ __forceinline__ void MmaRowRow(float (&acc)[NT][4], const float* __restrict__ A, int m0, const float* __restrict__ S,
                                          int n0, int lane) {
  const int g = lane >> 2, t = lane & 3;
  const float* a_lo = A + (m0 + g) * kLd + 2 * t;
  const float* a_hi = a_lo + 8 * kLd;
  const float* b_base = S + (n0 + g) * kLd + 2 * t;
#pragma unroll 4
  for (int kb = 0; kb < kD / 8; ++kb) {
    const float2 lo = *reinterpret_cast<const float2*>(a_lo + kb * 8);
    const float2 hi = *reinterpret_cast<const float2*>(a_hi + kb * 8);
    const uint32_t a0 = Tf32(lo.x), a2 = Tf32(lo.y), a1 = Tf32(hi.x), a3 = Tf32(hi.y);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const float2 b = *reinterpret_cast<const float2*>(b_base + nt * 8 * kLd + kb * 8);
      MmaTf32(acc[nt], a0, a1, a2, a3, Tf32(b.x), Tf32(b.y));
    }
  }
}

__device__ __forceinline__ void CopyRows(float* dst, int ld_dst, const float* src, size_t src_stride, int rows, int row_floats,
                                         int tid) {
  const int per_row = row_floats / 4;
  for (int i = tid; i < rows * per_row; i += 256) {
    const int r = i / per_row, o = (i % per_row) * 4;
    __pipeline_memcpy_async(dst + r * ld_dst + o, src + static_cast<size_t>(r) * src_stride + o, 16);
  }
}

// grid (H, 4), 256 threads: CTA (h, vb) owns state rows [32 vb, 32 vb + 32) of head h
__global__ void __launch_bounds__(256, 2) GdnChunkScanKernel(const float* __restrict__ q, const float* __restrict__ k,
                                                             const float* __restrict__ ws_ut, const float* __restrict__ ws_w,
                                                             const float* __restrict__ ws_p, const float* __restrict__ ws_g,
                                                             float* __restrict__ state, float* __restrict__ o, int T, int H,
                                                             int Hk) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  PhaseBSmem& sm = *reinterpret_cast<PhaseBSmem*>(smem_raw);
  const int h = blockIdx.x, vb = blockIdx.y, hk = h / (H / Hk);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  const int chunks = (T + kC - 1) / kC;
  const float scale = rsqrtf(static_cast<float>(kD));

  auto issue_wug = [&](int c, int buf) {      // W -> slot 0, U~ (this CTA's columns) and G
    const size_t ch = static_cast<size_t>(c) * H + h;
    CopyRows(sm.slot[0], kLd, ws_w + ch * kC * kD, kD, kC, kD, tid);
    CopyRows(&sm.U[buf][0][0], kLdU, ws_ut + ch * kC * kD + vb * 32, kD, kC, 32, tid);
    if (tid < kC / 4) __pipeline_memcpy_async(&sm.G[buf][tid * 4], ws_g + ch * kC + tid * 4, 16);
    __pipeline_commit();
  };
  auto issue_qk = [&](const float* src, int c, int slot) {     // token rows of q or k (clamped past the end)
    for (int i = tid; i < kC * (kD / 4); i += 256) {
      const int r = i / (kD / 4), off = (i % (kD / 4)) * 4;
      const int t = min(c * kC + r, T - 1);
      __pipeline_memcpy_async(&sm.slot[slot][r * kLd + off], src + (static_cast<size_t>(t) * Hk + hk) * kD + off, 16);
    }
    __pipeline_commit();
  };

  issue_wug(0, 0);
  for (int i = tid; i < 32 * (kD / 4); i += 256) {
    const int r = i / (kD / 4), off = (i % (kD / 4)) * 4;
    *reinterpret_cast<float4*>(&sm.S[r][off]) =
        *reinterpret_cast<const float4*>(state + (static_cast<size_t>(h) * kD + vb * 32 + r) * kD + off);
  }

  for (int c = 0; c < chunks; ++c) {
    const int buf = c & 1;
    const size_t ch = static_cast<size_t>(c) * H + h;
    __pipeline_wait_prior(0);
    __syncthreads();                       // W, U~, G of this chunk have landed; the state block is complete
    issue_qk(q, c, 1);
    if (tid < kC) {
      sm.eG[tid] = expf(sm.G[buf][tid]);
      sm.fG[tid] = expf(sm.G[buf][kC - 1] - sm.G[buf][tid]);
    }
    // ---- 1: U = U~ - W S^T   (64 x 32; warp: 16 rows x 16 columns) ----
    const int m0 = (warp & 3) * 16, nh = (warp >> 2) * 16;
    {
      float acc[2][4] = {};
      MmaRowRow<2>(acc, sm.slot[0], m0, &sm.S[0][0], nh, lane);
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        float2* lo = reinterpret_cast<float2*>(&sm.U[buf][m0 + g][nh + nt * 8 + 2 * t4]);
        float2* hi = reinterpret_cast<float2*>(&sm.U[buf][m0 + g + 8][nh + nt * 8 + 2 * t4]);
        float2 a = *lo, b = *hi;
        a.x -= acc[nt][0]; a.y -= acc[nt][1]; b.x -= acc[nt][2]; b.y -= acc[nt][3];
        *lo = a;
        *hi = b;
      }
    }
    __pipeline_wait_prior(0);
    __syncthreads();                       // U complete, Q landed, W no longer read
    CopyRows(sm.slot[0], kLdP, ws_p + ch * kC * kC, kC, kC, kC, tid);
    __pipeline_commit();
    // ---- 2a: O = diag(gamma) Q S^T ----
    float oacc[2][4] = {};
    MmaRowRow<2>(oacc, sm.slot[1], m0, &sm.S[0][0], nh, lane);
    {
      const float e_lo = sm.eG[m0 + g], e_hi = sm.eG[m0 + g + 8];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        oacc[nt][0] *= e_lo; oacc[nt][1] *= e_lo; oacc[nt][2] *= e_hi; oacc[nt][3] *= e_hi;
      }
    }
    __pipeline_wait_prior(0);
    __syncthreads();                       // P landed, Q no longer read
    issue_qk(k, c, 1);
    // ---- 2b: O += P U ----
    {
      const float* P = sm.slot[0];
#pragma unroll 2
      for (int kb = 0; kb < kC / 8; ++kb) {
        const uint32_t a0 = Tf32(P[(m0 + g) * kLdP + kb * 8 + t4]), a1 = Tf32(P[(m0 + g + 8) * kLdP + kb * 8 + t4]);
        const uint32_t a2 = Tf32(P[(m0 + g) * kLdP + kb * 8 + t4 + 4]), a3 = Tf32(P[(m0 + g + 8) * kLdP + kb * 8 + t4 + 4]);
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const uint32_t b0 = Tf32(sm.U[buf][kb * 8 + t4][nh + nt * 8 + g]);
          const uint32_t b1 = Tf32(sm.U[buf][kb * 8 + t4 + 4][nh + nt * 8 + g]);
          MmaTf32(oacc[nt], a0, a1, a2, a3, b0, b1);
        }
      }
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const int col = vb * 32 + nh + nt * 8 + 2 * t4;
        const int t_lo = c * kC + m0 + g, t_hi = t_lo + 8;
        if (t_lo < T)
          *reinterpret_cast<float2*>(o + (static_cast<size_t>(t_lo) * H + h) * kD + col) =
              make_float2(oacc[nt][0] * scale, oacc[nt][1] * scale);
        if (t_hi < T)
          *reinterpret_cast<float2*>(o + (static_cast<size_t>(t_hi) * H + h) * kD + col) =
              make_float2(oacc[nt][2] * scale, oacc[nt][3] * scale);
      }
    }
    __pipeline_wait_prior(0);
    __syncthreads();                       // K landed, P no longer read
    if (c + 1 < chunks) issue_wug(c + 1, buf ^ 1);
    // ---- 3: S = gamma_C S + U^T diag(gamma_C / gamma) K   (32 x 128; warp: 16 rows x 32 columns) ----
    {
      const int sm0 = (warp & 1) * 16, sn0 = (warp >> 1) * 32;
      const float e_c = sm.eG[kC - 1];
      float acc[4][4];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const float2 lo = *reinterpret_cast<const float2*>(&sm.S[sm0 + g][sn0 + nt * 8 + 2 * t4]);
        const float2 hi = *reinterpret_cast<const float2*>(&sm.S[sm0 + g + 8][sn0 + nt * 8 + 2 * t4]);
        acc[nt][0] = lo.x * e_c; acc[nt][1] = lo.y * e_c; acc[nt][2] = hi.x * e_c; acc[nt][3] = hi.y * e_c;
      }
      const float* Kt = sm.slot[1];
#pragma unroll 2
      for (int kb = 0; kb < kC / 8; ++kb) {
        const int j0 = kb * 8 + t4, j1 = j0 + 4;
        const float f0 = sm.fG[j0], f1 = sm.fG[j1];
        const uint32_t a0 = Tf32(sm.U[buf][j0][sm0 + g] * f0), a1 = Tf32(sm.U[buf][j0][sm0 + g + 8] * f0);
        const uint32_t a2 = Tf32(sm.U[buf][j1][sm0 + g] * f1), a3 = Tf32(sm.U[buf][j1][sm0 + g + 8] * f1);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          const uint32_t b0 = Tf32(Kt[j0 * kLd + sn0 + nt * 8 + g]), b1 = Tf32(Kt[j1 * kLd + sn0 + nt * 8 + g]);
          MmaTf32(acc[nt], a0, a1, a2, a3, b0, b1);
        }
      }
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        *reinterpret_cast<float2*>(&sm.S[sm0 + g][sn0 + nt * 8 + 2 * t4]) = make_float2(acc[nt][0], acc[nt][1]);
        *reinterpret_cast<float2*>(&sm.S[sm0 + g + 8][sn0 + nt * 8 + 2 * t4]) = make_float2(acc[nt][2], acc[nt][3]);
      }
    }
  }
  __pipeline_wait_prior(0);
  __syncthreads();
  for (int i = tid; i < 32 * (kD / 4); i += 256) {
    const int r = i / (kD / 4), off = (i % (kD / 4)) * 4;
    *reinterpret_cast<float4*>(state + (static_cast<size_t>(h) * kD + vb * 32 + r) * kD + off) =
        *reinterpret_cast<const float4*>(&sm.S[r][off]);
  }
}

}  // namespace

// Runs both phases on `stream`; ws must hold r4dxb_gdn_chunk_ws_floats(T, H) floats.
int LaunchGdnChunked(const float* q, const float* k, const float* v, const float* eg, const float* beta, float* state, float* o,
                     float* ws, int T, int H, int Hk, cudaStream_t s) {
  const int chunks = (T + kC - 1) / kC;
  const size_t per = static_cast<size_t>(chunks) * H * kC;
  float* ws_ut = ws;
  float* ws_w = ws_ut + per * kD;
  float* ws_p = ws_w + per * kD;
  float* ws_g = ws_p + per * kC;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(GdnChunkPrepKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sizeof(PhaseASmem)));
    cudaFuncSetAttribute(GdnChunkScanKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sizeof(PhaseBSmem)));
    configured = true;
  }
  GdnChunkPrepKernel<<<dim3(chunks, H), 256, sizeof(PhaseASmem), s>>>(q, k, v, eg, beta, ws_ut, ws_w, ws_p, ws_g, T, H, Hk);
  int e = FinishLaunch();
  if (e) return e;
  GdnChunkScanKernel<<<dim3(H, 4), 256, sizeof(PhaseBSmem), s>>>(q, k, ws_ut, ws_w, ws_p, ws_g, state, o, T, H, Hk);
  return FinishLaunch();
}

}  // namespace r4dxb

extern "C" {

/* fp32 workspace of the chunked GDN prefill for T tokens and H value heads (D = 128) */
long long r4dxb_gdn_chunk_ws_floats(int T, int H) {
  const long long chunks = (T + r4dxb::kC - 1) / r4dxb::kC;
  return chunks * H * r4dxb::kC * (2LL * r4dxb::kD + r4dxb::kC + 1);
}

}  // extern "C"
