// Device-side sampling support: row summary (top-K raw logits + ids in canonical order + log-sum-exp
// of the temperature-scaled row) and the repetition penalty on a logits row.
//
// The summary lets the host sample exactly from a few hundred bytes instead of the ~1 MB row
// (reference: src/kernels/include/r4dx/kernels/kernels.h:425-486, summary_sampler.hpp:1-30).
// Canonical order: raw logit descending, ties toward the lower id.  Two stages: 128 parts each keep
// their local top-K and (max, sum-exp); one CTA merges.
#include "common.cuh"

namespace r4dxb {
namespace {

constexpr int kParts = 128;
constexpr int kMaxTopK = 64;

__device__ __forceinline__ bool Better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

// Finds the best (value, index) among candidates held per thread; block of 256.
__device__ void BlockArgBest(float& bv, int& bi, float* sv, int* si) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (Better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
  __syncthreads();
  bv = sv[0]; bi = si[0];
  for (int w = 1; w < (blockDim.x >> 5); ++w)
    if (Better(sv[w], si[w], bv, bi)) { bv = sv[w]; bi = si[w]; }
}

// grid (kParts, T), block 256.  pvals/pids: [T][kParts][K]; pstat: [T][kParts][2] = (max of scaled, sum exp)
__global__ void TopkLsePartial(const float* __restrict__ logits, int V, int K, float inv_t, float* __restrict__ pvals,
                               int* __restrict__ pids, float* __restrict__ pstat) {
  __shared__ float sv[8];
  __shared__ int si[8];
  __shared__ float red[32];
  const int t = blockIdx.y, part = blockIdx.x;
  const int chunk = (V + kParts - 1) / kParts;
  const int b = part * chunk, e = min(V, b + chunk);
  const float* row = logits + static_cast<size_t>(t) * V;
  // lse pieces
  float mx = -INFINITY;
  for (int i = b + threadIdx.x; i < e; i += blockDim.x) mx = fmaxf(mx, row[i] * inv_t);
  mx = WarpMax(mx);
  {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    mx = red[0];
    for (int w = 1; w < (blockDim.x >> 5); ++w) mx = fmaxf(mx, red[w]);
    __syncthreads();
  }
  float se = 0.f;
  for (int i = b + threadIdx.x; i < e; i += blockDim.x) se += __expf(row[i] * inv_t - mx);
  se = BlockSum(se, red);
  if (threadIdx.x == 0) {
    pstat[(static_cast<size_t>(t) * kParts + part) * 2] = mx;
    pstat[(static_cast<size_t>(t) * kParts + part) * 2 + 1] = se;
  }
  // local top-K by K rounds of arg-best below the previous pick
  float lastv = INFINITY;
  int lasti = -1;
  for (int j = 0; j < K; ++j) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = b + threadIdx.x; i < e; i += blockDim.x) {
      const float v = row[i];
      const bool after_last = v < lastv || (v == lastv && i > lasti);
      if (after_last && Better(v, i, bv, bi)) { bv = v; bi = i; }
    }
    BlockArgBest(bv, bi, sv, si);
    if (threadIdx.x == 0) {
      pvals[(static_cast<size_t>(t) * kParts + part) * K + j] = bv;
      pids[(static_cast<size_t>(t) * kParts + part) * K + j] = bi;
    }
    lastv = bv;
    lasti = bi;
  }
}

// grid T, block 256
__global__ void TopkLseMerge(const float* __restrict__ pvals, const int* __restrict__ pids, const float* __restrict__ pstat, int K,
                             int id_offset, float* __restrict__ out_vals, int* __restrict__ out_ids, float* __restrict__ out_lse) {
  __shared__ float sv[8];
  __shared__ int si[8];
  const int t = blockIdx.x;
  const int n = kParts * K;
  const float* v = pvals + static_cast<size_t>(t) * n;
  const int* id = pids + static_cast<size_t>(t) * n;
  float lastv = INFINITY;
  int lasti = -1;
  for (int j = 0; j < K; ++j) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const float x = v[i];
      const int xi = id[i];
      if (xi == 0x7fffffff) continue;
      const bool after_last = x < lastv || (x == lastv && xi > lasti);
      if (after_last && Better(x, xi, bv, bi)) { bv = x; bi = xi; }
    }
    BlockArgBest(bv, bi, sv, si);
    if (threadIdx.x == 0) {
      out_vals[static_cast<size_t>(t) * K + j] = bv;
      out_ids[static_cast<size_t>(t) * K + j] = bi == 0x7fffffff ? -1 : bi + id_offset;
    }
    lastv = bv;
    lasti = bi;
  }
  if (threadIdx.x == 0) {
    float mx = -INFINITY;
    for (int p = 0; p < kParts; ++p) mx = fmaxf(mx, pstat[(static_cast<size_t>(t) * kParts + p) * 2]);
    float s = 0.f;
    for (int p = 0; p < kParts; ++p) {
      const float m = pstat[(static_cast<size_t>(t) * kParts + p) * 2];
      if (m != -INFINITY) s += pstat[(static_cast<size_t>(t) * kParts + p) * 2 + 1] * __expf(m - mx);
    }
    out_lse[t] = mx + __logf(s);
  }
}

__global__ void RepPenaltyKernel(float* __restrict__ logits, int V, const int* __restrict__ seen, int n, float penalty) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int id = seen[i];
  if (id < 0 || id >= V) return;
  // a token that occurs several times is penalised once: only its first occurrence acts
  for (int j = 0; j < i; ++j)
    if (seen[j] == id) return;
  const float v = logits[id];
  logits[id] = v > 0.f ? v / penalty : v * penalty;
}

}  // namespace
}  // namespace r4dxb

using namespace r4dxb;

extern "C" {

/* scratch: T * 128 * (2K + 2) * 4 bytes */
int r4dxb_topk_lse(const float* logits, int T, int V, int K, float temperature, int id_offset, float* out_vals, int* out_ids,
                   float* out_lse, void* scratch, void* stream) {
  if (T < 1 || K < 1 || K > kMaxTopK || V < K) return R4DXB_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* pvals = static_cast<float*>(scratch);
  int* pids = reinterpret_cast<int*>(pvals + static_cast<size_t>(T) * kParts * K);
  float* pstat = reinterpret_cast<float*>(pids + static_cast<size_t>(T) * kParts * K);
  const float inv_t = temperature > 0.f ? 1.0f / temperature : 1.0f;
  TopkLsePartial<<<dim3(kParts, T), 256, 0, s>>>(logits, V, K, inv_t, pvals, pids, pstat);
  int e = FinishLaunch();
  if (e) return e;
  TopkLseMerge<<<T, 256, 0, s>>>(pvals, pids, pstat, K, id_offset, out_vals, out_ids, out_lse);
  return FinishLaunch();
}

int r4dxb_repetition_penalty(float* logits, int V, const int* seen, int n, float penalty, void* stream) {
  if (n < 1) return 0;
  RepPenaltyKernel<<<(n + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(logits, V, seen, n, penalty);
  return FinishLaunch();
}

}  // extern "C"
