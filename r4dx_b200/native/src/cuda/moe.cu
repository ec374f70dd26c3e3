// Mixture-of-experts routing and combine kernels (softmax top-k router, device-side plan, weighted
// combine with the shared expert).  The grouped expert GEMV itself lives in trellis_gemv.cu.
//
// Semantics (reference: src/model/qwen4exp/include/r4dx/model/qwen4exp/moe_kernels.h:18-56):
//   * router: fp32 softmax over the expert logits, top-k (k <= 16, experts <= 1024), optional
//     renormalisation, weights rounded through bf16; ties go to the larger logit, then the lower id;
//   * plan: (token, slot) pairs sorted by expert id (stable), with per-expert offsets, built on
//     the device so that no routing decision is read back by the host;
//   * combine: out[t] = residual[t] + sum_j w[t,j] * y[pair(t,j)] in ascending expert id (a fixed
//     order: no atomics) + sigmoid(shared_gate[t]) * shared[t], one bf16 rounding.
#include "common.cuh"

namespace r4dxb {
namespace {

constexpr int kMaxK = 16;

// one warp per token row
//
// mode 1 is the sigmoid router of the short-conv MoE family (reference:
// src/kernels/include/r4dx/kernels/lfm2_kernels.h:38-50): s[e] = sigmoid(logit[e]); the SELECTION ranks s[e] + bias[e]
// (ties to the lower id), the weights are the unbiased s of the selected experts, divided by (their sum + 1e-6) when
// renorm is set, then multiplied by `scale`.
// One warp routes one row.  The row's selection values live in registers (E <= 1024: 32 per lane), so the k arg-max rounds
// touch no memory; a lane remembers its taken entries in a bit mask.
__device__ __forceinline__ void RouteRow(const float* __restrict__ row, const float* __restrict__ bias, int E, int k, int renorm,
                                         int mode, float scale, int lane, int* __restrict__ ids, float* __restrict__ weights) {
  float v[32];
  float mx = -INFINITY, z = 0.f;
#pragma unroll
  for (int s = 0; s < 32; ++s) {
    const int e = lane + 32 * s;
    float x = -INFINITY;
    if (e < E) x = mode == 0 ? row[e] : 1.0f / (1.0f + expf(-row[e])) + (bias ? bias[e] : 0.f);
    v[s] = x;
    mx = fmaxf(mx, x);
  }
  if (mode == 0) {
    mx = WarpMax(mx);
#pragma unroll
    for (int s = 0; s < 32; ++s) z += (lane + 32 * s < E) ? __expf(v[s] - mx) : 0.f;
    z = WarpSum(z);
  }
  float wsum = 0.f;
  uint32_t taken = 0;              // bit s: this lane's entry lane + 32 s is already picked
  float my_p = 0.f;                // lane j keeps the j-th pick (k <= 16 <= 32)
  int my_i = 0;
  for (int j = 0; j < k; ++j) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int s = 0; s < 32; ++s) {
      const int e = lane + 32 * s;
      if (e < E && !((taken >> s) & 1u) && (v[s] > bv || (v[s] == bv && e < bi))) { bv = v[s]; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((bi & 31) == lane) taken |= 1u << (bi >> 5);
    const float p = mode == 0 ? __expf(bv - mx) / z : 1.0f / (1.0f + expf(-row[bi]));
    if (lane == j) { my_p = p; my_i = bi; }
    wsum += p;
  }
  if (lane < k) {
    const float w = mode == 0 ? (renorm ? my_p / wsum : my_p) : (renorm ? my_p / (wsum + 1e-6f) : my_p) * scale;
    ids[lane] = my_i;
    weights[lane] = __bfloat162float(__float2bfloat16(w));
  }
}

__global__ void MoeRouterKernel(const float* __restrict__ logits, const float* __restrict__ bias, int T, int E, int k,
                                int renorm, int mode, float scale, int* __restrict__ ids, float* __restrict__ weights) {
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  RouteRow(logits + static_cast<size_t>(t) * E, bias, E, k, renorm, mode, scale, threadIdx.x & 31, ids + static_cast<size_t>(t) * k,
           weights + static_cast<size_t>(t) * k);
}

// Up to 8 rows (a decode step or a verify window): one CTA routes every row (a warp each) and then builds the plan of the
// T * k pairs itself, so routing is one launch instead of two.  Same results as MoeRouterKernel + MoePlanKernel.
__global__ void __launch_bounds__(256)
MoeRoutePlanKernel(const float* __restrict__ logits, const float* __restrict__ bias, int T, int E, int k, int renorm, int mode,
                   float scale, int* __restrict__ ids, float* __restrict__ weights, int e_begin, int e_count,
                   int* __restrict__ offsets, int* __restrict__ perm) {
  extern __shared__ int cnt[];     // [e_count + 1]
  __shared__ int s_ids[8 * kMaxK];
  const int warp = threadIdx.x >> 5;
  for (int e = threadIdx.x; e <= e_count; e += blockDim.x) cnt[e] = 0;
  if (warp < T)
    RouteRow(logits + static_cast<size_t>(warp) * E, bias, E, k, renorm, mode, scale, threadIdx.x & 31, ids + warp * k, weights + warp * k);
  __syncthreads();                 // the ids written above are visible to the whole CTA
  const int npairs = T * k;
  if (threadIdx.x < npairs) {
    const int e = ids[threadIdx.x] - e_begin;
    s_ids[threadIdx.x] = e;
    if (e >= 0 && e < e_count) atomicAdd(&cnt[e + 1], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int e = 0; e < e_count; ++e) cnt[e + 1] += cnt[e];
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= e_count; e += blockDim.x) offsets[e] = cnt[e];
  __syncthreads();
  if (threadIdx.x == 0) {          // stable placement: pairs in ascending index (at most 128 pairs)
    for (int p = 0; p < npairs; ++p) {
      const int e = s_ids[p];
      if (e >= 0 && e < e_count) perm[cnt[e]++] = p;
    }
  }
}

// Single CTA: counting sort of the T*k pairs by expert (stable in pair order).
__global__ void MoePlanKernel(const int* __restrict__ ids, int npairs, int E, int e_begin, int e_count,
                              int* __restrict__ offsets, int* __restrict__ perm) {
  extern __shared__ int cnt[];     // [e_count + 1]
  for (int e = threadIdx.x; e <= e_count; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < npairs; p += blockDim.x) {
    const int e = ids[p] - e_begin;
    if (e >= 0 && e < e_count) atomicAdd(&cnt[e + 1], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int e = 0; e < e_count; ++e) cnt[e + 1] += cnt[e];
    for (int e = 0; e <= e_count; ++e) offsets[e] = cnt[e];
    // stable placement: pairs in ascending index (serial, npairs is a few hundred)
    for (int p = 0; p < npairs; ++p) {
      const int e = ids[p] - e_begin;
      if (e >= 0 && e < e_count) perm[cnt[e]++] = p;
    }
  }
}

// The same plan for many pairs (prefill chunks, wide batches): one CTA of 32 warps, warp w owns a contiguous run of the
// pairs.  Pass 1 counts per (warp, expert), a prefix over experts and warps turns the counts into each warp's first slot
// per expert, pass 2 places the pairs; inside a 32-pair step the lanes of one expert are ranked with match_any, so the
// order inside an expert is the pair order, exactly as the serial kernel leaves it.
constexpr int kPlanWarps = 32;
__global__ void __launch_bounds__(kPlanWarps * 32)
MoePlanParallelKernel(const int* __restrict__ ids, int npairs, int e_begin, int e_count, int* __restrict__ offsets,
                      int* __restrict__ perm) {
  extern __shared__ int sm[];                  // [kPlanWarps][e_count] counts / cursors, then [e_count + 1] offsets
  int* hist = sm;
  int* offs = sm + kPlanWarps * e_count;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < kPlanWarps * e_count; i += blockDim.x) hist[i] = 0;
  __syncthreads();
  const int per = ((npairs + kPlanWarps - 1) / kPlanWarps + 31) & ~31;       // pairs per warp, a multiple of 32
  const int p0 = warp * per, p1 = min(npairs, p0 + per);
  int* mine = hist + warp * e_count;
  for (int base = p0; base < p1; base += 32) {
    const int p = base + lane;
    int e = p < p1 ? ids[p] - e_begin : -1;
    if (e >= e_count) e = -1;
    const unsigned same = __match_any_sync(0xffffffffu, e);
    if (e >= 0 && lane == __ffs(same) - 1) mine[e] += __popc(same);
    __syncwarp();
  }
  __syncthreads();
  // per expert: total, then each warp's first slot
  for (int e = threadIdx.x; e < e_count; e += blockDim.x) {
    int tot = 0;
    for (int w = 0; w < kPlanWarps; ++w) tot += hist[w * e_count + e];
    offs[e + 1] = tot;
  }
  if (threadIdx.x == 0) offs[0] = 0;
  __syncthreads();
  if (warp == 0) {                             // inclusive scan over the experts by one warp
    int carry = 0;
    for (int b = 0; b < e_count; b += 32) {
      const int e = b + lane;
      int v = e < e_count ? offs[e + 1] : 0;
      for (int d = 1; d < 32; d <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, v, d);
        if (lane >= d) v += u;
      }
      if (e < e_count) offs[e + 1] = v + carry;
      carry += __shfl_sync(0xffffffffu, v, 31);
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= e_count; e += blockDim.x) offsets[e] = offs[e];
  for (int e = threadIdx.x; e < e_count; e += blockDim.x) {
    int at = offs[e];
    for (int w = 0; w < kPlanWarps; ++w) {
      const int c = hist[w * e_count + e];
      hist[w * e_count + e] = at;              // becomes the warp's cursor
      at += c;
    }
  }
  __syncthreads();
  for (int base = p0; base < p1; base += 32) {
    const int p = base + lane;
    int e = p < p1 ? ids[p] - e_begin : -1;
    if (e >= e_count) e = -1;
    const unsigned same = __match_any_sync(0xffffffffu, e);
    if (e >= 0) {
      const int rank = __popc(same & ((1u << lane) - 1u));
      perm[mine[e] + rank] = p;
    }
    __syncwarp();
    if (e >= 0 && lane == __ffs(same) - 1) mine[e] += __popc(same);
    __syncwarp();
  }
}

// grid (T, ceil(H / 512)), block 256: out[t] = residual + sum_j w_j y[pair] (ascending expert id) + sigmoid(sg) * shared
constexpr int kCombineCols = 512;
__global__ void MoeCombineKernel(const __nv_bfloat16* __restrict__ y_pairs, const int* __restrict__ ids,
                                 const float* __restrict__ weights, const __nv_bfloat16* __restrict__ shared,
                                 const float* __restrict__ shared_gate, const __nv_bfloat16* __restrict__ residual,
                                 __nv_bfloat16* __restrict__ out, int H, int k) {
  const int t = blockIdx.x;
  __shared__ int order[kMaxK], sid[kMaxK];
  __shared__ float w[kMaxK], sw[kMaxK];
  if (threadIdx.x < k) {                     // one parallel read of the row's ids and weights; the sort runs on shared memory
    sid[threadIdx.x] = ids[t * k + threadIdx.x];
    sw[threadIdx.x] = weights[t * k + threadIdx.x];
  }
  __syncthreads();
  if (threadIdx.x < k) {                     // rank of slot j among the row's expert ids (ids of a row are distinct; ties by slot)
    const int mine = sid[threadIdx.x];
    int rank = 0;
    for (int j = 0; j < k; ++j) rank += (sid[j] < mine || (sid[j] == mine && j < static_cast<int>(threadIdx.x))) ? 1 : 0;
    order[rank] = threadIdx.x;
    w[rank] = sw[threadIdx.x];
  }
  __syncthreads();
  const float sg = shared_gate ? Sigmoid(shared_gate[t]) : 0.f;
  // grid.y splits the columns: a single row (decode) still spreads over several SMs
  const int c_lo = blockIdx.y * kCombineCols, c_hi = min(H, c_lo + kCombineCols);
  for (int c = c_lo + threadIdx.x * 2; c < c_hi; c += blockDim.x * 2) {
    float a0 = 0.f, a1 = 0.f;
    for (int j = 0; j < k; ++j) {
      const uint32_t v = *reinterpret_cast<const uint32_t*>(y_pairs + (static_cast<size_t>(t) * k + order[j]) * H + c);
      a0 = fmaf(w[j], BfLo(v), a0);
      a1 = fmaf(w[j], BfHi(v), a1);
    }
    if (shared) {
      const uint32_t s = *reinterpret_cast<const uint32_t*>(shared + static_cast<size_t>(t) * H + c);
      a0 = fmaf(sg, BfLo(s), a0);
      a1 = fmaf(sg, BfHi(s), a1);
    }
    if (residual) {
      const uint32_t r = *reinterpret_cast<const uint32_t*>(residual + static_cast<size_t>(t) * H + c);
      a0 += BfLo(r);
      a1 += BfHi(r);
    }
    *reinterpret_cast<uint32_t*>(out + static_cast<size_t>(t) * H + c) = PackBf16(a0, a1);
  }
}

}  // namespace
}  // namespace r4dxb

using namespace r4dxb;

extern "C" {

int r4dxb_moe_router(const float* logits, int T, int E, int k, int renorm, int* ids, float* weights, void* stream) {
  if (T < 1 || k < 1 || k > kMaxK || E > 1024 || E < k) return R4DXB_BAD_ARG;
  MoeRouterKernel<<<(T + 3) / 4, 128, 0, static_cast<cudaStream_t>(stream)>>>(logits, nullptr, T, E, k, renorm, 0, 1.0f, ids,
                                                                              weights);
  return FinishLaunch();
}

/* Sigmoid router: selection by sigmoid(logit) + bias (bias may be null), weights = unbiased sigmoids / (sum + 1e-6) * scale */
int r4dxb_moe_router_sigmoid(const float* logits, const float* bias, int T, int E, int k, int renorm, float scale, int* ids,
                             float* weights, void* stream) {
  if (T < 1 || k < 1 || k > kMaxK || E > 1024 || E < k) return R4DXB_BAD_ARG;
  MoeRouterKernel<<<(T + 3) / 4, 128, 0, static_cast<cudaStream_t>(stream)>>>(logits, bias, T, E, k, renorm, 1, scale, ids,
                                                                              weights);
  return FinishLaunch();
}

/* Router (mode 0 softmax, 1 sigmoid + bias) and routing plan of up to 8 rows in one launch */
int r4dxb_moe_route_plan(const float* logits, const float* bias, int T, int E, int k, int renorm, int mode, float scale, int* ids,
                         float* weights, int e_begin, int e_count, int* offsets, int* perm, void* stream) {
  if (T < 1 || T > 8 || k < 1 || k > kMaxK || E > 1024 || E < k || e_count < 1 || e_count > 8192 || (mode != 0 && mode != 1))
    return R4DXB_BAD_ARG;
  MoeRoutePlanKernel<<<1, 256, (e_count + 1) * sizeof(int), static_cast<cudaStream_t>(stream)>>>(
      logits, bias, T, E, k, renorm, mode, scale, ids, weights, e_begin, e_count, offsets, perm);
  return FinishLaunch();
}

/* offsets: [e_count + 1], perm: [npairs] pair indices sorted by expert (only experts in [e_begin, e_begin+e_count)) */
int r4dxb_moe_plan(const int* ids, int npairs, int E, int e_begin, int e_count, int* offsets, int* perm, void* stream) {
  if (npairs < 1 || e_count < 1 || e_count > 8192) return R4DXB_BAD_ARG;
  const size_t big = (static_cast<size_t>(kPlanWarps) * e_count + e_count + 1) * sizeof(int);
  if (npairs > 1024 && big <= 200 * 1024) {
    // many pairs: the serial placement of the small kernel would take milliseconds (2 ms for 40960 pairs)
    if (big > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(MoePlanParallelKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(big));
      if (e != cudaSuccess) return static_cast<int>(e);
    }
    MoePlanParallelKernel<<<1, kPlanWarps * 32, big, static_cast<cudaStream_t>(stream)>>>(ids, npairs, e_begin, e_count, offsets, perm);
    return FinishLaunch();
  }
  MoePlanKernel<<<1, 256, (e_count + 1) * sizeof(int), static_cast<cudaStream_t>(stream)>>>(ids, npairs, E, e_begin, e_count,
                                                                                             offsets, perm);
  return FinishLaunch();
}

int r4dxb_moe_combine(const void* y_pairs, const int* ids, const float* weights, const void* shared, const float* shared_gate,
                      const void* residual, void* out, int T, int H, int k, void* stream) {
  if (T < 1 || k < 1 || k > kMaxK || H % 2) return R4DXB_BAD_ARG;
  MoeCombineKernel<<<dim3(T, (H + kCombineCols - 1) / kCombineCols), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(y_pairs), ids, weights, static_cast<const __nv_bfloat16*>(shared), shared_gate,
      static_cast<const __nv_bfloat16*>(residual), static_cast<__nv_bfloat16*>(out), H, k);
  return FinishLaunch();
}

}  // extern "C"
