// Expert-parallel all-to-all around the grouped expert GEMV, over NVLink peer memory.
//
// Tokens are sharded by rank (each rank decodes its own sequences), experts are sharded by rank.
// Per MoE layer call:
//   dispatch (this file)  every rank routes its tokens, broadcasts the routing table to all ranks as
//                         (expert id, sequence) pairs, and stores each token row straight into the
//                         receive buffer of the rank that owns the chosen expert, then releases a
//                         per-row flag at system scope;
//   plan (this file)      every rank polls the routing tables and builds the per-expert row lists
//                         of the pairs that chose one of its experts (global pair index = source
//                         rank x pairs-per-rank + pair);
//   grouped gate_up / down (trellis_gemv.cu, grouped mode)
//                         the gate_up prologue waits for the row flags it needs and reads the rows
//                         from the receive buffer; the down epilogue stores each output block into
//                         the combine buffer of the rank that owns the token and bumps that row's
//                         arrival counter;
//   combine (this file)   the owner waits for all blocks of its k rows per token, sums them in
//                         ascending expert id with the router weights, adds the shared expert and
//                         the residual.
// Every wait is bounded (poll limit -> status word, the kernel returns).  Buffers are double-
// buffered by the parity of a device-resident call counter, so a CUDA graph can replay the layer.
// The reference has no expert parallelism (its MoE models split layers or halve every expert:
// reference src/model/qwen35moe_config.h:62-70); this is new.
#include "common.cuh"

namespace r4dxb {
namespace {

constexpr int kMaxWorld = 8;
constexpr int kMaxK = 16;

__device__ __forceinline__ void StoreReleaseSys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned LoadAcquireSys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

struct EpPeers {
  uint2* meta[kMaxWorld];          // [2][W][P] (expert id, seq)
  __nv_bfloat16* xrecv[kMaxWorld]; // [2][W][P][H]
  unsigned* xflag[kMaxWorld];      // [2][W][P]
};

// grid = pairs (T*k), block 128: one CTA moves one (token, slot) pair
__global__ void EpDispatchKernel(EpPeers peers, const __nv_bfloat16* __restrict__ h, const int* __restrict__ ids,
                                 const unsigned* __restrict__ seq_ptr, int T, int k, int H, int P, int world, int rank,
                                 int experts_per_rank) {
  const int pair = blockIdx.x;
  const unsigned seq = *seq_ptr + 1;
  const int par = seq & 1;
  const int valid = pair < T * k;
  const int e = valid ? ids[pair] : -1;
  // routing table entry to every rank (also the unused tail of the table, as "no expert")
  if (threadIdx.x < world) {
    uint2* dst = peers.meta[threadIdx.x] + (static_cast<size_t>(par) * world + rank) * P + pair;
    *dst = make_uint2(static_cast<unsigned>(e), seq);
  }
  if (!valid) return;
  const int dest = e / experts_per_rank;
  __nv_bfloat16* row = peers.xrecv[dest] + ((static_cast<size_t>(par) * world + rank) * P + pair) * H;
  const uint4* src = reinterpret_cast<const uint4*>(h + static_cast<size_t>(pair / k) * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) reinterpret_cast<uint4*>(row)[i] = src[i];
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) StoreReleaseSys(peers.xflag[dest] + (static_cast<size_t>(par) * world + rank) * P + pair, seq);
}

// single CTA: waits for the routing tables of all ranks, then a stable counting sort of the pairs that
// chose a local expert
__global__ void EpPlanKernel(const uint2* __restrict__ meta, const unsigned* __restrict__ seq_ptr, int world, int P,
                             int e_begin, int e_count, int* __restrict__ offsets, int* __restrict__ perm,
                             int spin_limit, int* __restrict__ status) {
  extern __shared__ int sm[];
  int* cnt = sm;                         // [e_count + 1]
  int* exp_of = sm + e_count + 1;        // [world * P]
  const unsigned seq = *seq_ptr + 1;
  const int par = seq & 1;
  const int total = world * P;
  for (int e = threadIdx.x; e <= e_count; e += blockDim.x) cnt[e] = 0;
  for (int g = threadIdx.x; g < total; g += blockDim.x) {
    const volatile uint2* p = reinterpret_cast<const volatile uint2*>(meta + static_cast<size_t>(par) * total + g);
    int e = -1;
    bool got = false;
    // sticky: once any wait of this communicator has run out nobody waits again until the host clears the word
    const int limit = StatusNow(status) != 0 ? 1 : spin_limit;
    for (int i = 0; i < limit; ++i) {
      const unsigned flag = p->y;
      if (flag == seq) { e = static_cast<int>(p->x); got = true; break; }
      if (i > 64) __nanosleep(32);
    }
    if (!got) atomicCAS(status, 0, 200 + g / P);
    exp_of[g] = e;
  }
  __syncthreads();
  for (int g = threadIdx.x; g < total; g += blockDim.x) {
    const int e = exp_of[g] - e_begin;
    if (exp_of[g] >= 0 && e >= 0 && e < e_count) atomicAdd(&cnt[e + 1], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int e = 0; e < e_count; ++e) cnt[e + 1] += cnt[e];
    for (int e = 0; e <= e_count; ++e) offsets[e] = cnt[e];
    for (int g = 0; g < total; ++g) {
      const int e = exp_of[g] - e_begin;
      if (exp_of[g] >= 0 && e >= 0 && e < e_count) perm[cnt[e]++] = g;
    }
  }
}

// grid T, block 256.  comb: [2][P][H] rows produced by the expert owners; ccount: [2][P] arrival counters
// (blocks_per_row arrivals complete a row); the owner resets the counters it consumed.
__global__ void EpCombineKernel(const __nv_bfloat16* __restrict__ comb, unsigned* __restrict__ ccount,
                                unsigned* __restrict__ seq_ptr, const int* __restrict__ ids, const float* __restrict__ weights,
                                const __nv_bfloat16* __restrict__ shared, const float* __restrict__ shared_gate,
                                __nv_bfloat16* __restrict__ x, int T, int H, int k, int P, int blocks_per_row, int spin_limit,
                                int* __restrict__ status) {
  const int t = blockIdx.x;
  const unsigned seq = *seq_ptr + 1;
  const int par = seq & 1;
  __shared__ int order[kMaxK];
  __shared__ float w[kMaxK];
  __shared__ int fail;
  if (threadIdx.x == 0) fail = 0;
  __syncthreads();
  if (threadIdx.x < k) {
    unsigned* c = ccount + static_cast<size_t>(par) * P + t * k + threadIdx.x;
    bool got = false;
    const int limit = StatusNow(status) != 0 ? 1 : spin_limit;
    for (int i = 0; i < limit; ++i) {
      if (LoadAcquireSys(c) >= static_cast<unsigned>(blocks_per_row)) { got = true; break; }
      if (i > 64) __nanosleep(32);
    }
    if (!got) { fail = 1; atomicCAS(status, 0, 300 + t); }
    *c = 0;                                  // ready for the call after next
  }
  if (threadIdx.x == 0) {
    int idx[kMaxK];
    for (int j = 0; j < k; ++j) idx[j] = j;
    for (int a = 1; a < k; ++a) {
      const int v = idx[a];
      int b = a - 1;
      while (b >= 0 && ids[t * k + idx[b]] > ids[t * k + v]) { idx[b + 1] = idx[b]; --b; }
      idx[b + 1] = v;
    }
    for (int j = 0; j < k; ++j) { order[j] = idx[j]; w[j] = weights[t * k + idx[j]]; }
  }
  __syncthreads();
  const float sg = shared_gate ? Sigmoid(shared_gate[t]) : 0.f;
  const __nv_bfloat16* rows = comb + (static_cast<size_t>(par) * P + t * k) * H;
  for (int c = threadIdx.x * 2; c < H; c += blockDim.x * 2) {
    float a0 = 0.f, a1 = 0.f;
    if (!fail) {
      for (int j = 0; j < k; ++j) {
        const uint32_t v = __ldcg(reinterpret_cast<const uint32_t*>(rows + static_cast<size_t>(order[j]) * H + c));
        a0 = fmaf(w[j], BfLo(v), a0);
        a1 = fmaf(w[j], BfHi(v), a1);
      }
    }
    if (shared) {
      const uint32_t s = *reinterpret_cast<const uint32_t*>(shared + static_cast<size_t>(t) * H + c);
      a0 = fmaf(sg, BfLo(s), a0);
      a1 = fmaf(sg, BfHi(s), a1);
    }
    const uint32_t r = *reinterpret_cast<const uint32_t*>(x + static_cast<size_t>(t) * H + c);
    *reinterpret_cast<uint32_t*>(x + static_cast<size_t>(t) * H + c) = PackBf16(a0 + BfLo(r), a1 + BfHi(r));
  }
}

__global__ void EpAdvanceKernel(unsigned* seq_ptr) { *seq_ptr += 1; }

}  // namespace
}  // namespace r4dxb

using namespace r4dxb;

extern "C" {

/* meta / xrecv / xflag: `world` peer-mapped pointers each.  P = pairs per rank (max rows x k). */
int r4dxb_ep_dispatch(void* const* meta, void* const* xrecv, void* const* xflag, const void* h, const int* ids,
                      const void* seq_ptr, int T, int k, int H, int P, int world, int rank, int experts_per_rank, void* stream) {
  if (world < 1 || world > kMaxWorld || T * k > P || H % 8) return R4DXB_BAD_ARG;
  EpPeers p;
  for (int i = 0; i < world; ++i) {
    p.meta[i] = static_cast<uint2*>(meta[i]);
    p.xrecv[i] = static_cast<__nv_bfloat16*>(xrecv[i]);
    p.xflag[i] = static_cast<unsigned*>(xflag[i]);
  }
  EpDispatchKernel<<<P, 128, 0, static_cast<cudaStream_t>(stream)>>>(p, static_cast<const __nv_bfloat16*>(h), ids,
                                                                      static_cast<const unsigned*>(seq_ptr), T, k, H, P, world, rank,
                                                                      experts_per_rank);
  return FinishLaunch();
}

int r4dxb_ep_plan(const void* meta_local, const void* seq_ptr, int world, int P, int e_begin, int e_count, int* offsets,
                  int* perm, int spin_limit, int* status, void* stream) {
  const size_t smem = (static_cast<size_t>(e_count) + 1 + static_cast<size_t>(world) * P) * sizeof(int);
  if (smem > 200 * 1024) return R4DXB_TOO_LARGE;
  if (smem > 48 * 1024) cudaFuncSetAttribute(EpPlanKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  EpPlanKernel<<<1, 512, smem, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint2*>(meta_local),
                                                                     static_cast<const unsigned*>(seq_ptr), world, P, e_begin,
                                                                     e_count, offsets, perm, spin_limit, status);
  return FinishLaunch();
}

int r4dxb_ep_combine(const void* comb, void* ccount, void* seq_ptr, const int* ids, const float* weights, const void* shared,
                     const float* shared_gate, void* x, int T, int H, int k, int P, int blocks_per_row, int spin_limit,
                     int* status, void* stream) {
  if (T < 1 || k > kMaxK || H % 2) return R4DXB_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  EpCombineKernel<<<T, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(comb), static_cast<unsigned*>(ccount),
                                    static_cast<unsigned*>(seq_ptr), ids, weights, static_cast<const __nv_bfloat16*>(shared),
                                    shared_gate, static_cast<__nv_bfloat16*>(x), T, H, k, P, blocks_per_row, spin_limit, status);
  int e = FinishLaunch();
  if (e) return e;
  EpAdvanceKernel<<<1, 1, 0, s>>>(static_cast<unsigned*>(seq_ptr));
  return FinishLaunch();
}

}  // extern "C"
