// Tail-biting Viterbi encoder for trellis tiles on the GPU: one CTA of 1024 threads per 16x16 tile.
//
// The code is a sliding 16-bit window over a ring of 256 * KB bits; position p's value depends on state_p and
// state_{p+1} = ((state_p << KB) | new bits) & 0xFFFF.  With T = 2^(16-KB) and cost_p[s] the best squared error of
// any path ending in state s at position p, only
//   M_p[t] = min_h cost_{p-1}[h T + t]           (the KB bits h that fall off the top; argmin kept as back pointer)
// has to persist, because cost_p[s] = M_p[s >> KB] + (x_p - code(s))^2.  Two M arrays (T floats each) live in shared
// memory, the code value is recomputed from the state (three integer instructions and one fp16 FMA), the back
// pointers (256 x T bytes per tile) go to a per-CTA scratch in global memory, and one thread walks them back.
// Tail biting as on the host (native/src/host/trellis.cpp): a first pass over the tile rotated by half a ring picks
// the overlap bits at the seam, a second pass pins both ends to them
// (reference: tools/reference/trellis_viterbi.hip:1-80 is the reference's GPU encoder).
#include "common.cuh"
#include "r4dxb_trellis.h"

namespace r4dxb {
namespace {

__device__ __forceinline__ float CodeValue(uint32_t s) {
  const uint32_t h = __dp4a(s * R4DXB_TRELLIS_MUL, 0x01010101u, 0x6400u);
  const __half v = __hfma(__ushort_as_half(static_cast<unsigned short>(h)), __ushort_as_half(R4DXB_TRELLIS_SCALE_F16),
                          __ushort_as_half(R4DXB_TRELLIS_BIAS_F16));
  return __half2float(v);
}

template <int KB>
struct EncSmem {
  static constexpr int T = 1 << (16 - KB);
  float m[2][T];
  float w[256];
  float wrot[256];
  unsigned short states[256];
  float red_v[32];
  int red_s[32];
  int best;
  float best_cost;
};

// One pass; leaves states[] and best_cost in shared memory.  overlap < 0: free ends.
template <int KB>
__device__ void ViterbiPass(EncSmem<KB>& sm, const float* x, int overlap, uint8_t* __restrict__ bp) {
  constexpr int T = 1 << (16 - KB), NH = 1 << KB, PER = T / 1024;
  const int tid = threadIdx.x;
  const float inf = INFINITY;
  for (int p = 1; p < 256; ++p) {
    const float* mp = sm.m[(p - 1) & 1];
    float* mc = sm.m[p & 1];
    const float xv = x[p - 1];
    uint32_t packed[(PER + 3) / 4] = {};
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int t = tid * PER + j;
      float best = inf;
      int bh = 0;
#pragma unroll 4
      for (int h = 0; h < NH; ++h) {
        const uint32_t s = static_cast<uint32_t>(h) * T + t;
        const float d = xv - CodeValue(s);
        float c;
        if (p == 1) c = (overlap < 0 || static_cast<int>(s >> KB) == overlap) ? d * d : inf;
        else c = mp[s >> KB] + d * d;
        if (c < best) { best = c; bh = h; }
      }
      mc[t] = best;
      packed[j / 4] |= static_cast<uint32_t>(bh) << (8 * (j & 3));
    }
    uint8_t* row = bp + static_cast<size_t>(p) * T + tid * PER;
    if (PER >= 4) {
#pragma unroll
      for (int q = 0; q < (PER + 3) / 4; ++q) reinterpret_cast<uint32_t*>(row)[q] = packed[q];
    } else {
      *reinterpret_cast<unsigned short*>(row) = static_cast<unsigned short>(packed[0]);      // PER == 2
    }
    __syncthreads();
  }
  // best end state
  const float* ml = sm.m[255 & 1];
  const float xl = x[255];
  if (overlap < 0) {
    float best = inf;
    int bs = 0;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int t = tid * PER + j;
      for (int b = 0; b < NH; ++b) {
        const uint32_t s = (static_cast<uint32_t>(t) << KB) + b;
        const float d = xl - CodeValue(s);
        const float c = ml[t] + d * d;
        if (c < best) { best = c; bs = static_cast<int>(s); }
      }
    }
    // block argmin, ties to the lower state (threads own ascending state ranges, so lower lane / warp wins ties)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_down_sync(0xffffffffu, best, o);
      const int os = __shfl_down_sync(0xffffffffu, bs, o);
      if (ov < best || (ov == best && os < bs)) { best = ov; bs = os; }
    }
    if ((tid & 31) == 0) { sm.red_v[tid >> 5] = best; sm.red_s[tid >> 5] = bs; }
    __syncthreads();
    if (tid == 0) {
      float bv = sm.red_v[0];
      int bi = sm.red_s[0];
      for (int i = 1; i < 32; ++i)
        if (sm.red_v[i] < bv || (sm.red_v[i] == bv && sm.red_s[i] < bi)) { bv = sm.red_v[i]; bi = sm.red_s[i]; }
      sm.best = bi;
      sm.best_cost = bv;
    }
  } else if (tid == 0) {
    float bv = inf;
    int bi = 0;
    for (int h = 0; h < NH; ++h) {
      const uint32_t s = static_cast<uint32_t>(h) * T + overlap;
      const float d = xl - CodeValue(s);
      const float c = ml[s >> KB] + d * d;
      if (c < bv) { bv = c; bi = static_cast<int>(s); }
    }
    sm.best = bi;
    sm.best_cost = bv;
  }
  __syncthreads();
  if (tid == 0) {
    int s = sm.best;
    for (int p = 255; p >= 1; --p) {
      sm.states[p] = static_cast<unsigned short>(s);
      const int t = s >> KB;
      s = (static_cast<int>(bp[static_cast<size_t>(p) * T + t]) << (16 - KB)) | t;
    }
    sm.states[0] = static_cast<unsigned short>(s);
  }
  __syncthreads();
}

template <int KB>
__global__ void __launch_bounds__(1024, 1) TrellisEncodeKernel(const float* __restrict__ vals, int ntiles,
                                                               uint32_t* __restrict__ words, float* __restrict__ err,
                                                               uint8_t* __restrict__ bp_all) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  EncSmem<KB>& sm = *reinterpret_cast<EncSmem<KB>*>(smem_raw);
  constexpr int T = 1 << (16 - KB);
  uint8_t* bp = bp_all + static_cast<size_t>(blockIdx.x) * 256 * T;
  const int tid = threadIdx.x;
  for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    if (tid < 256) {
      sm.w[tid] = vals[static_cast<size_t>(tile) * 256 + tid];
      sm.wrot[tid] = vals[static_cast<size_t>(tile) * 256 + ((tid + 128) & 255)];
    }
    __syncthreads();
    ViterbiPass<KB>(sm, sm.wrot, -1, bp);
    // rotated position 127 is original position 255: its low bits are the ring's wrap-around overlap
    const int overlap = sm.states[127] & (T - 1);
    __syncthreads();
    ViterbiPass<KB>(sm, sm.w, overlap, bp);
    if (tid < 8 * KB) {
      uint32_t wv = 0;
      for (int i = 0; i < 32; ++i) {
        const int pos = 32 * tid + i, p = pos / KB, b = pos % KB;
        wv |= ((static_cast<uint32_t>(sm.states[p]) >> (KB - 1 - b)) & 1u) << (31 - i);
      }
      words[static_cast<size_t>(tile) * 8 * KB + tid] = wv;
    }
    if (tid == 0) err[tile] = sm.best_cost;
    __syncthreads();
  }
}

template <int KB>
int LaunchEncode(const float* vals, int ntiles, uint32_t* words, float* err, uint8_t* bp, int ctas, cudaStream_t s) {
  auto kern = TrellisEncodeKernel<KB>;
  const int smem = static_cast<int>(sizeof(EncSmem<KB>));
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return static_cast<int>(e);
  kern<<<ctas, 1024, smem, s>>>(vals, ntiles, words, err, bp);
  return FinishLaunch();
}

}  // namespace
}  // namespace r4dxb

using namespace r4dxb;

extern "C" {

/* bytes of back-pointer scratch for `ctas` concurrent tiles */
long long r4dxb_trellis_encode_scratch_bytes(int kb, int ctas) { return 256LL * (1LL << (16 - kb)) * ctas; }

/* vals: [ntiles][256] fp32 in tile position order (unit variance); words: [ntiles][8 kb]; err: [ntiles] squared errors */
int r4dxb_trellis_encode_tiles(const float* vals, int ntiles, int kb, void* words, float* err, void* scratch, int ctas,
                               void* stream) {
  if (ntiles < 1 || ctas < 1) return R4DXB_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint32_t* w = static_cast<uint32_t*>(words);
  uint8_t* bp = static_cast<uint8_t*>(scratch);
  if (ctas > ntiles) ctas = ntiles;
  switch (kb) {
    case 3: return LaunchEncode<3>(vals, ntiles, w, err, bp, ctas, s);
    case 4: return LaunchEncode<4>(vals, ntiles, w, err, bp, ctas, s);
    case 5: return LaunchEncode<5>(vals, ntiles, w, err, bp, ctas, s);
    default: return R4DXB_BAD_ARG;
  }
}

}  // extern "C"
