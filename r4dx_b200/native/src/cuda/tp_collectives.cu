// Small tensor-parallel collectives that run as ONE kernel over NVLink peer memory, with the same push protocol
// as the all-reduce inside the weight-streaming kernels (tp_push.cuh): every value travels with the call's
// sequence number in the same 8-byte store, the receiver polls (bounded, sticky status word), no library call
// and no host round trip.
//
//   all-reduce of T <= 8 bf16 rows in place   -- for blocks whose output is normalised before it joins the
//       residual stream (the product cannot fold the add into its epilogue), and the communicator's self-test.
//       Shares the receive buffer and the per-block call counters with the fused products, so both kinds of call
//       may be mixed freely as long as every rank issues the same sequence.
//   vocabulary-parallel greedy pick            -- every rank holds (best logit, token id) of its vocabulary
//       shard per row; all ranks end with the global best, ties to the lowest id (reference semantics:
//       src/model/tp/tp_vocab.h:38-75; the reference gathers the pairs on the host).
#include "tp_push.cuh"

namespace r4dxb {
namespace {

// grid N / 128, 256 threads: warp t reduces row t of the block's 128 columns
__global__ void __launch_bounds__(256) TpAllReduceRowsKernel(__nv_bfloat16* x, int T, int N, TpPush tp) {
  PdlEnter();
  const int nb = blockIdx.x, t = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = nb * 128 + lane * 4;
  const unsigned seq = tp.block_seq[nb] + 1;
  float o[4] = {0.f, 0.f, 0.f, 0.f};
  if (t < T) {
    const uint2 v = *reinterpret_cast<const uint2*>(x + static_cast<size_t>(t) * N + n);
    o[0] = BfLo(v.x); o[1] = BfHi(v.x); o[2] = BfLo(v.y); o[3] = BfHi(v.y);
    TpAllReduceRow(tp, seq, t, N, n, o);
    uint2 ov;
    ov.x = PackBf16(o[0], o[1]);
    ov.y = PackBf16(o[2], o[3]);
    *reinterpret_cast<uint2*>(x + static_cast<size_t>(t) * N + n) = ov;
  }
  __syncthreads();
  if (threadIdx.x == 0) tp.block_seq[nb] = seq;
}

struct ArgmaxArgs {
  float2* slots[kMaxWorld];   // slots[p]: rank p's buffer [2][world][8 rows][2] of (payload, seq) pairs, peer-mapped
  unsigned* seq;              // local call counter
  int* ids;                   // [T] in: this shard's best id (global numbering); out: the global best
  float* vals;                // [T] in / out
  int* status;
  int T, world, rank, spin_limit;
};

// one CTA, 256 threads: warp t merges row t, lane r talks to rank r
__global__ void __launch_bounds__(256) TpArgmaxMergeKernel(ArgmaxArgs a) {
  PdlEnter();
  const int t = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned seq = *a.seq + 1;
  const float fs = __uint_as_float(seq);
  const size_t half = static_cast<size_t>(seq & 1) * a.world * 8 * 2;
  if (t < a.T) {
    const float my_val = a.vals[t];
    const int my_id = a.ids[t];
    float val = -INFINITY;
    int id = 0x7fffffff;
    if (lane < a.world) {
      if (lane == a.rank) {
        val = my_val;
        id = my_id;
      } else {
        float4* dst = reinterpret_cast<float4*>(a.slots[lane] + half + (static_cast<size_t>(a.rank) * 8 + t) * 2);
        *dst = make_float4(my_val, fs, __int_as_float(my_id), fs);
        const float4* src = reinterpret_cast<const float4*>(a.slots[a.rank] + half + (static_cast<size_t>(lane) * 8 + t) * 2);
        bool got = false;
        const int limit = StatusNow(a.status) != 0 ? 1 : a.spin_limit;
        float4 p;
        for (int i = 0; i < limit; ++i) {
          p = __ldcv(src);
          if (__float_as_uint(p.y) == seq && __float_as_uint(p.w) == seq) { got = true; break; }
          if (i > 256) __nanosleep(32);
        }
        if (got) {
          val = p.x;
          id = __float_as_int(p.z);
        } else {
          atomicCAS(a.status, 0, 150 + lane);
        }
      }
    }
    // larger value wins; equal values: the lower id (NaN never wins: comparisons with it are false)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, val, o);
      const int oi = __shfl_xor_sync(0xffffffffu, id, o);
      if (ov > val || (ov == val && oi < id)) { val = ov; id = oi; }
    }
    if (lane == 0) {
      a.vals[t] = val;
      a.ids[t] = id == 0x7fffffff ? my_id : id;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) *a.seq = seq;
}

}  // namespace
}  // namespace r4dxb

using namespace r4dxb;

extern "C" {

/* In-place sum over the ranks of T <= 8 bf16 rows [T, N] (N % 128 == 0).  recv / block_seq / status: the buffers of
   r4dxb_trellis_gemv_allreduce (same layout, same counters). */
int r4dxb_tp_allreduce_rows(void* x, int T, int N, void* const* recv, void* block_seq, int* status, int world, int rank,
                            int spin_limit, void* stream) {
  if (T < 1 || T > 8 || N % 128 || world < 2 || world > kMaxWorld || rank < 0 || rank >= world) return R4DXB_BAD_ARG;
  TpPush tp = {};
  for (int p = 0; p < world; ++p) tp.recv[p] = static_cast<float2*>(recv[p]);
  tp.block_seq = static_cast<unsigned*>(block_seq);
  tp.status = status;
  tp.world = world;
  tp.rank = rank;
  tp.spin_limit = spin_limit;
  return LaunchPdl(TpAllReduceRowsKernel, dim3(N / 128), dim3(256), 0, static_cast<cudaStream_t>(stream),
                   static_cast<__nv_bfloat16*>(x), T, N, tp);
}

/* Global (max value, lowest id) per row over the ranks' vocabulary shards, in place on ids / vals.
   slots: `world` peer-mapped pointers to 2 * world * 8 * 2 float2 each, zero-initialised; seq: local u32 counter. */
int r4dxb_tp_argmax_merge(int* ids, float* vals, int T, void* const* slots, void* seq, int* status, int world, int rank,
                          int spin_limit, void* stream) {
  if (T < 1 || T > 8 || world < 2 || world > kMaxWorld || rank < 0 || rank >= world) return R4DXB_BAD_ARG;
  ArgmaxArgs a = {};
  for (int p = 0; p < world; ++p) a.slots[p] = static_cast<float2*>(slots[p]);
  a.seq = static_cast<unsigned*>(seq);
  a.ids = ids;
  a.vals = vals;
  a.status = status;
  a.T = T;
  a.world = world;
  a.rank = rank;
  a.spin_limit = spin_limit;
  return LaunchPdl(TpArgmaxMergeKernel, dim3(1), dim3(256), 0, static_cast<cudaStream_t>(stream), a);
}

}  // extern "C"
