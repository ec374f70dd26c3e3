// Tensor-parallel epilogue shared by the weight-streaming kernels: all-reduce by one-shot push over NVLink
// peer memory.
//
// Each value travels as an 8-byte (fp32 value, sequence number) pair, so data and "ready" flag arrive in one
// store and no fence or separate flag round is needed; the receiver polls the pairs it needs (bounded).  Every
// rank sums the world's partials in rank order, so all ranks hold identical bits.  Receive slots are
// double-buffered by the parity of a per-block call counter kept in device memory (a captured graph can be
// replayed).
//
// Failure is sticky: the first wait that runs out writes 100 + the silent rank into the status word, and every
// later call that finds the word non-zero skips its polls (it still pushes and still advances its counters), so
// one lost rank costs one timeout, not one per collective, until the host has run its recovery and cleared the
// word (reference: src/kernels/src/r4dx_tp_kernels.hip:109-125 keeps an abort word with the same rule).
#pragma once
#include "common.cuh"

namespace r4dxb {

constexpr int kMaxWorld = 8;

struct TpPush {
  float2* recv[kMaxWorld];         // recv[p]: rank p's buffer [2][world][8][N] of (value, seq) pairs, peer-mapped
  unsigned* block_seq;             // local [N/128] call counters
  int* status;                     // local: set to 100 + rank when that rank did not answer in time (sticky)
  int world, rank, spin_limit;
  // expert-parallel output (grouped mode): row gp = (rank gp / ep_P, pair gp % ep_P) goes to that rank's
  // combine buffer ep_y[rank] ([2][ep_P][N] bf16) and bumps ep_cnt[rank] ([2][ep_P]) once per 128-column block
  __nv_bfloat16* ep_y[kMaxWorld];
  unsigned* ep_cnt[kMaxWorld];
  int ep_P;
};

__device__ __forceinline__ int TpStatusNow(const int* status) { return StatusNow(status); }

// One warp finishes row t of a 128-column block: lane holds columns n .. n+3 of its partial in o[], call number
// `seq` (block_seq[nb] + 1).  Pushes to every peer, then sums all ranks' partials in rank order into o[].
// On a timeout (or when the status word was already set) o[] keeps the local partial.
__device__ __forceinline__ void TpAllReduceRow(const TpPush& tp, unsigned seq, int t, int N, int n, float (&o)[4]) {
  const size_t slot_pairs = static_cast<size_t>(tp.world) * 8 * N;
  const size_t my_off = (seq & 1) * slot_pairs + (static_cast<size_t>(tp.rank) * 8 + t) * N + n;
  const float fs = __uint_as_float(seq);
  for (int p = 0; p < tp.world; ++p) {
    if (p == tp.rank) continue;
    float4* dst = reinterpret_cast<float4*>(tp.recv[p] + my_off);
    dst[0] = make_float4(o[0], fs, o[1], fs);
    dst[1] = make_float4(o[2], fs, o[3], fs);
  }
  if (TpStatusNow(tp.status) != 0) return;       // sticky abort: do not wait for anybody
  float a4[4] = {0.f, 0.f, 0.f, 0.f};
  const float2* mine = tp.recv[tp.rank] + (seq & 1) * slot_pairs;
  for (int r = 0; r < tp.world; ++r) {           // rank order, identical on every rank
    if (r == tp.rank) {
      a4[0] += o[0]; a4[1] += o[1]; a4[2] += o[2]; a4[3] += o[3];
      continue;
    }
    const float4* src = reinterpret_cast<const float4*>(mine + (static_cast<size_t>(r) * 8 + t) * N + n);
    float4 p0, p1;
    bool got = false;
    for (int i = 0; i < tp.spin_limit; ++i) {
      p0 = __ldcv(src);
      p1 = __ldcv(src + 1);
      if (__float_as_uint(p0.y) == seq && __float_as_uint(p0.w) == seq && __float_as_uint(p1.y) == seq &&
          __float_as_uint(p1.w) == seq) { got = true; break; }
      if (i > 256) {
        __nanosleep(32);
        if ((i & 1023) == 0 && TpStatusNow(tp.status) != 0) break;     // another warp or kernel already gave up
      }
    }
    if (!got) {
      atomicCAS(tp.status, 0, 100 + r);          // first failure wins and stays
      return;
    }
    a4[0] += p0.x; a4[1] += p0.z; a4[2] += p1.x; a4[3] += p1.z;
  }
  o[0] = a4[0]; o[1] = a4[1]; o[2] = a4[2]; o[3] = a4[3];
}

}  // namespace r4dxb
