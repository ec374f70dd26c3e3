// Tensor-parallel prefill, the part after the row-parallel product's reduce-scatter epilogue
// (trellis_gemm.cu, RsArgs):
//
//   reduce + push : the owner of a block of token rows waits (bounded) until every rank's partial rows have
//                   arrived, sums them in rank order in fp32 on top of the residual row, and stores the new
//                   residual row into EVERY rank's copy of the residual stream over NVLink peer mappings -
//                   the all-gather half of the all-reduce, issued by the kernel that produced the rows;
//   wait          : a one-CTA kernel that lets the stream pass once all rows of the call have been pushed
//                   to this rank (the next kernel reads the gathered residual stream).
// Every wait has an iteration limit; when it runs out the kernel records a status code and carries on, so a
// missing peer ends in an error the host reads, never in a hang.
#include "common.cuh"

namespace r4dxb {
namespace {

// Sticky: with the status word already set (an earlier wait of this communicator ran out) one look is all a
// wait gets, so a lost rank costs one timeout and not one per collective.
__device__ __forceinline__ bool WaitCounter(const unsigned* p, unsigned target, int spin_limit, const int* status) {
  if (StatusNow(status) != 0) spin_limit = 1;
  for (int i = 0; i < spin_limit; ++i) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    if (static_cast<int>(v - target) >= 0) return true;
    if (i > 64) __nanosleep(64);
  }
  return false;
}

struct PushArgs {
  __nv_bfloat16* x[8];          // peer-mapped residual streams [T, H], indexed by rank
  unsigned* xflag[8];           // peer-mapped "rows pushed" counters, indexed by rank
  const __nv_bfloat16* recv;    // this rank's receive buffer [world][rows_per_rank][H]
  const unsigned* cnt;          // this rank's arrival counter
  unsigned target;
  int world, rank, rows_per_rank, rows_own, H, spin_limit;
  int* status;
};

// grid rows_own, 256 threads: one owned token row per CTA
__global__ void __launch_bounds__(256) TpReducePushKernel(PushArgs a) {
  __shared__ int ok;
  if (threadIdx.x == 0) {
    ok = WaitCounter(a.cnt, a.target, a.spin_limit, a.status) ? 1 : 0;
    if (!ok) atomicCAS(a.status, 0, 200 + a.rank);
  }
  __syncthreads();
  const int tl = blockIdx.x;
  const size_t t = static_cast<size_t>(a.rank) * a.rows_per_rank + tl;
  const int H8 = a.H / 8;
  for (int c = threadIdx.x; c < H8; c += blockDim.x) {
    const uint4 xv = *reinterpret_cast<const uint4*>(a.x[a.rank] + t * a.H + c * 8);
    float acc[8] = {BfLo(xv.x), BfHi(xv.x), BfLo(xv.y), BfHi(xv.y), BfLo(xv.z), BfHi(xv.z), BfLo(xv.w), BfHi(xv.w)};
    for (int s = 0; s < a.world; ++s) {        // rank order: every owner adds in the same order
      // peers wrote these rows: read them from L2, not from a stale L1 line of an earlier call
      const uint4 v = __ldcg(reinterpret_cast<const uint4*>(a.recv + (static_cast<size_t>(s) * a.rows_per_rank + tl) * a.H + c * 8));
      acc[0] += BfLo(v.x); acc[1] += BfHi(v.x); acc[2] += BfLo(v.y); acc[3] += BfHi(v.y);
      acc[4] += BfLo(v.z); acc[5] += BfHi(v.z); acc[6] += BfLo(v.w); acc[7] += BfHi(v.w);
    }
    uint4 o;
    o.x = PackBf16(acc[0], acc[1]); o.y = PackBf16(acc[2], acc[3]); o.z = PackBf16(acc[4], acc[5]); o.w = PackBf16(acc[6], acc[7]);
    for (int p = 0; p < a.world; ++p) *reinterpret_cast<uint4*>(a.x[p] + t * a.H + c * 8) = o;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < a.world) atomicAdd_system(a.xflag[threadIdx.x], 1u);
}

__global__ void TpWaitKernel(const unsigned* flag, unsigned target, int spin_limit, int code, int* status) {
  if (threadIdx.x == 0 && !WaitCounter(flag, target, spin_limit, status)) atomicCAS(status, 0, code);
}

}  // namespace
}  // namespace r4dxb

using namespace r4dxb;

extern "C" {

/* x, xflag: `world` peer-mapped pointers; recv, cnt: this rank's own buffers.  target: the value cnt must reach. */
int r4dxb_tp_reduce_push(void* const* x, void* const* xflag, const void* recv, const void* cnt, unsigned target, int world, int rank,
                         int rows_per_rank, int rows_own, int H, int spin_limit, int* status, void* stream) {
  if (world < 2 || world > 8 || rank < 0 || rank >= world || H % 8 || rows_own < 0 || rows_own > rows_per_rank) return R4DXB_BAD_ARG;
  if (rows_own == 0) return 0;
  PushArgs a;
  for (int p = 0; p < world; ++p) {
    a.x[p] = static_cast<__nv_bfloat16*>(x[p]);
    a.xflag[p] = static_cast<unsigned*>(xflag[p]);
  }
  a.recv = static_cast<const __nv_bfloat16*>(recv);
  a.cnt = static_cast<const unsigned*>(cnt);
  a.target = target;
  a.world = world; a.rank = rank; a.rows_per_rank = rows_per_rank; a.rows_own = rows_own; a.H = H; a.spin_limit = spin_limit;
  a.status = status;
  TpReducePushKernel<<<rows_own, 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return FinishLaunch();
}

int r4dxb_tp_wait(const void* flag, unsigned target, int spin_limit, int code, int* status, void* stream) {
  TpWaitKernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const unsigned*>(flag), target, spin_limit, code, status);
  return FinishLaunch();
}

}  // extern "C"
