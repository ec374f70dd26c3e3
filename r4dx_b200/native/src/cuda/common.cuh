// Shared device/host helpers for the sm_100a kernel library.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "r4dxb.h"

namespace r4dxb {

// Every launcher bumps this host counter (one per kernel launch), so a caller can report how many
// kernels of this library ran in a region (reference keeps the same kind of counter:
// src/kernels/include/r4dx/kernels/kernels.h:666-680).
extern unsigned long long g_launch_count;

inline int FinishLaunch() {
  ++g_launch_count;
  return static_cast<int>(cudaGetLastError());
}

// Programmatic dependent launch for the small kernels between the weight-streaming products of a decode step: the
// kernel is launched with the stream-serialization attribute, lets its own successor begin launching right away
// and waits on the device for its predecessor before it touches any buffer (PdlEnter is the first statement of
// such a kernel).  What this hides is launch latency, a few microseconds at each of the ~500 kernel boundaries of a step.
extern bool g_use_pdl;

__device__ __forceinline__ void PdlEnter() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

template <typename... KArgs, typename... Args>
inline int LaunchPdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_use_pdl ? 1 : 0;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, args...);
  ++g_launch_count;
  return static_cast<int>(e);
}

// Status word of a communicator, read past the caches: non-zero means an earlier bounded wait ran out, and
// every later wait gives up at once (the failure is sticky until the host has recovered and cleared it).
__device__ __forceinline__ int StatusNow(const int* status) {
  int v;
  asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(status) : "memory");
  return v;
}

__device__ __forceinline__ float WarpSum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float WarpMax(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum; `red` needs 32 floats of shared memory. All threads get the result.
__device__ __forceinline__ float BlockSum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = WarpSum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = (lane < nw) ? red[lane] : 0.0f;
  r = WarpSum(r);
  return r;
}

__device__ __forceinline__ float Bf16Bits(uint16_t b) { return __uint_as_float(static_cast<uint32_t>(b) << 16); }
__device__ __forceinline__ float BfLo(uint32_t p) { return __uint_as_float(p << 16); }
__device__ __forceinline__ float BfHi(uint32_t p) { return __uint_as_float(p & 0xFFFF0000u); }
__device__ __forceinline__ uint32_t PackBf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float Sigmoid(float x) { return 1.0f / (1.0f + __expf(-x)); }
__device__ __forceinline__ float Silu(float x) { return x / (1.0f + __expf(-x)); }
__device__ __forceinline__ float GeluTanh(float x) {
  return 0.5f * x * (1.0f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
}
// gate activation of a gated MLP: 0 = SiLU (SwiGLU), 1 = tanh-GELU (GeGLU)
__device__ __forceinline__ float GateAct(float x, int act) { return act == 0 ? Silu(x) : GeluTanh(x); }

// 128-point Sylvester FWHT held by one warp: lane l owns elements 4l .. 4l+3 (unnormalised).
__device__ __forceinline__ void WarpFwht128(float (&v)[4]) {
  const int lane = threadIdx.x & 31;
  {
    const float a = v[0] + v[1], b = v[0] - v[1], c = v[2] + v[3], d = v[2] - v[3];
    v[0] = a + c; v[1] = b + d; v[2] = a - c; v[3] = b - d;
  }
#pragma unroll
  for (int m = 1; m < 32; m <<= 1) {
    const bool upper = lane & m;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float o = __shfl_xor_sync(0xffffffffu, v[i], m);
      v[i] = upper ? (o - v[i]) : (v[i] + o);
    }
  }
}

}  // namespace r4dxb
