// Shared device/host helpers for the sm_100a kernels.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace q38 {

// ---- error reporting -------------------------------------------------------------------------------------
// Kernels never trap and never spin without bound.  A wait that runs out (or a failed self-check) stores a
// non-zero code into a device word that the host reads after the stream is synchronised.
enum ErrorCode : int {
  ERR_NONE = 0,
  ERR_TMA_WAIT = 1,       // consumer gave up waiting for a TMA stage
  ERR_MMA_WAIT = 2,       // producer gave up waiting for a stage to be released by the tensor core
  ERR_EPILOGUE_WAIT = 3,  // epilogue gave up waiting for the accumulator
  ERR_PEER_WAIT = 4,      // a flag that a peer GPU writes did not arrive in time
  ERR_BOUNDS = 5,         // an index self-check failed; the access was skipped
};

__device__ __forceinline__ void report_error(int* flag, int code) {
  if (flag != nullptr) atomicCAS(flag, 0, code);
}

// ---- small numeric helpers --------------------------------------------------------------------------------
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float siluf_(float x) { return x * sigmoidf_(x); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum; `scratch` holds at least 32 floats of shared memory.  All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < nwarp) ? scratch[lane] : 0.f;
  return warp_sum(t);
}

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

constexpr int kNumSMs = 148;

}  // namespace q38
