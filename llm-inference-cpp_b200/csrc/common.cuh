// Shared device helpers for the sm_100a kernels of this library.
//
// Conventions every kernel here follows:
//  * storage type T is float or __nv_bfloat16; arithmetic that decides a result
//    (sums of squares, softmax, rotation angles, residual sums, accumulators) is fp32;
//  * launchers are extern "C", take raw device pointers, sizes and a stream, launch on
//    that stream, allocate nothing, and return 0 or a negative LLMI_ERR_* code;
//  * a size a kernel cannot take is refused by its launcher, never mis-computed.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define LLMI_DTYPE_F32 0
#define LLMI_DTYPE_BF16 1

#define LLMI_OK 0
#define LLMI_ERR_BAD_DTYPE (-1)
#define LLMI_ERR_BAD_SIZE (-2)
#define LLMI_ERR_LAUNCH (-3)
#define LLMI_ERR_ALIGN (-4)
#define LLMI_ERR_UNSUPPORTED (-5)
#define LLMI_ERR_DRIVER (-6)

#define LLMI_EXPORT extern "C" __attribute__((visibility("default")))

namespace llmi {

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

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

// Sum over a block of up to 1024 threads in a fixed order: lanes by butterfly, warps in
// index order.  `scratch` holds at least 32 floats.  Every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from a previous call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < nwarp; ++w) total += scratch[w];
  return total;
}

inline int launch_status() { return cudaPeekAtLastError() == cudaSuccess ? LLMI_OK : LLMI_ERR_LAUNCH; }

}  // namespace llmi
