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
#include <stdlib.h>

#define LLMI_DTYPE_F32 0
#define LLMI_DTYPE_BF16 1

#define LLMI_OK 0
#define LLMI_ERR_BAD_DTYPE (-1)
#define LLMI_ERR_BAD_SIZE (-2)
#define LLMI_ERR_LAUNCH (-3)
#define LLMI_ERR_ALIGN (-4)
#define LLMI_ERR_UNSUPPORTED (-5)
#define LLMI_ERR_DRIVER (-6)
#define LLMI_ERR_STATIC_SCRATCH (-7)  // the problem needs more scratch than a built-in array holds

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

// 2^x on the special-function unit, one instruction (ex2.approx: relative error about 2^-22; the results
// here end up in bf16).  exp2f() costs several such instructions.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// The rotation of one pair, with its roundings spelled out so that every kernel that rotates gives the
// same bits whatever the compiler would contract: the result must not depend on which kernel a step's
// size selects.
__device__ __forceinline__ float rot_lo(float a, float b, float c, float s) { return __fmaf_rn(a, c, -__fmul_rn(b, s)); }
__device__ __forceinline__ float rot_hi(float a, float b, float c, float s) { return __fmaf_rn(b, c, __fmul_rn(a, s)); }
// Facts and one-time set-up per device.  A process may drive several GPUs, and a function attribute (the
// dynamic shared memory a kernel may ask for) or a count derived from the device (how many blocks are
// resident at once) belongs to the device that was current when it was set or read.
constexpr int MAX_DEVICES = 64;
inline int current_device() {
  int d = 0;
  if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= MAX_DEVICES) d = 0;
  return d;
}
// Streaming multiprocessors of the current device (a B200 has 148; a part with fewer enabled has fewer).
inline int sm_count() {
  static int n[MAX_DEVICES] = {};
  const int d = current_device();
  if (n[d] == 0) {
    int v = 0;
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, d);
    n[d] = v > 0 ? v : 1;
  }
  return n[d];
}
// `static PerDevice<bool> configured; if (!configured.here()) { ...; configured.here() = true; }`
template <typename V> struct PerDevice {
  V v[MAX_DEVICES] = {};
  V& here() { return v[current_device()]; }
};

// The size of a persistent grid whose blocks take every grid-th item of items numbered with `period` as the fastest
// index (for instance the splits of a sequence-head): at most `resident`, and coprime to `period` when a block takes
// several items.  With a common factor a block gets the same residues every time, and an item kind that is slower
// than the others (the split that holds a sequence's newest page) always falls to the same blocks (measured on the
// decode attention kernel at batch 32, 64 pages: splits of 16 / 11 / 22 pages 187 / 184 / 173 us, of 13 pages 163 us
// with 444 blocks; 166 / 163 / 166 / 165 us with 443).
inline int coprime_grid(long n_items, int resident, int period) {
  int grid = (int)(n_items < resident ? n_items : resident);
  if (n_items > grid && period > 1) {
    auto gcd = [](int a, int b) { while (b) { const int t = a % b; a = b; b = t; } return a; };
    while (grid > 1 && gcd(grid, period) != 1) --grid;
  }
  return grid;
}

inline int launch_status() { return cudaPeekAtLastError() == cudaSuccess ? LLMI_OK : LLMI_ERR_LAUNCH; }

// Programmatic dependent launch.  A kernel launched with launch_pdl may start while the kernel before
// it in the stream is still running; it must call pdl_wait() before it touches anything that kernel
// wrote (and before it writes anything that kernel may still read).  pdl_launch_dependents() lets the
// kernel after it start early in turn.  Both are no-ops in a kernel launched the plain way.  A decode
// step is a chain of hundreds of few-microsecond kernels: this overlaps each kernel's launch and
// set-up (and, in the matrix product, its first weight loads) with the tail of the one before.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// LLMI_PDL is a bit mask of the kernel kinds that launch this way (default: all).  One rule came from
// measurement: the decode attention kernel must not start while the product before the rotary kernel
// still runs (batch 16: 3.86 ms a step against 3.18 ms; batch 64: 13.6 against 10.5), so the rotary
// kernel signals its dependents only after its own wait, where every other kernel signals at once.
constexpr int PDL_SMALL = 1, PDL_GEMM = 2, PDL_ATTENTION = 4, PDL_ROPE = 8;
inline bool pdl_enabled(int kind) {
  static int mask = -1;
  if (mask < 0) {
    const char* e = getenv("LLMI_PDL");
    mask = e ? atoi(e) : (PDL_SMALL | PDL_GEMM | PDL_ATTENTION | PDL_ROPE);
  }
  return (mask & kind) != 0;
}

template <typename... KArgs, typename... Args>
inline int launch_pdl(int kind, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                      Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled(kind) ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...) == cudaSuccess ? LLMI_OK : LLMI_ERR_LAUNCH;
}

}  // namespace llmi
