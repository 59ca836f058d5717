// Row-wise kernels: embedding gather, RMSNorm, SwiGLU gating.
//
// Formulas (reference, CPU): embedding row copy src/model/weight.cpp:39-45 and
// src/model/transformer.cpp:214-217; RMSNorm src/model/kernels.cpp:115-120
// (y = w * (x * scale), scale = 1/sqrt(mean(x^2) + eps)); SiLU gate
// src/model/kernels.cpp:148 with src/model/transformer.cpp:290.
#include "common.cuh"

namespace llmi {

// out[t, :] = float(table[ids[t], :]); a negative id (padding) gives a zero row.
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int32_t* __restrict__ ids, float* __restrict__ out,
                             int width) {
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int id = ids[t];
  float* o = out + (size_t)t * width;
  if (id < 0) {
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = 0.f;
    return;
  }
  const T* row = table + (size_t)id * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = to_f32(row[i]);
}

// One block per output row.  x is the fp32 residual stream; `rows` (optional) picks the
// input row of each output row, so the last norm runs only where logits are wanted.
template <typename T>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ weight, T* __restrict__ out,
                               const int32_t* __restrict__ rows, int width, float eps) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  T* o = out + (size_t)r * width;
  if (src < 0) {
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = from_f32<T>(0.f);
    return;
  }
  const float* xr = x + (size_t)src * width;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = xr[i];
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = from_f32<T>(weight[i] * (xr[i] * scale));
}

// The same, with the row held in registers between the sum of squares and the scaling: one read of x,
// 16-byte loads (VPT of them in flight per thread, which is what keeps a many-row launch at memory speed)
// and one store per four outputs.  Needs width % 4 == 0 and width <= 4 * VPT * blockDim.x.
__device__ __forceinline__ void store4(float* o, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(o) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(__nv_bfloat16* o, float a, float b, float c, float d) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 u;
  u.x = *reinterpret_cast<const uint32_t*>(&lo);
  u.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(o) = u;
}

template <typename T, int VPT>
__global__ void rmsnorm_reg_kernel(const float* __restrict__ x, const float* __restrict__ weight, T* __restrict__ out,
                                   const int32_t* __restrict__ rows, int width, float eps) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  T* o = out + (size_t)r * width;
  const int nvec = width >> 2;
  float4 v[VPT];
  float ss = 0.f;
  if (src >= 0) {
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)src * width);
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      v[j] = i < nvec ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < VPT; ++j) ss = fmaf(v[j].x, v[j].x, fmaf(v[j].y, v[j].y, fmaf(v[j].z, v[j].z, fmaf(v[j].w, v[j].w, ss))));
  } else {
#pragma unroll
    for (int j = 0; j < VPT; ++j) v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)width + eps);
  const float4* wv = reinterpret_cast<const float4*>(weight);
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = threadIdx.x + j * blockDim.x;
    if (i < nvec) {
      const float4 w = wv[i];
      store4(o + 4 * i, w.x * (v[j].x * scale), w.y * (v[j].y * scale), w.z * (v[j].z * scale), w.w * (v[j].w * scale));
    }
  }
}

// The same for MANY rows (a prompt): one warp per row, the row in registers (VPT 16-byte loads in flight per lane),
// the sum of squares by shuffles — no block barrier between the read and the write of a row.
template <typename T, int VPT>
__global__ void __launch_bounds__(256)
rmsnorm_warp_kernel(const float* __restrict__ x, const float* __restrict__ weight, T* __restrict__ out,
                    const int32_t* __restrict__ rows, int n_rows, int width, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= n_rows) return;
  const int src = rows ? rows[r] : r;
  T* o = out + (size_t)r * width;
  const int nvec = width >> 2;
  float4 v[VPT];
  float ss = 0.f;
  if (src >= 0) {
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)src * width);
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int i = lane + j * 32;
      v[j] = i < nvec ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < VPT; ++j) ss = fmaf(v[j].x, v[j].x, fmaf(v[j].y, v[j].y, fmaf(v[j].z, v[j].z, fmaf(v[j].w, v[j].w, ss))));
  } else {
#pragma unroll
    for (int j = 0; j < VPT; ++j) v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  ss = warp_sum(ss);
  const float scale = 1.0f / sqrtf(ss / (float)width + eps);
  const float4* wv = reinterpret_cast<const float4*>(weight);
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = lane + j * 32;
    if (i < nvec) {
      const float4 w = wv[i];
      store4(o + 4 * i, w.x * (v[j].x * scale), w.y * (v[j].y * scale), w.z * (v[j].z * scale), w.w * (v[j].w * scale));
    }
  }
}

// gate_up is [rows, 2*inner]: gate in the first half of a row, up in the second.
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inner, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / inner, c = i - r * inner;
    const float g = to_f32(gate_up[r * 2 * inner + c]);
    const float u = to_f32(gate_up[r * 2 * inner + inner + c]);
    const float s = g / (1.0f + expf(-g));
    out[i] = from_f32<T>(s * u);
  }
}

}  // namespace llmi

using namespace llmi;

LLMI_EXPORT int llmi_embed(int dtype, const void* table, const int32_t* ids, float* out, int n_tokens, int width,
                           cudaStream_t stream) {
  if (n_tokens <= 0 || width <= 0) return LLMI_ERR_BAD_SIZE;
  const int threads = width >= 1024 ? 256 : 128;
  if (dtype == LLMI_DTYPE_F32)
    embed_kernel<float><<<n_tokens, threads, 0, stream>>>((const float*)table, ids, out, width);
  else if (dtype == LLMI_DTYPE_BF16)
    embed_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>((const __nv_bfloat16*)table, ids, out, width);
  else
    return LLMI_ERR_BAD_DTYPE;
  return launch_status();
}

LLMI_EXPORT int llmi_rmsnorm(int out_dtype, const float* x, const float* weight, void* out, const int32_t* rows,
                             int n_rows, int width, float eps, cudaStream_t stream) {
  if (n_rows <= 0 || width <= 0) return LLMI_ERR_BAD_SIZE;
  const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
  if (out_dtype != LLMI_DTYPE_F32 && out_dtype != LLMI_DTYPE_BF16) return LLMI_ERR_BAD_DTYPE;
  const bool aligned = (width % 4 == 0) && !((uintptr_t)x & 15) && !((uintptr_t)weight & 15) && !((uintptr_t)out & 15);
  constexpr int VPT = 4;
  const int reg_threads = ((width / 4 + VPT - 1) / VPT + 31) / 32 * 32;    // four 16-byte loads per thread
  // many rows, compute-type output: a warp per row (the 32-bit path keeps one kernel for every number of rows, so that
  // a row's bits do not depend on how many rows are normalised with it)
  constexpr int WVPT = 16;                                                  // width <= 2048
  if (aligned && n_rows >= 512 && width <= 4 * 32 * WVPT && out_dtype == LLMI_DTYPE_BF16)
    return launch_pdl(PDL_SMALL, rmsnorm_warp_kernel<__nv_bfloat16, WVPT>, (n_rows + 7) / 8, 256, 0, stream, x, weight,
                      (__nv_bfloat16*)out, rows, n_rows, width, eps);
  if (aligned && reg_threads <= 1024) {
    if (out_dtype == LLMI_DTYPE_F32)
      return launch_pdl(PDL_SMALL, rmsnorm_reg_kernel<float, VPT>, n_rows, reg_threads, 0, stream, x, weight, (float*)out, rows, width, eps);
    else
      return launch_pdl(PDL_SMALL, rmsnorm_reg_kernel<__nv_bfloat16, VPT>, n_rows, reg_threads, 0, stream, x, weight, (__nv_bfloat16*)out, rows, width, eps);
  } else if (out_dtype == LLMI_DTYPE_F32)
    return launch_pdl(PDL_SMALL, rmsnorm_kernel<float>, n_rows, threads, 0, stream, x, weight, (float*)out, rows, width, eps);
  else
    return launch_pdl(PDL_SMALL, rmsnorm_kernel<__nv_bfloat16>, n_rows, threads, 0, stream, x, weight, (__nv_bfloat16*)out, rows, width, eps);
  return launch_status();
}

// Streaming multiprocessors of the current device, for dispatch rules that live on the host side of the library.
LLMI_EXPORT int llmi_sm_count() { return sm_count(); }

// A step's index block from pinned host memory to the device, on the stream: one plain asynchronous copy, here so
// that the host pays one call for it instead of a tensor operation (22 us of a decode step's 55 us of host time
// before its launches).  `done` (or null) is a mark from llmi_mark_new, set behind the copy: llmi_mark_wait returns
// once the copy has read the host bytes, so that they can be written again (copy and mark in one call: marking by a
// call of its own cost 10 us more).
LLMI_EXPORT int llmi_copy_to_device(void* dst, const void* src, long bytes, void* done, cudaStream_t stream) {
  if (bytes <= 0) return LLMI_ERR_BAD_SIZE;
  if (cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyHostToDevice, stream) != cudaSuccess) return LLMI_ERR_LAUNCH;
  if (done && cudaEventRecord((cudaEvent_t)done, stream) != cudaSuccess) return LLMI_ERR_LAUNCH;
  return LLMI_OK;
}
LLMI_EXPORT void* llmi_mark_new() {
  cudaEvent_t e = nullptr;
  return cudaEventCreateWithFlags(&e, cudaEventDisableTiming) == cudaSuccess ? (void*)e : nullptr;
}
LLMI_EXPORT int llmi_mark_wait(void* mark) {
  return mark && cudaEventSynchronize((cudaEvent_t)mark) == cudaSuccess ? LLMI_OK : LLMI_ERR_LAUNCH;
}
LLMI_EXPORT void llmi_mark_free(void* mark) {
  if (mark) cudaEventDestroy((cudaEvent_t)mark);
}

// A step's result (the chosen ids, a few bytes) to pinned host memory, waited for: one call for the copy and the wait.
// A tensor's own way to the host goes through pageable memory and costs about 27 us after the device is done.
LLMI_EXPORT int llmi_copy_to_host(void* dst, const void* src, long bytes, cudaStream_t stream) {
  if (bytes <= 0) return LLMI_ERR_BAD_SIZE;
  if (cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDeviceToHost, stream) != cudaSuccess) return LLMI_ERR_LAUNCH;
  return cudaStreamSynchronize(stream) == cudaSuccess ? LLMI_OK : LLMI_ERR_LAUNCH;
}

LLMI_EXPORT int llmi_swiglu(int dtype, const void* gate_up, void* out, int n_rows, int inner, cudaStream_t stream) {
  if (n_rows <= 0 || inner <= 0) return LLMI_ERR_BAD_SIZE;
  const size_t total = (size_t)n_rows * inner;
  const int threads = 256;
  const size_t most = (size_t)sm_count() * 16;       // a grid-stride loop takes the rest
  const int blocks = (int)((total + threads - 1) / threads < most ? (total + threads - 1) / threads : most);
  if (dtype == LLMI_DTYPE_F32)
    return launch_pdl(PDL_SMALL, swiglu_kernel<float>, blocks, threads, 0, stream, (const float*)gate_up, (float*)out, inner, total);
  else if (dtype == LLMI_DTYPE_BF16)
    return launch_pdl(PDL_SMALL, swiglu_kernel<__nv_bfloat16>, blocks, threads, 0, stream, (const __nv_bfloat16*)gate_up,
                      (__nv_bfloat16*)out, inner, total);
  else
    return LLMI_ERR_BAD_DTYPE;
  return launch_status();
}
