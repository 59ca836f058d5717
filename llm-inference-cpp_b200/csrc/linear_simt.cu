// y = x · Wᵀ (+ bias) with fp32 FMA arithmetic on the CUDA cores.
//
// This is the true 32-bit matrix product of the library (no tensor-core mode, no
// reduced-precision inputs when T = float) and the fallback for bf16 shapes the
// tensor-core kernel refuses.  W is [out, in] row-major as the reference stores it
// (include/llmi/model/kernels.hpp:15-17; src/model/kernels.cpp:97-113), x is [rows, in].
// Every output element is one thread's running sum over k = 0..K-1 in ascending order, so
// the value of y[r, o] does not depend on how many rows are in the call or where r lies.
#include "common.cuh"

namespace llmi {

constexpr int BM = 64, BN = 64, BK = 16;

// Output modes of the product.
constexpr int OUT_STORE = 0;      // y (type T) = acc
constexpr int OUT_STORE_F32 = 1;  // y (float) = acc
constexpr int OUT_ADD_F32 = 2;    // y (float) += acc       (residual sum kept in fp32)

template <typename T, int MODE>
__global__ void __launch_bounds__(256)
linear_simt_kernel(const T* __restrict__ x, long ldx, const T* __restrict__ w, long ldw,
                   const float* __restrict__ bias, void* __restrict__ yv, long ldy, int M, int N, int K) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int lr = tid >> 2;        // row of the tile this thread loads
  const int lk = (tid & 3) * 4;   // first of its four k

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  // The next k block is fetched into registers while the current one is multiplied, so that a block pays the
  // latency of global memory once, not once per k block.  The order of the additions is untouched.
  const int m_ld = m0 + lr, n_ld = n0 + lr;
  float a_next[4], b_next[4];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int k = k0 + lk + e;
      a_next[e] = (m_ld < M && k < K) ? to_f32(x[(long)m_ld * ldx + k]) : 0.f;
      b_next[e] = (n_ld < N && k < K) ? to_f32(w[(long)n_ld * ldw + k]) : 0.f;
    }
  };
  fetch(0);
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      As[lk + e][lr] = a_next[e];
      Bs[lk + e][lr] = b_next[e];
    }
    __syncthreads();
    if (k0 + BK < K) fetch(k0 + BK);
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[n];
      if (MODE == OUT_STORE) {
        ((T*)yv)[(long)m * ldy + n] = from_f32<T>(v);
      } else if (MODE == OUT_STORE_F32) {
        ((float*)yv)[(long)m * ldy + n] = v;
      } else {
        float* p = (float*)yv + (long)m * ldy + n;
        *p = *p + v;
      }
    }
  }
}

template <typename T>
int launch_linear_simt(const void* x, long ldx, const void* w, long ldw, const float* bias, void* y, long ldy, int M,
                       int N, int K, int mode, cudaStream_t stream) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return LLMI_ERR_BAD_SIZE;
  switch (mode) {
    case OUT_STORE:
      linear_simt_kernel<T, OUT_STORE><<<grid, 256, 0, stream>>>((const T*)x, ldx, (const T*)w, ldw, bias, y, ldy, M, N, K);
      break;
    case OUT_STORE_F32:
      linear_simt_kernel<T, OUT_STORE_F32><<<grid, 256, 0, stream>>>((const T*)x, ldx, (const T*)w, ldw, bias, y, ldy, M, N, K);
      break;
    case OUT_ADD_F32:
      linear_simt_kernel<T, OUT_ADD_F32><<<grid, 256, 0, stream>>>((const T*)x, ldx, (const T*)w, ldw, bias, y, ldy, M, N, K);
      break;
    default:
      return LLMI_ERR_UNSUPPORTED;
  }
  return launch_status();
}

}  // namespace llmi

using namespace llmi;

// x [M, K] (row pitch ldx), w [N, K] (row pitch ldw), y [M, N] (row pitch ldy), pitches in elements.
LLMI_EXPORT int llmi_linear_simt(int dtype, const void* x, long ldx, const void* w, long ldw, const float* bias,
                                 void* y, long ldy, int M, int N, int K, int mode, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return LLMI_ERR_BAD_SIZE;
  if (dtype == LLMI_DTYPE_F32) return launch_linear_simt<float>(x, ldx, w, ldw, bias, y, ldy, M, N, K, mode, stream);
  if (dtype == LLMI_DTYPE_BF16)
    return launch_linear_simt<__nv_bfloat16>(x, ldx, w, ldw, bias, y, ldy, M, N, K, mode, stream);
  return LLMI_ERR_BAD_DTYPE;
}
