// Causal grouped-query attention over the paged cache, any sizes, fp32 arithmetic.
//
// Reference: src/model/transformer.cpp:263-282 — for query head hh the kv head is hh / group
// (integer division), score[s] = dot(q, k_s) * scale for s = 0..pos, softmax
// (src/model/kernels.cpp:136-146), out = sum_s p_s * v_s.
//
// One warp owns one (token, query head).  Keys are taken 32 at a time in blocks anchored at
// absolute positions 0, 32, 64, ... with a running maximum and sum, so the order of every
// addition depends only on the key's position, not on how the step was cut or batched.
// `window` > 0 limits a query at position p to keys p-window+1..p.
// This kernel serves prefill and decode of the fp32 path, and bf16 head sizes that the
// tensor-core kernels do not take.
#include <math.h>

#include "common.cuh"
#include "step_meta.cuh"

namespace llmi {

constexpr int ATT_WARPS = 4;
constexpr int ATT_MAX_HD = 256;

template <typename T>
__device__ __forceinline__ float dot_q_row(const float* __restrict__ q, const T* __restrict__ k, int hd) {
  float acc = 0.f;
  for (int d = 0; d < hd; ++d) acc = fmaf(q[d], to_f32(k[d]), acc);
  return acc;
}

template <>
__device__ __forceinline__ float dot_q_row<__nv_bfloat16>(const float* __restrict__ q,
                                                          const __nv_bfloat16* __restrict__ k, int hd) {
  float acc = 0.f;
  if ((hd & 7) == 0) {
    for (int d = 0; d < hd; d += 8) {
      const uint4 raw = *reinterpret_cast<const uint4*>(k + d);
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(p[e]);
        acc = fmaf(q[d + 2 * e], f.x, acc);
        acc = fmaf(q[d + 2 * e + 1], f.y, acc);
      }
    }
  } else {
    for (int d = 0; d < hd; ++d) acc = fmaf(q[d], __bfloat162float(k[d]), acc);
  }
  return acc;
}

template <>
__device__ __forceinline__ float dot_q_row<float>(const float* __restrict__ q, const float* __restrict__ k, int hd) {
  float acc = 0.f;
  if ((hd & 3) == 0) {
    for (int d = 0; d < hd; d += 4) {
      const float4 f = *reinterpret_cast<const float4*>(k + d);
      acc = fmaf(q[d], f.x, acc);
      acc = fmaf(q[d + 1], f.y, acc);
      acc = fmaf(q[d + 2], f.z, acc);
      acc = fmaf(q[d + 3], f.w, acc);
    }
  } else {
    for (int d = 0; d < hd; ++d) acc = fmaf(q[d], k[d], acc);
  }
  return acc;
}

// NJ = ceil(head_dim / 32): output elements per lane.
template <typename T, int NJ>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attention_generic_kernel(const T* __restrict__ q, long ldq, T* __restrict__ out, long ldo,
                         const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                         const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ tok_pos, PagedKV kv,
                         int n_tokens, int n_heads, float scale, int window) {
  __shared__ float q_s[ATT_WARPS][ATT_MAX_HD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long item = (long)blockIdx.x * ATT_WARPS + warp;
  if (item >= (long)n_tokens * n_heads) return;
  const int t = (int)(item / n_heads), h = (int)(item - (long)t * n_heads);
  const int hd = kv.head_dim;
  const int seq = tok_seq[t];
  T* o = out + (size_t)t * ldo + (size_t)h * hd;
  if (seq < 0) {
    for (int d = lane; d < hd; d += 32) o[d] = from_f32<T>(0.f);
    return;
  }
  const int pos = tok_pos[t];
  const int kvh = h / (n_heads / kv.n_kv_heads);
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

  const T* qp = q + (size_t)t * ldq + (size_t)h * hd;
  for (int d = lane; d < hd; d += 32) q_s[warp][d] = to_f32(qp[d]);
  __syncwarp();

  float m = -INFINITY, l = 0.f;
  float acc[NJ];
#pragma unroll
  for (int j = 0; j < NJ; ++j) acc[j] = 0.f;

  for (int c0 = (lo / 32) * 32; c0 <= pos; c0 += 32) {
    const int s = c0 + lane;
    const bool valid = s >= lo && s <= pos;
    float score = -INFINITY;
    if (valid) score = dot_q_row<T>(q_s[warp], k_cache + kv_row_offset(kv, seq, s, kvh), hd) * scale;
    const float m_new = fmaxf(m, warp_max(score));
    const float p = valid ? expf(score - m_new) : 0.f;
    const float corr = expf(m - m_new);  // first block: exp(-inf) = 0
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int j = 0; j < NJ; ++j) acc[j] *= corr;
    const int kend = (pos - c0 + 1 < 32) ? pos - c0 + 1 : 32;
    for (int kk = 0; kk < kend; ++kk) {
      const float pk = __shfl_sync(0xffffffffu, p, kk);
      if (c0 + kk < lo) continue;
      const T* vr = v_cache + kv_row_offset(kv, seq, c0 + kk, kvh);
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        const int d = lane + 32 * j;
        if (d < hd) acc[j] = fmaf(pk, to_f32(vr[d]), acc[j]);
      }
    }
    m = m_new;
  }
  const float inv = 1.0f / l;
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    const int d = lane + 32 * j;
    if (d < hd) o[d] = from_f32<T>(acc[j] * inv);
  }
}

template <typename T>
int launch_attention_generic(const void* q, long ldq, void* out, long ldo, const void* k_cache, const void* v_cache,
                             const int32_t* tok_seq, const int32_t* tok_pos, PagedKV kv, int n_tokens, int n_heads,
                             float scale, int window, cudaStream_t stream) {
  const long items = (long)n_tokens * n_heads;
  const long blocks = (items + ATT_WARPS - 1) / ATT_WARPS;
  if (blocks > 0x7fffffffL) return LLMI_ERR_BAD_SIZE;
  const int nj = (kv.head_dim + 31) / 32;
#define LLMI_LAUNCH(NJ)                                                                                              \
  attention_generic_kernel<T, NJ><<<(unsigned)blocks, ATT_WARPS * 32, 0, stream>>>(                                  \
      (const T*)q, ldq, (T*)out, ldo, (const T*)k_cache, (const T*)v_cache, tok_seq, tok_pos, kv, n_tokens, n_heads, \
      scale, window)
  if (nj <= 1) LLMI_LAUNCH(1);
  else if (nj <= 2) LLMI_LAUNCH(2);
  else if (nj <= 4) LLMI_LAUNCH(4);
  else LLMI_LAUNCH(8);
#undef LLMI_LAUNCH
  return launch_status();
}

}  // namespace llmi

using namespace llmi;

LLMI_EXPORT int llmi_attention_generic(int dtype, const void* q, long ldq, void* out, long ldo, const void* k_cache,
                                       const void* v_cache, const int32_t* tok_seq, const int32_t* tok_pos,
                                       const int32_t* seq_pages, int pages_stride, int page_size, int n_tokens,
                                       int n_heads, int n_kv_heads, int head_dim, float scale, int window,
                                       cudaStream_t stream) {
  if (n_tokens <= 0 || n_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0 || page_size <= 0) return LLMI_ERR_BAD_SIZE;
  if (head_dim > ATT_MAX_HD || n_heads % n_kv_heads != 0) return LLMI_ERR_BAD_SIZE;
  PagedKV kv{seq_pages, pages_stride, page_size, n_kv_heads, head_dim};
  if (dtype == LLMI_DTYPE_F32)
    return launch_attention_generic<float>(q, ldq, out, ldo, k_cache, v_cache, tok_seq, tok_pos, kv, n_tokens,
                                           n_heads, scale, window, stream);
  if (dtype == LLMI_DTYPE_BF16)
    return launch_attention_generic<__nv_bfloat16>(q, ldq, out, ldo, k_cache, v_cache, tok_seq, tok_pos, kv, n_tokens,
                                                   n_heads, scale, window, stream);
  return LLMI_ERR_BAD_DTYPE;
}
