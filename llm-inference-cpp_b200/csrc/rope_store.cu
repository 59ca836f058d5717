// Rotary position encoding of q and k, fused with the append of k and v to the paged cache.
//
// Reference formulas: src/model/kernels.cpp:122-134 (rotate-half pairing (i, i + half),
// angle = float(pos) * inv_freq[i] in fp32, then cos and sin), applied to every q head and
// every k head but not to v (src/model/transformer.cpp:251-254); k enters the cache already
// rotated (src/model/transformer.cpp:255-262).  inv_freq is given by the caller
// (src/model/transformer.cpp:59-65).
//
// qkv is one row per token: [q heads | k heads | v heads], each head head_dim wide.
// q is rotated in place; k (rotated) and v go to the cache page of (sequence, position).
// rotary_dim <= head_dim may be smaller than the head (the rest passes through); 0 turns
// the rotation off, leaving a plain cache append.
#include "common.cuh"
#include "step_meta.cuh"

namespace llmi {

constexpr int MAX_HALF = 256;

template <typename T>
__global__ void __launch_bounds__(128)
rope_store_kernel(T* __restrict__ qkv, long ld, const float* __restrict__ inv_freq, int rotary_dim,
                  const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ tok_pos, PagedKV kv,
                  T* __restrict__ k_cache, T* __restrict__ v_cache, int n_heads, int write_kv) {
  __shared__ float cs[MAX_HALF], sn[MAX_HALF];
  const int t = blockIdx.x;
  const int seq = tok_seq[t];
  if (seq < 0) return;
  const int pos = tok_pos[t];
  const int hd = kv.head_dim, nkv = kv.n_kv_heads;
  const int half = rotary_dim / 2;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float angle = (float)pos * inv_freq[i];
    float s, c;
    sincosf(angle, &s, &c);
    cs[i] = c;
    sn[i] = s;
  }
  __syncthreads();

  T* row = qkv + (size_t)t * ld;
  // q heads, in place
  for (int idx = threadIdx.x; idx < n_heads * half; idx += blockDim.x) {
    const int h = idx / half, i = idx - h * half;
    T* p = row + (size_t)h * hd;
    const float a = to_f32(p[i]), b = to_f32(p[i + half]);
    p[i] = from_f32<T>(a * cs[i] - b * sn[i]);
    p[i + half] = from_f32<T>(b * cs[i] + a * sn[i]);
  }
  if (!write_kv) return;

  const T* krow = row + (size_t)n_heads * hd;
  const T* vrow = krow + (size_t)nkv * hd;
  for (int idx = threadIdx.x; idx < nkv * hd; idx += blockDim.x) {
    const int h = idx / hd, d = idx - h * hd;
    const size_t dst = kv_row_offset(kv, seq, pos, h) + d;
    float kval;
    if (d < half) {
      kval = to_f32(krow[h * hd + d]) * cs[d] - to_f32(krow[h * hd + d + half]) * sn[d];
    } else if (d < rotary_dim) {
      const int i = d - half;
      kval = to_f32(krow[h * hd + d]) * cs[i] + to_f32(krow[h * hd + i]) * sn[i];
    } else {
      kval = to_f32(krow[h * hd + d]);
    }
    k_cache[dst] = from_f32<T>(kval);
    v_cache[dst] = vrow[h * hd + d];
  }
}

}  // namespace llmi

using namespace llmi;

LLMI_EXPORT int llmi_rope_store(int dtype, void* qkv, long ld, const float* inv_freq, int rotary_dim,
                                const int32_t* tok_seq, const int32_t* tok_pos, const int32_t* seq_pages,
                                int pages_stride, int page_size, void* k_cache, void* v_cache, int n_tokens,
                                int n_heads, int n_kv_heads, int head_dim, int write_kv, cudaStream_t stream) {
  if (n_tokens <= 0 || n_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0 || page_size <= 0) return LLMI_ERR_BAD_SIZE;
  if (rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1) || rotary_dim / 2 > MAX_HALF) return LLMI_ERR_BAD_SIZE;
  PagedKV kv{seq_pages, pages_stride, page_size, n_kv_heads, head_dim};
  if (dtype == LLMI_DTYPE_F32)
    rope_store_kernel<float><<<n_tokens, 128, 0, stream>>>((float*)qkv, ld, inv_freq, rotary_dim, tok_seq, tok_pos, kv,
                                                           (float*)k_cache, (float*)v_cache, n_heads, write_kv);
  else if (dtype == LLMI_DTYPE_BF16)
    rope_store_kernel<__nv_bfloat16><<<n_tokens, 128, 0, stream>>>(
        (__nv_bfloat16*)qkv, ld, inv_freq, rotary_dim, tok_seq, tok_pos, kv, (__nv_bfloat16*)k_cache,
        (__nv_bfloat16*)v_cache, n_heads, write_kv);
  else
    return LLMI_ERR_BAD_DTYPE;
  return launch_status();
}
