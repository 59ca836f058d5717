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

constexpr int ROPE_WARPS = 4;
constexpr int ROWS_MIN_TOKENS = 256;   // from here on the kernel that shares sines and cosines among the heads pays

// One warp per (token, head): heads 0..n_heads-1 are query heads (rotated in place), heads
// n_heads..n_heads+n_kv-1 are key heads (rotated into the cache) together with their value heads.
template <typename T>
__global__ void __launch_bounds__(ROPE_WARPS * 32)
rope_store_kernel(T* __restrict__ qkv, long ld, const float* __restrict__ inv_freq, int rotary_dim,
                  const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ tok_pos, PagedKV kv,
                  T* __restrict__ k_cache, T* __restrict__ v_cache, int n_heads, int write_kv, long n_items) {
  pdl_wait();
  pdl_launch_dependents();   // not earlier: the attention kernel behind this one must not start while the product before still runs
  const long item = (long)blockIdx.x * ROPE_WARPS + (threadIdx.x >> 5);
  if (item >= n_items) return;
  const int lane = threadIdx.x & 31;
  const int per_tok = n_heads + kv.n_kv_heads;
  const int t = (int)(item / per_tok), j = (int)(item - (long)t * per_tok);
  const int seq = tok_seq[t];
  if (seq < 0) return;
  const int pos = tok_pos[t];
  const int hd = kv.head_dim, half = rotary_dim / 2;
  T* row = qkv + (size_t)t * ld;
  if (j < n_heads) {
    T* p = row + (size_t)j * hd;
    for (int i = lane; i < half; i += 32) {
      float s, c;
      sincosf((float)pos * inv_freq[i], &s, &c);
      const float a = to_f32(p[i]), b = to_f32(p[i + half]);
      p[i] = from_f32<T>(rot_lo(a, b, c, s));
      p[i + half] = from_f32<T>(rot_hi(a, b, c, s));
    }
    return;
  }
  if (!write_kv) return;
  const int h = j - n_heads;
  const T* ksrc = row + (size_t)(n_heads + h) * hd;
  const T* vsrc = row + (size_t)(n_heads + kv.n_kv_heads + h) * hd;
  const size_t dst = kv_row_offset(kv, seq, pos, h);
  for (int i = lane; i < half; i += 32) {
    float s, c;
    sincosf((float)pos * inv_freq[i], &s, &c);
    const float a = to_f32(ksrc[i]), b = to_f32(ksrc[i + half]);
    k_cache[dst + i] = from_f32<T>(rot_lo(a, b, c, s));
    k_cache[dst + i + half] = from_f32<T>(rot_hi(a, b, c, s));
  }
  for (int d = rotary_dim + lane; d < hd; d += 32) k_cache[dst + d] = ksrc[d];
  for (int d = lane; d < hd; d += 32) v_cache[dst + d] = vsrc[d];
}

// The same for whole-head rotation with head_dim % 4 == 0: one thread per two neighbouring pairs, so that
// every access is a pair of elements (4 bytes in bf16) and a prompt of thousands of tokens moves at
// memory speed.
template <typename T> struct Pair;
template <> struct Pair<float> {
  static __device__ __forceinline__ float2 load(const float* p) { return *reinterpret_cast<const float2*>(p); }
  static __device__ __forceinline__ void store(float* p, float2 v) { *reinterpret_cast<float2*>(p) = v; }
};
template <> struct Pair<__nv_bfloat16> {
  static __device__ __forceinline__ float2 load(const __nv_bfloat16* p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float2 v) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v.x, v.y);
  }
};

template <typename T>
__global__ void __launch_bounds__(256)
rope_store_vec_kernel(T* __restrict__ qkv, long ld, const float* __restrict__ inv_freq, const int32_t* __restrict__ tok_seq,
                      const int32_t* __restrict__ tok_pos, PagedKV kv, T* __restrict__ k_cache, T* __restrict__ v_cache,
                      int n_heads, int write_kv, long n_items) {
  pdl_wait();
  pdl_launch_dependents();   // not earlier: the attention kernel behind this one must not start while the product before still runs
  const long item = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (item >= n_items) return;
  const int hd = kv.head_dim, half = hd / 2, per_head = half / 2;
  const int per_tok = (n_heads + kv.n_kv_heads) * per_head;
  const int t = (int)(item / per_tok);
  const int rest = (int)(item - (long)t * per_tok);
  const int j = rest / per_head, i = (rest - j * per_head) * 2;    // head j, pairs i and i+1
  const int seq = tok_seq[t];
  if (seq < 0) return;
  const int pos = tok_pos[t];
  float s0, c0, s1, c1;
  sincosf((float)pos * inv_freq[i], &s0, &c0);
  sincosf((float)pos * inv_freq[i + 1], &s1, &c1);
  T* row = qkv + (size_t)t * ld;
  if (j < n_heads) {
    T* p = row + (size_t)j * hd;
    const float2 a = Pair<T>::load(p + i), b = Pair<T>::load(p + i + half);
    Pair<T>::store(p + i, make_float2(rot_lo(a.x, b.x, c0, s0), rot_lo(a.y, b.y, c1, s1)));
    Pair<T>::store(p + i + half, make_float2(rot_hi(a.x, b.x, c0, s0), rot_hi(a.y, b.y, c1, s1)));
    return;
  }
  if (!write_kv) return;
  const int h = j - n_heads;
  const T* ksrc = row + (size_t)(n_heads + h) * hd;
  const T* vsrc = row + (size_t)(n_heads + kv.n_kv_heads + h) * hd;
  const size_t dst = kv_row_offset(kv, seq, pos, h);
  const float2 a = Pair<T>::load(ksrc + i), b = Pair<T>::load(ksrc + i + half);
  Pair<T>::store(k_cache + dst + i, make_float2(rot_lo(a.x, b.x, c0, s0), rot_lo(a.y, b.y, c1, s1)));
  Pair<T>::store(k_cache + dst + i + half, make_float2(rot_hi(a.x, b.x, c0, s0), rot_hi(a.y, b.y, c1, s1)));
  Pair<T>::store(v_cache + dst + i, Pair<T>::load(vsrc + i));
  Pair<T>::store(v_cache + dst + i + half, Pair<T>::load(vsrc + i + half));
}

// The same for a long prompt: the angle of (position, pair) is the same for every head of a token, and
// sine and cosine are the costly part.  A thread takes one 16-byte chunk of the first half of a head and
// its partner chunk in the second half, computes the chunk's sines and cosines once, and walks over every
// ROWS_HEAD_LANES-th head of the token with 16-byte loads and stores.  The arithmetic of an element is
// that of the kernels above, so the results are the same bits.
constexpr int ROWS_HEAD_LANES = 16;

template <typename T> struct Chunk;
template <> struct Chunk<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float* f) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x, f[1] = v.y, f[2] = v.z, f[3] = v.w;
  }
  static __device__ __forceinline__ void store(float* p, const float* f) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  }
  static __device__ __forceinline__ void copy(float* dst, const float* src) {
    *reinterpret_cast<float4*>(dst) = *reinterpret_cast<const float4*>(src);
  }
};
template <> struct Chunk<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* f) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 v = __bfloat1622float2(h[e]);
      f[2 * e] = v.x, f[2 * e + 1] = v.y;
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* f) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
  }
  static __device__ __forceinline__ void copy(__nv_bfloat16* dst, const __nv_bfloat16* src) {
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
  }
};

template <typename T>
__global__ void __launch_bounds__(128)
rope_store_rows_kernel(T* __restrict__ qkv, long ld, const float* __restrict__ inv_freq, const int32_t* __restrict__ tok_seq,
                       const int32_t* __restrict__ tok_pos, PagedKV kv, T* __restrict__ k_cache, T* __restrict__ v_cache,
                       int n_heads, int write_kv, long n_items) {
  constexpr int N = Chunk<T>::N;
  pdl_wait();
  pdl_launch_dependents();   // not earlier: the attention kernel behind this one must not start while the product before still runs
  const long item = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (item >= n_items) return;
  const int hd = kv.head_dim, half = hd / 2, n_chunks = half / N;
  const int per_tok = n_chunks * ROWS_HEAD_LANES;
  const int t = (int)(item / per_tok);
  const int rest = (int)(item - (long)t * per_tok);
  const int hl = rest / n_chunks, i0 = (rest - hl * n_chunks) * N;
  const int seq = tok_seq[t];
  if (seq < 0) return;
  const int pos = tok_pos[t];
  float sn[N], cs[N];
#pragma unroll
  for (int e = 0; e < N; ++e) sincosf((float)pos * inv_freq[i0 + e], &sn[e], &cs[e]);
  T* row = qkv + (size_t)t * ld;
#pragma unroll 4
  for (int j = hl; j < n_heads; j += ROWS_HEAD_LANES) {
    T* p = row + (size_t)j * hd + i0;
    float a[N], b[N], lo[N], hi[N];
    Chunk<T>::load(p, a);
    Chunk<T>::load(p + half, b);
#pragma unroll
    for (int e = 0; e < N; ++e) {
      lo[e] = rot_lo(a[e], b[e], cs[e], sn[e]);
      hi[e] = rot_hi(a[e], b[e], cs[e], sn[e]);
    }
    Chunk<T>::store(p, lo);
    Chunk<T>::store(p + half, hi);
  }
  if (!write_kv) return;
#pragma unroll 4
  for (int h = hl; h < kv.n_kv_heads; h += ROWS_HEAD_LANES) {
    const T* ksrc = row + (size_t)(n_heads + h) * hd + i0;
    const T* vsrc = row + (size_t)(n_heads + kv.n_kv_heads + h) * hd + i0;
    const size_t dst = kv_row_offset(kv, seq, pos, h) + i0;
    float a[N], b[N], lo[N], hi[N];
    Chunk<T>::load(ksrc, a);
    Chunk<T>::load(ksrc + half, b);
#pragma unroll
    for (int e = 0; e < N; ++e) {
      lo[e] = rot_lo(a[e], b[e], cs[e], sn[e]);
      hi[e] = rot_hi(a[e], b[e], cs[e], sn[e]);
    }
    Chunk<T>::store(k_cache + dst, lo);
    Chunk<T>::store(k_cache + dst + half, hi);
    Chunk<T>::copy(v_cache + dst, vsrc);
    Chunk<T>::copy(v_cache + dst + half, vsrc + half);
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
  const size_t esz = dtype == LLMI_DTYPE_F32 ? 4 : 2;
  const bool pair_aligned = !(((uintptr_t)qkv | (uintptr_t)k_cache | (uintptr_t)v_cache) & (2 * esz - 1)) && !(ld & 1);
  const int chunk = 16 / (int)esz;
  const bool chunk_aligned = !(((uintptr_t)qkv | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) && !((ld * esz) & 15) &&
                             (head_dim / 2) % chunk == 0;
  if (rotary_dim == head_dim && chunk_aligned && n_tokens >= ROWS_MIN_TOKENS &&
      (dtype == LLMI_DTYPE_F32 || dtype == LLMI_DTYPE_BF16)) {
    const long n_thr = (long)n_tokens * (head_dim / 2 / chunk) * ROWS_HEAD_LANES;
    const long rblocks = (n_thr + 127) / 128;
    if (rblocks > 0x7fffffffL) return LLMI_ERR_BAD_SIZE;
    if (dtype == LLMI_DTYPE_F32)
      return launch_pdl(PDL_ROPE, rope_store_rows_kernel<float>, (unsigned)rblocks, 128, 0, stream, (float*)qkv, ld, inv_freq,
                        tok_seq, tok_pos, kv, (float*)k_cache, (float*)v_cache, n_heads, write_kv, n_thr);
    return launch_pdl(PDL_ROPE, rope_store_rows_kernel<__nv_bfloat16>, (unsigned)rblocks, 128, 0, stream, (__nv_bfloat16*)qkv,
                      ld, inv_freq, tok_seq, tok_pos, kv, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, n_heads,
                      write_kv, n_thr);
  }
  if (rotary_dim == head_dim && head_dim % 4 == 0 && pair_aligned && (dtype == LLMI_DTYPE_F32 || dtype == LLMI_DTYPE_BF16)) {
    const long n_vec = (long)n_tokens * (n_heads + n_kv_heads) * (head_dim / 4);
    const long vblocks = (n_vec + 255) / 256;
    if (vblocks > 0x7fffffffL) return LLMI_ERR_BAD_SIZE;
    if (dtype == LLMI_DTYPE_F32)
      return launch_pdl(PDL_ROPE, rope_store_vec_kernel<float>, (unsigned)vblocks, 256, 0, stream, (float*)qkv, ld, inv_freq,
                        tok_seq, tok_pos, kv, (float*)k_cache, (float*)v_cache, n_heads, write_kv, n_vec);
    return launch_pdl(PDL_ROPE, rope_store_vec_kernel<__nv_bfloat16>, (unsigned)vblocks, 256, 0, stream, (__nv_bfloat16*)qkv,
                      ld, inv_freq, tok_seq, tok_pos, kv, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, n_heads,
                      write_kv, n_vec);
  }
  const long n_items = (long)n_tokens * (n_heads + n_kv_heads);
  const long blocks = (n_items + ROPE_WARPS - 1) / ROPE_WARPS;
  if (blocks > 0x7fffffffL) return LLMI_ERR_BAD_SIZE;
  if (dtype == LLMI_DTYPE_F32)
    return launch_pdl(PDL_ROPE, rope_store_kernel<float>, (unsigned)blocks, ROPE_WARPS * 32, 0, stream, (float*)qkv, ld, inv_freq,
                      rotary_dim, tok_seq, tok_pos, kv, (float*)k_cache, (float*)v_cache, n_heads, write_kv, n_items);
  else if (dtype == LLMI_DTYPE_BF16)
    return launch_pdl(PDL_ROPE, rope_store_kernel<__nv_bfloat16>, (unsigned)blocks, ROPE_WARPS * 32, 0, stream,
                      (__nv_bfloat16*)qkv, ld, inv_freq, rotary_dim, tok_seq, tok_pos, kv, (__nv_bfloat16*)k_cache,
                      (__nv_bfloat16*)v_cache, n_heads, write_kv, n_items);
  else
    return LLMI_ERR_BAD_DTYPE;
  return launch_status();
}
