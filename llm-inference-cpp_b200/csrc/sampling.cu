// Next-token choice on the device: first-maximum argmax, and temperature / top-k / top-p
// sampling with an inverse-CDF draw.
//
// Reference semantics (src/model/sampling.cpp:11-76; include/llmi/model/sampling.hpp:11-24):
//   p = softmax(logits / temperature); order by p descending, equal values by ascending id;
//   keep the first k (top_k == 0 or > n keeps all); if top_p < 1 keep the shortest prefix whose
//   running sum reaches top_p (never fewer than one); renormalise by the kept sum; walk ids in
//   ascending order and return the first id whose running sum reaches u.
// Argmax returns the first maximum (src/model/transformer.cpp:22-24).
//
// No sort is done.  The kept set is { p > thr } plus the first n_eq ids with p == thr, and
// (thr, n_eq) is found by building thr's bit pattern from the top bit down with counting
// (top-k) or mass (top-p) passes: probabilities are non-negative floats, so their bit patterns
// order like their values.  Counts are integers and masses are summed in double in a fixed
// order, so a row's result does not depend on which other rows are in the launch.
//
// `probs` is caller-provided scratch of n_rows * vocab floats.
#include <math.h>

#include "common.cuh"

namespace llmi {

constexpr int SAMPLE_THREADS = 1024;

__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_kernel(const float* __restrict__ logits, long ld, int vocab, int32_t* __restrict__ out) {
  __shared__ float best_v[32];
  __shared__ int best_i[32];
  pdl_launch_dependents();
  pdl_wait();
  const float* row = logits + (size_t)blockIdx.x * ld;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  if ((vocab & 3) == 0 && (((uintptr_t)row) & 15) == 0) {
    const float4* r4 = reinterpret_cast<const float4*>(row);
    for (int i = threadIdx.x; i < (vocab >> 2); i += blockDim.x) {   // ascending i: the first maximum stays
      const float4 v = r4[i];
      if (bi == 0x7fffffff || v.x > bv) { bv = v.x; bi = 4 * i; }
      if (v.y > bv) { bv = v.y; bi = 4 * i + 1; }
      if (v.z > bv) { bv = v.z; bi = 4 * i + 2; }
      if (v.w > bv) { bv = v.w; bi = 4 * i + 3; }
    }
  } else {
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const float v = row[i];
      if (bi == 0x7fffffff || v > bv) { bv = v; bi = i; }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
      if (best_v[w] > bv || (best_v[w] == bv && best_i[w] < bi)) { bv = best_v[w]; bi = best_i[w]; }
    out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
  }
}

// Block-wide reductions in a fixed order: lanes by butterfly, then the warps' results by butterfly again in
// every warp (no thread walks over 32 values one by one).  Every thread gets the result.
struct BlockReduce {
  double* d;   // [32]
  long long* n;  // [32]
  __device__ double sum(double v) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) d[warp] = v;
    __syncthreads();
    double t = lane < nw ? d[lane] : 0.0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    return t;
  }
  __device__ long long count(long long v) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) n[warp] = v;
    __syncthreads();
    long long t = lane < nw ? n[lane] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    return t;
  }
  __device__ float max(float v) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) d[warp] = (double)v;
    __syncthreads();
    return warp_max(lane < nw ? (float)d[lane] : -INFINITY);
  }
  // Exclusive prefix sums over the threads of the block in thread order (and the total): lanes by shuffles,
  // then the warps' totals the same way.  `buf` holds 32 values.
  template <typename V>
  __device__ V exclusive_scan(V v, V* buf, V* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    V incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const V up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    __syncthreads();
    if (lane == 31) buf[warp] = incl;
    __syncthreads();
    V w = lane < nw ? buf[lane] : V(0);
    V wincl = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const V up = __shfl_up_sync(0xffffffffu, wincl, o);
      if (lane >= o) wincl += up;
    }
    const V warp_base = __shfl_sync(0xffffffffu, wincl - w, warp);
    *total = __shfl_sync(0xffffffffu, wincl, nw - 1);
    return warp_base + (incl - v);
  }
};

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, long ld, int vocab, float temperature, int top_k, float top_p,
              const double* __restrict__ uniforms, float* __restrict__ probs, int32_t* __restrict__ out, int probs_in_smem) {
  __shared__ double red_d[32];
  __shared__ long long red_n[32];
  __shared__ int result_first, result_last;
  BlockReduce red{red_d, red_n};
  const int tid = threadIdx.x, nthr = blockDim.x;
  const float* row = logits + (size_t)blockIdx.x * ld;
  // The probabilities are read some seventy times (two threshold searches bit by bit, scans): they live in
  // shared memory when the vocabulary fits there (`probs_in_smem`), else in the caller's scratch.
  extern __shared__ float smem_probs[];
  float* p = probs_in_smem ? smem_probs : probs + (size_t)blockIdx.x * vocab;
  const uint32_t* pb = reinterpret_cast<const uint32_t*>(p);

  // softmax(logits / temperature), denominator in double
  float mx = -INFINITY;
  for (int i = tid; i < vocab; i += nthr) mx = fmaxf(mx, row[i] / temperature);
  mx = red.max(mx);
  double part = 0;
  for (int i = tid; i < vocab; i += nthr) {
    const float e = expf(row[i] / temperature - mx);
    p[i] = e;
    part += (double)e;
  }
  const double denom = red.sum(part);
  const float inv = (float)(1.0 / denom);
  for (int i = tid; i < vocab; i += nthr) p[i] *= inv;
  __syncthreads();

  // top-k: thr_k = the k-th largest value; n_eq = how many of the ties at thr_k are kept
  const long long k = (top_k <= 0 || top_k > vocab) ? vocab : top_k;
  uint32_t thr = 0;
  long long n_eq;
  if (k < vocab) {
    for (int bit = 30; bit >= 0; --bit) {  // bit 31 is the sign: never set
      const uint32_t cand = thr | (1u << bit);
      long long c = 0;
      for (int i = tid; i < vocab; i += nthr) c += pb[i] >= cand;
      if (red.count(c) >= k) thr = cand;
    }
    long long c = 0;
    for (int i = tid; i < vocab; i += nthr) c += pb[i] > thr;
    n_eq = k - red.count(c);
  } else {
    long long c = 0;
    for (int i = tid; i < vocab; i += nthr) c += pb[i] == 0u;
    n_eq = red.count(c);  // thr = 0: everything is kept
  }

  // top-p inside the top-k set
  if (top_p < 1.0f) {
    const uint32_t thr_k = thr;
    const long long n_eq_k = n_eq;
    const double tie_mass_k = (double)n_eq_k * (double)__uint_as_float(thr_k);
    double m = 0;
    for (int i = tid; i < vocab; i += nthr) m += pb[i] > thr_k ? (double)p[i] : 0.0;
    const double total_k = red.sum(m) + tie_mass_k;
    if (total_k >= (double)top_p) {
      // largest value v (>= thr_k) with mass{p >= v, in the set} >= top_p
      uint32_t t2 = 0;
      for (int bit = 30; bit >= 0; --bit) {
        const uint32_t cand = t2 | (1u << bit);
        double mm = 0;
        for (int i = tid; i < vocab; i += nthr) mm += (pb[i] >= cand && pb[i] > thr_k) ? (double)p[i] : 0.0;
        mm = red.sum(mm);
        if (cand <= thr_k) mm += tie_mass_k;
        if (mm >= (double)top_p) t2 = cand;
      }
      if (t2 < thr_k) t2 = thr_k;
      double mg = 0;
      long long ce = 0;
      for (int i = tid; i < vocab; i += nthr) {
        mg += pb[i] > t2 ? (double)p[i] : 0.0;
        ce += pb[i] == t2;
      }
      mg = red.sum(mg);
      long long avail = red.count(ce);
      if (t2 == thr_k) avail = n_eq_k;
      const double tv = (double)__uint_as_float(t2);
      long long need = 1;
      double cum = mg + tv;
      while (cum < (double)top_p && need < avail) { cum += tv; ++need; }
      thr = t2;
      n_eq = need;
    }
  }

  // kept set = { p > thr } + the first n_eq ids with p == thr.  Each thread owns a contiguous
  // id range; ranks of ties and running sums come from scans over the threads in id order.
  const int chunk = (vocab + nthr - 1) / nthr;
  const int i0 = tid * chunk, i1 = min(vocab, i0 + chunk);
  int eq_local = 0;
  for (int i = i0; i < i1; ++i) eq_local += pb[i] == thr;
  long long eq_total;
  int eq_rank = (int)red.exclusive_scan<long long>((long long)eq_local, red_n, &eq_total);
  const int eq_rank0 = eq_rank;
  double local = 0;
  for (int i = i0; i < i1; ++i) {
    if (pb[i] > thr) local += (double)p[i];
    else if (pb[i] == thr) { if (eq_rank < n_eq) local += (double)p[i]; ++eq_rank; }
  }
  if (tid == 0) { result_first = 0x7fffffff; result_last = -1; }
  double kept;
  const double mass_before = red.exclusive_scan<double>(local, red_d, &kept);
  const double target = uniforms[blockIdx.x] * kept;
  __syncthreads();        // result_first / result_last are set
  double cum = mass_before;
  eq_rank = eq_rank0;
  int first = 0x7fffffff, last = -1;
  for (int i = i0; i < i1; ++i) {
    bool in = false;
    if (pb[i] > thr) in = true;
    else if (pb[i] == thr) { in = eq_rank < n_eq; ++eq_rank; }
    if (!in || p[i] <= 0.f) continue;
    cum += (double)p[i];
    last = i;
    if (cum >= target && first == 0x7fffffff) first = i;
  }
  if (first != 0x7fffffff) atomicMin(&result_first, first);
  if (last >= 0) atomicMax(&result_last, last);
  __syncthreads();
  if (tid == 0) {
    int r = result_first;
    if (r == 0x7fffffff) r = result_last >= 0 ? result_last : 0;
    out[blockIdx.x] = r;
  }
}

}  // namespace llmi

using namespace llmi;

LLMI_EXPORT int llmi_argmax(const float* logits, long ld, int n_rows, int vocab, int32_t* out, cudaStream_t stream) {
  if (n_rows <= 0 || vocab <= 0) return LLMI_ERR_BAD_SIZE;
  return launch_pdl(PDL_SMALL, argmax_kernel, n_rows, SAMPLE_THREADS, 0, stream, logits, ld, vocab, out);
}

// temperature must be > 0 (the caller maps temperature <= 0 to llmi_argmax, as the reference does).
LLMI_EXPORT int llmi_sample(const float* logits, long ld, int n_rows, int vocab, float temperature, int top_k,
                            float top_p, const double* uniforms, float* probs_scratch, int32_t* out,
                            cudaStream_t stream) {
  if (n_rows <= 0 || vocab <= 0) return LLMI_ERR_BAD_SIZE;
  if (!(temperature > 0.f)) return LLMI_ERR_UNSUPPORTED;
  // up to 200 KB of shared memory for a row's probabilities (one block per SM; a step has few rows)
  const size_t bytes = (size_t)vocab * sizeof(float);
  static int smem_max = -1;
  if (smem_max < 0) {
    int dev = 0, v = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    smem_max = v - 20 * 1024;     // the kernel's static arrays take 12.6 KB
    if (smem_max < 0) smem_max = 0;
    if (cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_max) != cudaSuccess) smem_max = 0;
  }
  const int in_smem = bytes <= (size_t)smem_max ? 1 : 0;
  sample_kernel<<<n_rows, SAMPLE_THREADS, in_smem ? bytes : 0, stream>>>(logits, ld, vocab, temperature, top_k, top_p, uniforms,
                                                                         probs_scratch, out, in_smem);
  return launch_status();
}
