// Prefill attention: the tokens of several prompts attend causally over their sequences' cache pages
// (bf16, head size 64 or 128), flash style on the tensor cores.
//
// Reference loop: src/model/transformer.cpp:263-282 — for query head hh the kv head is hh / group,
// score[s] = dot(q, k_s) * scale for the keys s the query may see, softmax, weighted sum of values.
// Here a block takes 128 consecutive queries of one sequence and one query head; keys and values
// come one cache page (64 positions) at a time:
//   * a page's K and V tiles are fetched by TMA (cp.async.bulk.tensor, 128-byte swizzle) into a ring
//     of shared-memory stages, completion on mbarriers, so the fetch of later pages overlaps the math;
//   * S = Q·Kᵀ and O += P·V run on mma.sync m16n8k16 (bf16 in, fp32 out), 16 query rows per warp;
//   * softmax is the running-maximum form in fp32 registers (exp2 with the scale folded in), and
//     only pages a query can see are visited (causal; `window` > 0 also bounds them from below).
// The sequences of a step are ragged: block b finds its (sequence, 128-query block) from the
// per-sequence query offsets.  Long blocks (late queries) are issued first.
#include <cuda.h>
#include <math.h>

#include "common.cuh"
#include "sm100.cuh"

namespace llmi {

constexpr int PF_BM = 128;      // queries per block
constexpr int PF_PAGE = 64;     // keys per step = the cache's page size
constexpr int PF_THREADS = 256;
constexpr int PF_STAGES = 3;

struct PrefillParams {
  const __nv_bfloat16* q;   // [tokens, >= n_heads*HD], row pitch ldq (already rotated)
  long ldq;
  __nv_bfloat16* out;       // [tokens, n_heads*HD], row pitch ldo
  long ldo;
  const int32_t* seq_pages;    // [n_seqs, pages_stride]
  const int32_t* seq_q_start;  // [n_seqs + 1]
  const int32_t* seq_kv_len;   // [n_seqs] length after this step
  int pages_stride;
  int n_seqs;
  int n_heads, n_kv_heads;
  float scale_log2;            // scale * log2(e)
  int window;
  int* error_flag;
};

__device__ __forceinline__ void mma_bf16(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void tma_load_tile(uint32_t dst, const CUtensorMap* map, int col, int row, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(col), "r"(row)
      : "memory");
}
// Byte offset of element (row, col) in a [64 rows][64 cols] bf16 tile stored with the 128-byte swizzle.
__device__ __forceinline__ uint32_t swz(int row, int col) {
  return (uint32_t)(row * 128 + ((((col >> 3) ^ (row & 7)) << 4) | ((col & 7) << 1)));
}

template <int HD>
__global__ void __launch_bounds__(PF_THREADS, HD <= 64 ? 2 : 1)
attention_prefill_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                         PrefillParams p) {
  constexpr int NSUB = HD / 64;                 // 64-column sub-tiles of a page tile
  constexpr int SUB_BYTES = PF_PAGE * 64 * 2;   // 8 KB
  constexpr int TILE_BYTES = NSUB * SUB_BYTES;
  constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = base + PF_STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bars + 8u * s; };

  pdl_launch_dependents();
  // which sequence and which block of 128 queries: late blocks, which see more keys, come first, for ALL heads (the
  // head is the fast grid index: a long block that starts late is the kernel's tail)
  int mb = gridDim.y - 1 - blockIdx.y;
  int seq = 0, q_start = 0, q_len = 0;
  for (; seq < p.n_seqs; ++seq) {
    q_start = p.seq_q_start[seq];
    q_len = p.seq_q_start[seq + 1] - q_start;
    const int nb = (q_len + PF_BM - 1) / PF_BM;
    if (mb < nb) break;
    mb -= nb;
  }
  if (seq >= p.n_seqs) return;
  const int head = blockIdx.x;
  const int kvh = head / (p.n_heads / p.n_kv_heads);
  const int kv_len = p.seq_kv_len[seq];
  const int pos0 = kv_len - q_len;              // position of the sequence's first query in this step
  const int m0 = mb * PF_BM;
  const int rows_here = min(PF_BM, q_len - m0);
  const int first_q = pos0 + m0, last_q = pos0 + m0 + rows_here - 1;
  const int lo_key = (p.window > 0 && first_q - p.window + 1 > 0) ? first_q - p.window + 1 : 0;
  const int pg_first = lo_key / PF_PAGE, pg_last = last_q / PF_PAGE;
  const int n_pg = pg_last - pg_first + 1;
  const int32_t* pages = p.seq_pages + (size_t)seq * p.pages_stride;

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
    for (int s = 0; s < PF_STAGES; ++s) mbar_init(full_bar(s), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  auto issue = [&](int i) {   // thread 0: fetch page i of this block's range into its stage
    const int s = i % PF_STAGES;
    const int row = (pages[pg_first + i] * p.n_kv_heads + kvh) * PF_PAGE;
    mbar_expect_tx(full_bar(s), STAGE_BYTES);
#pragma unroll
    for (int u = 0; u < NSUB; ++u) {
      tma_load_tile(base + s * STAGE_BYTES + u * SUB_BYTES, &map_k, u * 64, row, full_bar(s));
      tma_load_tile(base + s * STAGE_BYTES + TILE_BYTES + u * SUB_BYTES, &map_v, u * 64, row, full_bar(s));
    }
  };
  if (threadIdx.x == 0)
    for (int i = 0; i < PF_STAGES - 1 && i < n_pg; ++i) issue(i);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int row0 = m0 + warp * 16 + g, row1 = row0 + 8;           // this thread's two query rows
  const bool v0 = row0 < q_len, v1 = row1 < q_len;
  const int qpos0 = pos0 + row0, qpos1 = pos0 + row1;

  // Q fragments (A operand), straight from global memory
  uint32_t qa[HD / 16][4];
  {
    const __nv_bfloat16* q0 = p.q + (size_t)(q_start + row0) * p.ldq + (size_t)head * HD;
    const __nv_bfloat16* q1 = p.q + (size_t)(q_start + row1) * p.ldq + (size_t)head * HD;
#pragma unroll
    for (int kc = 0; kc < HD / 16; ++kc) {
      qa[kc][0] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + kc * 16 + 2 * t) : 0u;
      qa[kc][1] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + kc * 16 + 2 * t) : 0u;
      qa[kc][2] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + kc * 16 + 8 + 2 * t) : 0u;
      qa[kc][3] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + kc * 16 + 8 + 2 * t) : 0u;
    }
  }
  float o[HD / 8][4];
#pragma unroll
  for (int dc = 0; dc < HD / 8; ++dc)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[dc][e] = 0.f;
  float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};

  bool ok = true;
  for (int i = 0; i < n_pg; ++i) {
    const int s = i % PF_STAGES;
    if (threadIdx.x == 0 && i + PF_STAGES - 1 < n_pg) issue(i + PF_STAGES - 1);   // its stage was freed by the sync below
    ok = mbar_wait(full_bar(s), (i / PF_STAGES) & 1, p.error_flag, 21);
    if (!ok) break;
    const uint32_t k_tile = base + s * STAGE_BYTES, v_tile = k_tile + TILE_BYTES;
    const int key0 = (pg_first + i) * PF_PAGE;
    if (key0 + PF_PAGE > kv_len) {
      // The sequence ends inside this page.  What lies behind its end is not the sequence's: those
      // value rows are cleared, so that their zero probabilities cannot meet a NaN or an infinity.
      const int first_bad = kv_len - key0;
      for (int idx = threadIdx.x; idx < (PF_PAGE - first_bad) * (HD / 8); idx += PF_THREADS) {
        const int row = first_bad + idx / (HD / 8), ch = idx % (HD / 8);
        asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(v_tile + (ch / 8) * SUB_BYTES + (uint32_t)(row * 128 + ((ch & 7) << 4))), "r"(0u)
                     : "memory");
      }
      __syncthreads();
    }

    // S = Q Kᵀ for 16 rows x 64 keys
    float sc[8][4];
#pragma unroll
    for (int nc = 0; nc < 8; ++nc)
#pragma unroll
      for (int e = 0; e < 4; ++e) sc[nc][e] = 0.f;
#pragma unroll
    for (int kc = 0; kc < HD / 16; ++kc) {
      const uint32_t sub = k_tile + (kc / 4) * SUB_BYTES;
#pragma unroll
      for (int nc = 0; nc < 8; nc += 2) {
        // one ldmatrix.x4 = the B fragments (k 0-7 and k 8-15 of this chunk) of two blocks of 8 keys
        const int mtx = lane >> 3, r = lane & 7;
        const int row = (nc + (mtx >> 1)) * 8 + r, kch = (kc % 4) * 2 + (mtx & 1);
        uint32_t b0, b1, b2, b3;
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                     : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3)
                     : "r"(sub + (uint32_t)(row * 128 + ((kch ^ (row & 7)) << 4))));
        mma_bf16(sc[nc], qa[kc], b0, b1);
        mma_bf16(sc[nc + 1], qa[kc], b2, b3);
      }
    }
    // mask, running maximum, probabilities
    // Running maximum on the raw scores (the scale is positive), masked only where a page can hold keys a
    // query may not see; the scale enters with the subtraction of the maximum: p = 2^(s*scale - m*scale).
    const bool need_mask = (key0 + PF_PAGE - 1 > first_q) || (p.window > 0);
    float mx0 = -INFINITY, mx1 = -INFINITY;
    if (need_mask) {
#pragma unroll
      for (int nc = 0; nc < 8; ++nc)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = key0 + nc * 8 + 2 * t + (e & 1);
          const int qp = (e < 2) ? qpos0 : qpos1;
          if (key > qp || (p.window > 0 && key < qp - p.window + 1)) sc[nc][e] = -INFINITY;
        }
    }
#pragma unroll
    for (int nc = 0; nc < 8; ++nc) {
      mx0 = fmaxf(mx0, fmaxf(sc[nc][0], sc[nc][1]));
      mx1 = fmaxf(mx1, fmaxf(sc[nc][2], sc[nc][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(mrow[0], mx0 * p.scale_log2), mn1 = fmaxf(mrow[1], mx1 * p.scale_log2);   // scaled maxima
    const float c0 = (mn0 == -INFINITY) ? 1.f : fast_exp2(mrow[0] - mn0);
    const float c1 = (mn1 == -INFINITY) ? 1.f : fast_exp2(mrow[1] - mn1);
    mrow[0] = mn0;
    mrow[1] = mn1;
    if (__any_sync(0xffffffffu, c0 != 1.f || c1 != 1.f)) {   // the maximum settles after a few pages: then nothing to rescale
      lrow[0] *= c0;
      lrow[1] *= c1;
#pragma unroll
      for (int dc = 0; dc < HD / 8; ++dc) {
        o[dc][0] *= c0;
        o[dc][1] *= c0;
        o[dc][2] *= c1;
        o[dc][3] *= c1;
      }
    }
    const float nm0 = (mn0 == -INFINITY) ? 0.f : -mn0, nm1 = (mn1 == -INFINITY) ? 0.f : -mn1;
    uint32_t pa[4][4];
#pragma unroll
    for (int nc = 0; nc < 8; ++nc) {
      const float p0 = fast_exp2(fmaf(sc[nc][0], p.scale_log2, nm0));   // 2^(-inf) = 0 for masked keys
      const float p1 = fast_exp2(fmaf(sc[nc][1], p.scale_log2, nm0));
      const float p2 = fast_exp2(fmaf(sc[nc][2], p.scale_log2, nm1));
      const float p3 = fast_exp2(fmaf(sc[nc][3], p.scale_log2, nm1));
      lrow[0] += p0 + p1;
      lrow[1] += p2 + p3;
      pa[nc >> 1][(nc & 1) * 2 + 0] = pack_bf16(p0, p1);
      pa[nc >> 1][(nc & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
    // O += P V
#pragma unroll
    for (int kc = 0; kc < 4; ++kc) {
#pragma unroll
      for (int dc = 0; dc < HD / 8; dc += 2) {
        const int mtx = lane >> 3, r = lane & 7;
        const int key = kc * 16 + (mtx & 1) * 8 + r;
        const int dchunk = dc + (mtx >> 1);
        const uint32_t addr = v_tile + (dchunk / 8) * SUB_BYTES + (uint32_t)(key * 128 + (((dchunk & 7) ^ (key & 7)) << 4));
        uint32_t r0, r1, r2, r3;
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                     : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                     : "r"(addr));
        mma_bf16(o[dc], pa[kc], r0, r1);
        mma_bf16(o[dc + 1], pa[kc], r2, r3);
      }
    }
    fence_reads_before_async_writes();
    __syncthreads();   // every warp is done with stage s
  }
  if (!ok) return;

  lrow[0] += __shfl_xor_sync(0xffffffffu, lrow[0], 1);
  lrow[0] += __shfl_xor_sync(0xffffffffu, lrow[0], 2);
  lrow[1] += __shfl_xor_sync(0xffffffffu, lrow[1], 1);
  lrow[1] += __shfl_xor_sync(0xffffffffu, lrow[1], 2);
  const float inv0 = 1.f / lrow[0], inv1 = 1.f / lrow[1];
  __nv_bfloat16* o0 = p.out + (size_t)(q_start + row0) * p.ldo + (size_t)head * HD;
  __nv_bfloat16* o1 = p.out + (size_t)(q_start + row1) * p.ldo + (size_t)head * HD;
#pragma unroll
  for (int dc = 0; dc < HD / 8; ++dc) {
    if (v0) *reinterpret_cast<uint32_t*>(o0 + dc * 8 + 2 * t) = pack_bf16(o[dc][0] * inv0, o[dc][1] * inv0);
    if (v1) *reinterpret_cast<uint32_t*>(o1 + dc * 8 + 2 * t) = pack_bf16(o[dc][2] * inv1, o[dc][3] * inv1);
  }
}

typedef CUresult (*EncodeTiledFn2)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The cache of one layer as a matrix [pages * kv_heads * 64 rows, head_dim]: tiles of [64 rows, 64 cols].
static int make_cache_map(CUtensorMap* map, const void* ptr, long rows, int head_dim) {
  static EncodeTiledFn2 fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return LLMI_ERR_DRIVER;
    fn = (EncodeTiledFn2)sym;
  }
  const cuuint64_t dims[2] = {(cuuint64_t)head_dim, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)head_dim * 2};
  const cuuint32_t box[2] = {64, 64};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS
             ? LLMI_OK
             : LLMI_ERR_DRIVER;
}

template <int HD>
static int launch_prefill(const CUtensorMap& mk, const CUtensorMap& mv, const PrefillParams& p, int n_blocks,
                          cudaStream_t stream) {
  constexpr int SMEM = PF_STAGES * 2 * (HD / 64) * PF_PAGE * 64 * 2 + 1024 + 64;
  static PerDevice<bool> configured_on;
  bool& configured = configured_on.here();
  if (!configured) {
    if (cudaFuncSetAttribute(attention_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
      return LLMI_ERR_LAUNCH;
    configured = true;
  }
  if (n_blocks > 65535) return LLMI_ERR_BAD_SIZE;
  dim3 grid(p.n_heads, n_blocks);
  attention_prefill_kernel<HD><<<grid, PF_THREADS, SMEM, stream>>>(mk, mv, p);
  return launch_status();
}

}  // namespace llmi

using namespace llmi;

LLMI_EXPORT int llmi_attention_prefill_supported(int head_dim) { return head_dim == 64 || head_dim == 128; }

// n_blocks = sum over the step's sequences of ceil(query tokens / 128); n_cache_pages = pages of the layer's cache.
LLMI_EXPORT int llmi_attention_prefill(const void* q, long ldq, void* out, long ldo, const void* k_cache,
                                       const void* v_cache, long n_cache_pages, const int32_t* seq_pages,
                                       int pages_stride, const int32_t* seq_q_start, const int32_t* seq_kv_len,
                                       int n_seqs, int n_blocks, int n_heads, int n_kv_heads, int head_dim, float scale,
                                       int window, int* error_flag, cudaStream_t stream) {
  if (n_seqs <= 0 || n_blocks <= 0 || n_heads <= 0 || n_kv_heads <= 0 || n_cache_pages <= 0) return LLMI_ERR_BAD_SIZE;
  if (n_heads % n_kv_heads || n_heads > 65535) return LLMI_ERR_BAD_SIZE;
  if (!llmi_attention_prefill_supported(head_dim)) return LLMI_ERR_UNSUPPORTED;
  if (((uintptr_t)q & 3) || (ldq & 1) || ((uintptr_t)out & 3) || (ldo & 1) || ((uintptr_t)k_cache & 15) ||
      ((uintptr_t)v_cache & 15))
    return LLMI_ERR_ALIGN;
  const long rows = n_cache_pages * n_kv_heads * PF_PAGE;
  if (rows > 0x7fffffffL) return LLMI_ERR_BAD_SIZE;
  CUtensorMap mk, mv;
  int rc = make_cache_map(&mk, k_cache, rows, head_dim);
  if (rc != LLMI_OK) return rc;
  rc = make_cache_map(&mv, v_cache, rows, head_dim);
  if (rc != LLMI_OK) return rc;
  PrefillParams p{(const __nv_bfloat16*)q, ldq, (__nv_bfloat16*)out, ldo, seq_pages, seq_q_start, seq_kv_len,
                  pages_stride, n_seqs, n_heads, n_kv_heads, scale * 1.4426950408889634f, window, error_flag};
  return head_dim == 64 ? launch_prefill<64>(mk, mv, p, n_blocks, stream) : launch_prefill<128>(mk, mv, p, n_blocks, stream);
}
