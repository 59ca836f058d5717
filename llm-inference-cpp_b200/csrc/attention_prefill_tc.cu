// Prefill attention on the 5th-generation tensor cores (tcgen05), bf16, head size 64.
//
// Same operation as attention_prefill.cu (reference loop: src/model/transformer.cpp:263-282): causal
// grouped-query attention of the prompts of a step over their cache pages.  A block takes 128 queries of
// one sequence and one query head and walks the pages (64 keys) the queries can see:
//
//   S_j = Q · K_jᵀ        tcgen05.mma, M = 128 queries on TMEM lanes, N = 64 keys on TMEM columns
//   softmax               four warps, ONE QUERY ROW PER THREAD: tcgen05.ld of the row, mask, running
//                         maximum, exp2, sum — no shuffles; P_j goes to shared memory as bf16 in the
//                         swizzled layout an MMA A-operand wants
//   O_j = P_j · V_j       tcgen05.mma again (V is the MN-major B operand, straight from the cache page)
//   O  += O_j             the row's thread reads O_j from TMEM and adds it to its fp32 registers, scaled
//                         by the running-maximum correction — the accumulator never lives in TMEM, so
//                         nothing there is read, rescaled and written back
//
// Roles: warp 0 = TMA producer (Q once, then K_j / V_j pages into a ring), warp 1 = TMEM allocation and MMA
// issue, warps 2..5 = softmax and output.  S and O_j are double-buffered in TMEM and P in shared memory, so
// S_{j+1} is computed while the softmax of S_j runs.  Every wait is bounded (see sm100.cuh).
#include <cuda.h>
#include <math.h>

#include "common.cuh"
#include "sm100.cuh"

namespace llmi {

constexpr int FT_BM = 128, FT_PAGE = 64, FT_HD = 64;
constexpr int FT_STAGES = 3;
constexpr int FT_THREADS = 192;
constexpr int FT_TILE = FT_PAGE * FT_HD * 2;          // 8 KB: one K or V page tile
constexpr int FT_QBYTES = FT_BM * FT_HD * 2;          // 16 KB
constexpr int FT_PBYTES = FT_BM * FT_PAGE * 2;        // 16 KB
constexpr int FT_SMEM = FT_QBYTES + FT_STAGES * 2 * FT_TILE + 2 * FT_PBYTES + 1024 + 256;

struct PrefillTcParams {
  __nv_bfloat16* out;
  long ldo;
  const int32_t* seq_pages;
  const int32_t* seq_q_start;
  const int32_t* seq_kv_len;
  int pages_stride;
  int n_seqs;
  int n_heads, n_kv_heads;
  float scale_log2;
  int window;
  int* error_flag;
};

__device__ __forceinline__ void ft_tma(uint32_t dst, const CUtensorMap* map, int col, int row, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(col), "r"(row)
      : "memory");
}
// K-major operand tile (rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart)
__device__ __forceinline__ uint64_t ft_desc(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}
__device__ __forceinline__ void ft_mma(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void ft_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 16 consecutive fp32 columns of this thread's TMEM lane; no wait
__device__ __forceinline__ void ft_ld16(uint32_t taddr, float* v) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void ft_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__global__ void __launch_bounds__(FT_THREADS, 2)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, PrefillTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem = base;
  const uint32_t kv_smem = base + FT_QBYTES;                        // stage s: K at +s*16K, V at +s*16K+8K
  const uint32_t p_smem = kv_smem + FT_STAGES * 2 * FT_TILE;        // two P buffers
  const uint32_t bars = p_smem + 2 * FT_PBYTES;
  // barriers: q_full, kv_full[3], kv_empty[3], s_full[2], s_free[2], p_ready[2], o_full[2], o_free[2], tmem slot
  const uint32_t q_full = bars;
  auto kv_full = [&](int s) { return bars + 8u * (1 + s); };
  auto kv_empty = [&](int s) { return bars + 8u * (1 + FT_STAGES + s); };
  auto s_full = [&](int b) { return bars + 8u * (1 + 2 * FT_STAGES + b); };
  auto s_free = [&](int b) { return bars + 8u * (3 + 2 * FT_STAGES + b); };
  auto p_ready = [&](int b) { return bars + 8u * (5 + 2 * FT_STAGES + b); };
  auto o_full = [&](int b) { return bars + 8u * (7 + 2 * FT_STAGES + b); };
  auto o_free = [&](int b) { return bars + 8u * (9 + 2 * FT_STAGES + b); };
  const uint32_t tmem_slot = bars + 8u * (11 + 2 * FT_STAGES);

  pdl_launch_dependents();
  // which sequence and which block of 128 queries (late blocks, which see more keys, come first)
  int mb = gridDim.x - 1 - blockIdx.x;
  int seq = 0, q_start = 0, q_len = 0;
  for (; seq < p.n_seqs; ++seq) {
    q_start = p.seq_q_start[seq];
    q_len = p.seq_q_start[seq + 1] - q_start;
    const int nb = (q_len + FT_BM - 1) / FT_BM;
    if (mb < nb) break;
    mb -= nb;
  }
  if (seq >= p.n_seqs) return;
  const int head = blockIdx.y;
  const int kvh = head / (p.n_heads / p.n_kv_heads);
  const int kv_len = p.seq_kv_len[seq];
  const int pos0 = kv_len - q_len;
  const int m0 = mb * FT_BM;
  const int rows_here = min(FT_BM, q_len - m0);
  const int first_q = pos0 + m0, last_q = pos0 + m0 + rows_here - 1;
  const int lo_key = (p.window > 0 && first_q - p.window + 1 > 0) ? first_q - p.window + 1 : 0;
  const int pg_first = lo_key / FT_PAGE, pg_last = last_q / FT_PAGE;
  const int n_pg = pg_last - pg_first + 1;
  const int32_t* pages = p.seq_pages + (size_t)seq * p.pages_stride;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
    mbar_init(q_full, 1);
    for (int s = 0; s < FT_STAGES; ++s) {
      mbar_init(kv_full(s), 1);
      mbar_init(kv_empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(s_full(b), 1);
      mbar_init(s_free(b), 4);
      mbar_init(p_ready(b), 4);
      mbar_init(o_full(b), 1);
      mbar_init(o_free(b), 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(256));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  uint32_t tmem;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem) : "r"(tmem_slot));
  // TMEM columns: S buffers at 0 and 64, O_j buffers at 128 and 192

  if (warp == 0) {
    if (lane == 0) {
      // ---- producer ----
      mbar_expect_tx(q_full, FT_QBYTES);
      ft_tma(q_smem, &map_q, head * FT_HD, q_start + m0, q_full);
      for (int j = 0; j < n_pg; ++j) {
        const int s = j % FT_STAGES;
        if (j >= FT_STAGES && !mbar_wait(kv_empty(s), ((j / FT_STAGES) - 1) & 1, p.error_flag, 41)) break;
        const int row = (pages[pg_first + j] * p.n_kv_heads + kvh) * FT_PAGE;
        mbar_expect_tx(kv_full(s), 2 * FT_TILE);
        ft_tma(kv_smem + s * 2 * FT_TILE, &map_k, 0, row, kv_full(s));
        ft_tma(kv_smem + s * 2 * FT_TILE + FT_TILE, &map_v, 0, row, kv_full(s));
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer ----
      // S: A = Q (K-major), B = K page (K-major), N = 64.  O_j: A = P (K-major), B = V page (MN-major), N = 64.
      const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(64 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      const uint32_t idesc_o = idesc_s | (1u << 16);
      auto issue_s = [&](int j) {
        const uint64_t a = ft_desc(q_smem), b = ft_desc(kv_smem + (j % FT_STAGES) * 2 * FT_TILE);
#pragma unroll
        for (int k4 = 0; k4 < FT_HD / 16; ++k4) ft_mma(tmem + (uint32_t)((j & 1) * 64), a + 2 * k4, b + 2 * k4, idesc_s, k4 > 0);
        ft_commit(s_full(j & 1));
      };
      bool ok = mbar_wait(q_full, 0, p.error_flag, 42) && mbar_wait(kv_full(0), 0, p.error_flag, 43);
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        issue_s(0);
      }
      for (int j = 0; j < n_pg && ok; ++j) {
        if (j + 1 < n_pg) {
          ok = mbar_wait(kv_full((j + 1) % FT_STAGES), ((j + 1) / FT_STAGES) & 1, p.error_flag, 44);
          if (ok && j + 1 >= 2) ok = mbar_wait(s_free((j + 1) & 1), (((j + 1) >> 1) - 1) & 1, p.error_flag, 45);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          issue_s(j + 1);
        }
        ok = mbar_wait(p_ready(j & 1), (j >> 1) & 1, p.error_flag, 46);
        if (ok && j >= 2) ok = mbar_wait(o_free(j & 1), ((j >> 1) - 1) & 1, p.error_flag, 47);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t a = ft_desc(p_smem + (j & 1) * FT_PBYTES);
        const uint64_t b = ft_desc(kv_smem + (j % FT_STAGES) * 2 * FT_TILE + FT_TILE);
#pragma unroll
        for (int k4 = 0; k4 < FT_PAGE / 16; ++k4)   // 16 keys further: +32 bytes in a P row, +16 rows of 128 bytes in V
          ft_mma(tmem + (uint32_t)(128 + (j & 1) * 64), a + 2 * k4, b + (uint64_t)(k4 * ((16 * 128) >> 4)), idesc_o, k4 > 0);
        ft_commit(o_full(j & 1));
        ft_commit(kv_empty(j % FT_STAGES));
      }
    }
  } else {
    // ---- softmax and output: one query row per thread ----
    const int quad = warp & 3;
    const int row = quad * 32 + lane;                 // row of the 128-query block = TMEM lane
    const int qrow = m0 + row;
    const bool row_ok = qrow < q_len;
    const int qpos = pos0 + qrow;
    const uint32_t t_lane = tmem + ((uint32_t)(quad * 32) << 16);
    float o[FT_HD];
#pragma unroll
    for (int d = 0; d < FT_HD; ++d) o[d] = 0.f;
    float m_run = -INFINITY, l_run = 0.f, corr = 1.f;
    bool ok = true;
    for (int j = 0; j < n_pg && ok; ++j) {
      const int b = j & 1;
      ok = mbar_wait(s_full(b), (j >> 1) & 1, p.error_flag, 48);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float sc[FT_PAGE];
#pragma unroll
      for (int c = 0; c < FT_PAGE; c += 16) ft_ld16(t_lane + (uint32_t)(b * 64 + c), sc + c);
      ft_ld_wait();
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(s_free(b));
      const int key0 = (pg_first + j) * FT_PAGE;
      const bool need_mask = (key0 + FT_PAGE - 1 > first_q) || (p.window > 0);
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < FT_PAGE; ++c) {
        float v = sc[c] * p.scale_log2;
        const int key = key0 + c;
        if (need_mask && (key > qpos || (p.window > 0 && key < qpos - p.window + 1))) v = -INFINITY;
        sc[c] = v;
        mx = fmaxf(mx, v);
      }
      const float m_new = fmaxf(m_run, mx);
      corr = (m_new == -INFINITY) ? 1.f : fast_exp2(m_run - m_new);
      m_run = m_new;
      float sum = 0.f;
      uint32_t packed[FT_PAGE / 2];
#pragma unroll
      for (int c = 0; c < FT_PAGE; c += 2) {
        const float p0 = (m_new == -INFINITY) ? 0.f : fast_exp2(sc[c] - m_new);
        const float p1 = (m_new == -INFINITY) ? 0.f : fast_exp2(sc[c + 1] - m_new);
        sum += p0 + p1;
        __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
        packed[c >> 1] = *reinterpret_cast<uint32_t*>(&h);
      }
      l_run = l_run * corr + sum;
#pragma unroll
      for (int d = 0; d < FT_HD; ++d) o[d] *= corr;
      // P row -> shared memory, swizzled as an MMA operand (chunk c of row r at r*128 + ((c ^ (r & 7)) << 4))
      const uint32_t prow = p_smem + b * FT_PBYTES + (uint32_t)row * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c)
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(prow + (uint32_t)(((c ^ (row & 7)) << 4))),
                     "r"(packed[4 * c]), "r"(packed[4 * c + 1]), "r"(packed[4 * c + 2]), "r"(packed[4 * c + 3])
                     : "memory");
      if (key0 + FT_PAGE > kv_len) {
        // The sequence ends inside this page: value rows behind its end are cleared so that their zero
        // probabilities cannot meet a NaN.  (The page is in shared memory: S_j was computed from it.)
        const uint32_t v_tile = kv_smem + (j % FT_STAGES) * 2 * FT_TILE + FT_TILE;
        const int first_bad = kv_len - key0;
        for (int idx = (warp - 2) * 32 + lane; idx < (FT_PAGE - first_bad) * 8; idx += 128) {
          const int r = first_bad + (idx >> 3), ch = idx & 7;
          asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(v_tile + (uint32_t)(r * 128 + (ch << 4))), "r"(0u) : "memory");
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> visible to the MMA's reads
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready(b));
      if (j >= 1) {
        // O_{j-1} = P_{j-1} V_{j-1} is relative to the maximum before this page: scale it like the registers
        const int pb = (j - 1) & 1;
        ok = mbar_wait(o_full(pb), ((j - 1) >> 1) & 1, p.error_flag, 49);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int c = 0; c < FT_HD; c += 16) {
          float t[16];
          ft_ld16(t_lane + (uint32_t)(128 + pb * 64 + c), t);
          ft_ld_wait();
#pragma unroll
          for (int e = 0; e < 16; ++e) o[c + e] = fmaf(corr, t[e], o[c + e]);
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(o_free(pb));
      }
    }
    if (ok) {
      const int pb = (n_pg - 1) & 1;
      ok = mbar_wait(o_full(pb), ((n_pg - 1) >> 1) & 1, p.error_flag, 50);
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int c = 0; c < FT_HD; c += 16) {
          float t[16];
          ft_ld16(t_lane + (uint32_t)(128 + pb * 64 + c), t);
          ft_ld_wait();
#pragma unroll
          for (int e = 0; e < 16; ++e) o[c + e] += t[e];
        }
        if (row_ok) {
          const float inv = 1.f / l_run;
          __nv_bfloat16* dst = p.out + (size_t)(q_start + qrow) * p.ldo + (size_t)head * FT_HD;
#pragma unroll
          for (int c = 0; c < FT_HD; c += 8) {
            uint4 v;
            __nv_bfloat162 h0 = __floats2bfloat162_rn(o[c] * inv, o[c + 1] * inv), h1 = __floats2bfloat162_rn(o[c + 2] * inv, o[c + 3] * inv);
            __nv_bfloat162 h2 = __floats2bfloat162_rn(o[c + 4] * inv, o[c + 5] * inv), h3 = __floats2bfloat162_rn(o[c + 6] * inv, o[c + 7] * inv);
            v.x = *reinterpret_cast<uint32_t*>(&h0);
            v.y = *reinterpret_cast<uint32_t*>(&h1);
            v.z = *reinterpret_cast<uint32_t*>(&h2);
            v.w = *reinterpret_cast<uint32_t*>(&h3);
            *reinterpret_cast<uint4*>(dst + c) = v;
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256));
}

typedef CUresult (*FtEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// A bf16 matrix [rows, cols] with row pitch ld (elements): tiles of [box_rows, 64 columns], 128-byte swizzle.
static int ft_make_map(CUtensorMap* map, const void* ptr, long rows, long cols, long ld, int box_rows) {
  static FtEncodeFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return LLMI_ERR_DRIVER;
    fn = (FtEncodeFn)sym;
  }
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS
             ? LLMI_OK
             : LLMI_ERR_DRIVER;
}

}  // namespace llmi

using namespace llmi;

LLMI_EXPORT int llmi_attention_prefill_tc_supported(int head_dim) { return head_dim == 64; }

// q: [n_tokens, >= n_heads*64] rotated queries (row pitch ldq, 16-byte aligned rows); otherwise as llmi_attention_prefill.
LLMI_EXPORT int llmi_attention_prefill_tc(const void* q, long ldq, long n_tokens, void* out, long ldo, const void* k_cache,
                                          const void* v_cache, long n_cache_pages, const int32_t* seq_pages,
                                          int pages_stride, const int32_t* seq_q_start, const int32_t* seq_kv_len,
                                          int n_seqs, int n_blocks, int n_heads, int n_kv_heads, int head_dim, float scale,
                                          int window, int* error_flag, cudaStream_t stream) {
  if (n_seqs <= 0 || n_blocks <= 0 || n_heads <= 0 || n_kv_heads <= 0 || n_cache_pages <= 0 || n_tokens <= 0) return LLMI_ERR_BAD_SIZE;
  if (n_heads % n_kv_heads || n_heads > 65535) return LLMI_ERR_BAD_SIZE;
  if (head_dim != FT_HD) return LLMI_ERR_UNSUPPORTED;
  if (((uintptr_t)q & 15) || (ldq & 7) || ((uintptr_t)out & 15) || (ldo & 7) || ((uintptr_t)k_cache & 15) ||
      ((uintptr_t)v_cache & 15))
    return LLMI_ERR_ALIGN;
  const long rows = n_cache_pages * n_kv_heads * FT_PAGE;
  if (rows > 0x7fffffffL) return LLMI_ERR_BAD_SIZE;
  CUtensorMap mq, mk, mv;
  int rc = ft_make_map(&mq, q, n_tokens, (long)n_heads * FT_HD, ldq, FT_BM);
  if (rc != LLMI_OK) return rc;
  rc = ft_make_map(&mk, k_cache, rows, FT_HD, FT_HD, FT_PAGE);
  if (rc != LLMI_OK) return rc;
  rc = ft_make_map(&mv, v_cache, rows, FT_HD, FT_HD, FT_PAGE);
  if (rc != LLMI_OK) return rc;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FT_SMEM) != cudaSuccess)
      return LLMI_ERR_LAUNCH;
    configured = true;
  }
  PrefillTcParams p{(__nv_bfloat16*)out, ldo, seq_pages, seq_q_start, seq_kv_len, pages_stride, n_seqs, n_heads,
                    n_kv_heads, scale * 1.4426950408889634f, window, error_flag};
  dim3 grid(n_blocks, n_heads);
  attention_prefill_tc_kernel<<<grid, FT_THREADS, FT_SMEM, stream>>>(mq, mk, mv, p);
  return launch_status();
}
