// Prefill attention on the 5th-generation tensor cores (tcgen05), bf16, head size 64.
//
// Same operation as attention_prefill.cu (reference loop: src/model/transformer.cpp:263-282): causal
// grouped-query attention of the prompts of a step over their cache pages.  A block takes 128 queries of
// one sequence and one query head and walks the pages (64 keys) the queries can see:
//
//   S_j = Q · K_jᵀ        tcgen05.mma, M = 128 queries on TMEM lanes, N = 64 keys on TMEM columns
//   softmax               four warps, ONE QUERY ROW PER THREAD: tcgen05.ld of the row, mask, maximum, exp2,
//                         sum — no shuffles; P_j goes to shared memory as bf16 in the swizzled layout an MMA
//                         A-operand wants
//   O += P_j · V_j        tcgen05.mma again (V is the MN-major B operand, straight from the cache page),
//                         ACCUMULATING in TMEM over the pages
//
// The accumulator is scaled lazily: P_j and O are kept relative to a reference maximum that follows the
// row's running maximum only when that has grown by more than 8 (in base 2), so P stays below 256 and the
// read-multiply-write of O in TMEM happens a few times per row instead of once per page; the final division
// by the row sum makes the result the same.
//
// A causal prompt's query blocks differ 16-fold in the keys they see, and the kernel is as long as its longest
// block: with `split_pages` > 0 a block's key range is cut into parts of that many pages, each part a block of
// its own that leaves (reference maximum, sum, unnormalised output) per row in a workspace; the part that takes
// a (query block, head)'s last ticket adds the parts in key order and writes the output.
//
// A block is small on purpose (64 KB of shared memory, 128 TMEM columns, 192 threads): three are resident
// per SM and hide one another's chain S -> softmax -> PV.  Roles: warp 0 = TMA producer (Q once, then
// K_j / V_j pages into a ring of two), warp 1 = TMEM allocation and MMA issue, warps 2..5 = softmax and
// output.  S_{j+1} is computed while the softmax of S_j runs (the softmax frees S as soon as it has read
// it).  Every wait is bounded (see sm100.cuh).
#include <cuda.h>
#include <math.h>

#include "common.cuh"
#include "sm100.cuh"

namespace llmi {

constexpr int FT_BM = 128, FT_PAGE = 64, FT_HD = 64;
constexpr int FT_STAGES = 2;
constexpr int FT_THREADS = 192;
constexpr int FT_TILE = FT_PAGE * FT_HD * 2;          // 8 KB: one K or V page tile
constexpr int FT_QBYTES = FT_BM * FT_HD * 2;          // 16 KB
constexpr int FT_PBYTES = FT_BM * FT_PAGE * 2;        // 16 KB
constexpr int FT_SMEM = FT_QBYTES + FT_STAGES * 2 * FT_TILE + FT_PBYTES + 1024 + 128;
constexpr int FT_TMEM_COLS = 128;                     // S at columns 0..63, O at 64..127
constexpr float FT_LAZY = 8.0f;                       // the reference maximum follows the running one in steps of 2^8

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
  int n_tiles;              // blocks of 128 queries over all sequences
  int split_pages;          // 0: a query block's keys are one job; else jobs of at most this many pages
  float* partials;          // [job (gridDim.x)][head][66][128]: per row m_ref, l, O[64], when split
  int* tickets;             // [n_tiles * n_heads], zero before and after the launch
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
// 16 consecutive fp32 columns of this thread's TMEM lane, written; no wait
__device__ __forceinline__ void ft_st16(uint32_t taddr, const float* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
        "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15]))
      : "memory");
}
__device__ __forceinline__ void ft_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__global__ void __launch_bounds__(FT_THREADS, 3)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, PrefillTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem = base;
  const uint32_t kv_smem = base + FT_QBYTES;                        // stage s: K at +s*16K, V at +s*16K+8K
  const uint32_t p_smem = kv_smem + FT_STAGES * 2 * FT_TILE;
  const uint32_t bars = p_smem + FT_PBYTES;
  // barriers: q_full, kv_full[2], kv_empty[2], s_full, s_free, p_ready, o_done, tmem slot
  const uint32_t q_full = bars;
  auto kv_full = [&](int s) { return bars + 8u * (1 + s); };
  auto kv_empty = [&](int s) { return bars + 8u * (1 + FT_STAGES + s); };
  const uint32_t s_full = bars + 8u * (1 + 2 * FT_STAGES);
  const uint32_t s_free = s_full + 8u, p_ready = s_full + 16u, o_done = s_full + 24u;
  const uint32_t tmem_slot = s_full + 32u;

  pdl_launch_dependents();
  // which sequence, which block of 128 queries and which part of its keys: jobs are counted from the last
  // block of the last sequence backwards (late blocks, which see more keys, come first), a block's parts in key order
  int seq = p.n_seqs - 1, mb = 0, part = 0, n_parts = 1, tile_id = p.n_tiles;
  int q_start = 0, q_len = 0, kv_len = 0, pos0 = 0, m0 = 0, rows_here = 0, first_q = 0, last_q = 0, pg_first = 0, n_pg = 0;
  {
    int x = blockIdx.x;
    bool found = false;
    for (; seq >= 0 && !found; --seq) {
      q_start = p.seq_q_start[seq];
      q_len = p.seq_q_start[seq + 1] - q_start;
      kv_len = p.seq_kv_len[seq];
      pos0 = kv_len - q_len;
      for (mb = (q_len + FT_BM - 1) / FT_BM - 1; mb >= 0; --mb) {
        --tile_id;
        m0 = mb * FT_BM;
        rows_here = min(FT_BM, q_len - m0);
        first_q = pos0 + m0;
        last_q = first_q + rows_here - 1;
        const int lo_key = (p.window > 0 && first_q - p.window + 1 > 0) ? first_q - p.window + 1 : 0;
        pg_first = lo_key / FT_PAGE;
        n_pg = last_q / FT_PAGE - pg_first + 1;
        n_parts = p.split_pages > 0 ? (n_pg + p.split_pages - 1) / p.split_pages : 1;
        if (x < n_parts) {
          part = x;
          found = true;
          break;
        }
        x -= n_parts;
      }
      if (found) break;
    }
    if (!found) return;
  }
  if (n_parts > 1) {                       // this block's part of the key range
    pg_first += part * p.split_pages;
    n_pg = min(p.split_pages, n_pg - part * p.split_pages);
  }
  const int head = blockIdx.y;
  const int kvh = head / (p.n_heads / p.n_kv_heads);
  const int32_t* pages = p.seq_pages + (size_t)seq * p.pages_stride;
  __shared__ int s_last;

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
    mbar_init(s_full, 1);
    mbar_init(s_free, 4);
    mbar_init(p_ready, 4);
    mbar_init(o_done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(FT_TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  uint32_t tmem;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem) : "r"(tmem_slot));
  const uint32_t tmem_s = tmem, tmem_o = tmem + 64;

  if (warp == 0) {
    if (lane == 0) {
      // ---- producer ----
      pdl_wait();   // q and the cache pages of this step come from the kernels before
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
      // S: A = Q (K-major), B = K page (K-major), N = 64.  O: A = P (K-major), B = V page (MN-major), N = 64.
      const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(64 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      const uint32_t idesc_o = idesc_s | (1u << 16);
      auto issue_s = [&](int j) {
        const uint64_t a = ft_desc(q_smem), b = ft_desc(kv_smem + (j % FT_STAGES) * 2 * FT_TILE);
#pragma unroll
        for (int k4 = 0; k4 < FT_HD / 16; ++k4) ft_mma(tmem_s, a + 2 * k4, b + 2 * k4, idesc_s, k4 > 0);
        ft_commit(s_full);
      };
      bool ok = mbar_wait(q_full, 0, p.error_flag, 42) && mbar_wait(kv_full(0), 0, p.error_flag, 43);
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        issue_s(0);
      }
      for (int j = 0; j < n_pg && ok; ++j) {
        if (j + 1 < n_pg) {
          // S_{j+1} as soon as its page is here and the softmax has read S_j
          ok = mbar_wait(kv_full((j + 1) % FT_STAGES), ((j + 1) / FT_STAGES) & 1, p.error_flag, 44) &&
               mbar_wait(s_free, j & 1, p.error_flag, 45);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          issue_s(j + 1);
        }
        ok = mbar_wait(p_ready, j & 1, p.error_flag, 46);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t a = ft_desc(p_smem);
        const uint64_t b = ft_desc(kv_smem + (j % FT_STAGES) * 2 * FT_TILE + FT_TILE);
#pragma unroll
        for (int k4 = 0; k4 < FT_PAGE / 16; ++k4)   // 16 keys further: +32 bytes in a P row, +16 rows of 128 bytes in V
          ft_mma(tmem_o, a + 2 * k4, b + (uint64_t)(k4 * ((16 * 128) >> 4)), idesc_o, (j > 0 || k4 > 0) ? 1u : 0u);
        ft_commit(o_done);
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
    const uint32_t t_lane = (uint32_t)(quad * 32) << 16;
    float m_run = -INFINITY, m_ref = -INFINITY, l_run = 0.f;   // maxima in base 2, scaled
    bool ok = true;
    for (int j = 0; j < n_pg && ok; ++j) {
      ok = mbar_wait(s_full, j & 1, p.error_flag, 48);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float sc[FT_PAGE];
#pragma unroll
      for (int c = 0; c < FT_PAGE; c += 16) ft_ld16(tmem_s + t_lane + (uint32_t)c, sc + c);
      ft_ld_wait();
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(s_free);
      const int key0 = (pg_first + j) * FT_PAGE;
      const bool need_mask = (key0 + FT_PAGE - 1 > first_q) || (p.window > 0);
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < FT_PAGE; ++c) {
          const int key = key0 + c;
          if (key > qpos || (p.window > 0 && key < qpos - p.window + 1)) sc[c] = -INFINITY;
        }
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};      // four chains instead of one long one
#pragma unroll
      for (int c = 0; c < FT_PAGE; c += 8) {
#pragma unroll
        for (int u = 0; u < 4; ++u) mx4[u] = fmaxf(mx4[u], fmaxf(sc[c + 2 * u], sc[c + 2 * u + 1]));
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      m_run = fmaxf(m_run, mx * p.scale_log2);
      float corr = 1.f;
      if (m_run > m_ref + FT_LAZY || m_ref == -INFINITY) {     // (both -inf: nothing seen yet, nothing to scale)
        corr = (m_ref == -INFINITY) ? 0.f : fast_exp2(m_ref - m_run);
        m_ref = m_run;
        l_run *= corr;
      }
      const float neg_ref = (m_ref == -INFINITY) ? 0.f : -m_ref;
      // two keys per instruction where the hardware has it (fma.rn.f32x2, add.rn.f32x2)
      float2 sum2[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
      const float2 scale2 = make_float2(p.scale_log2, p.scale_log2), neg2 = make_float2(neg_ref, neg_ref);
      uint32_t packed[FT_PAGE / 2];
#pragma unroll
      for (int c = 0; c < FT_PAGE; c += 2) {
        const float2 x = __ffma2_rn(make_float2(sc[c], sc[c + 1]), scale2, neg2);
        const float2 e = make_float2(fast_exp2(x.x), fast_exp2(x.y));          // 2^(-inf) = 0 for masked keys
        sum2[(c >> 1) & 3] = __fadd2_rn(sum2[(c >> 1) & 3], e);
        __nv_bfloat162 h = __floats2bfloat162_rn(e.x, e.y);
        packed[c >> 1] = *reinterpret_cast<uint32_t*>(&h);
      }
      {
        const float2 a = __fadd2_rn(sum2[0], sum2[1]), b = __fadd2_rn(sum2[2], sum2[3]);
        const float2 t = __fadd2_rn(a, b);
        l_run += t.x + t.y;
      }
      if (j >= 1) {
        // O += P_{j-1} V_{j-1} has to be finished: P's buffer is written below, and O may be rescaled
        ok = mbar_wait(o_done, (j - 1) & 1, p.error_flag, 49);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (__any_sync(0xffffffffu, corr != 1.f)) {
#pragma unroll
          for (int c = 0; c < FT_HD; c += 16) {
            float t[16];
            ft_ld16(tmem_o + t_lane + (uint32_t)c, t);
            ft_ld_wait();
#pragma unroll
            for (int e = 0; e < 16; ++e) t[e] *= corr;
            ft_st16(tmem_o + t_lane + (uint32_t)c, t);
          }
          ft_st_wait();
        }
      }
      // P row -> shared memory, swizzled as an MMA operand (chunk c of row r at r*128 + ((c ^ (r & 7)) << 4))
      const uint32_t prow = p_smem + (uint32_t)row * 128;
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
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);
    }
    {
      // (a warp whose wait gave up still goes through the barriers below: nobody is left waiting for it)
      const bool fine = ok && mbar_wait(o_done, (n_pg - 1) & 1, p.error_flag, 50);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float o[FT_HD];
#pragma unroll
      for (int c = 0; c < FT_HD; c += 16) ft_ld16(tmem_o + t_lane + (uint32_t)c, o + c);
      ft_ld_wait();
      bool write_out = fine;
      if (n_parts > 1) {
        // this part's (m_ref, l, O) to the workspace; the part that comes last adds them all in key order
        const size_t slot_floats = (size_t)(FT_HD + 2) * FT_BM;
        float* mine = p.partials + ((size_t)blockIdx.x * p.n_heads + head) * slot_floats + row;
        mine[0] = m_ref;
        mine[FT_BM] = l_run;
#pragma unroll
        for (int c = 0; c < FT_HD; ++c) mine[(size_t)(2 + c) * FT_BM] = o[c];
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");          // the four softmax warps
        int* ticket = p.tickets + tile_id * p.n_heads + head;
        if (threadIdx.x == 64) s_last = (atomicAdd(ticket, 1) == n_parts - 1);
        asm volatile("bar.sync 1, 128;" ::: "memory");
        write_out = fine && s_last != 0;
        if (s_last != 0) {
          __threadfence();
          const float* first = p.partials + ((size_t)(blockIdx.x - part) * p.n_heads + head) * slot_floats + row;
          const size_t part_stride = (size_t)p.n_heads * slot_floats;
          float M = -INFINITY;
          for (int z = 0; z < n_parts; ++z) M = fmaxf(M, __ldcg(first + z * part_stride));
          float L = 0.f;
#pragma unroll
          for (int c = 0; c < FT_HD; ++c) o[c] = 0.f;
          for (int z = 0; z < n_parts; ++z) {
            const float* pz = first + z * part_stride;
            const float mz = __ldcg(pz);
            const float w = (mz == -INFINITY) ? 0.f : fast_exp2(mz - M);
            L = fmaf(__ldcg(pz + FT_BM), w, L);
#pragma unroll
            for (int c = 0; c < FT_HD; ++c) o[c] = fmaf(w, __ldcg(pz + (size_t)(2 + c) * FT_BM), o[c]);
          }
          l_run = L;
          if (threadIdx.x == 64) *ticket = 0;
        }
      }
      if (write_out && row_ok) {
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
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(FT_TMEM_COLS));
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
                                          int window, int n_jobs, int split_pages, float* partials, long partials_floats,
                                          int* tickets, int n_tickets, int* error_flag, cudaStream_t stream) {
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
  // n_jobs: blocks along x — n_blocks without a split, else the sum over the query blocks of their parts (the caller
  // counts them with the same rule as the kernel); the workspace holds one slot per job and head
  if (split_pages > 0) {
    if (n_jobs < n_blocks || !partials || !tickets || (long)n_jobs * n_heads * (FT_HD + 2) * FT_BM > partials_floats ||
        (long)n_blocks * n_heads > n_tickets)
      return LLMI_ERR_BAD_SIZE;
  } else {
    n_jobs = n_blocks;
  }
  PrefillTcParams p{(__nv_bfloat16*)out, ldo, seq_pages, seq_q_start, seq_kv_len, pages_stride, n_seqs, n_heads,
                    n_kv_heads, scale * 1.4426950408889634f, window, error_flag, n_blocks, split_pages, partials, tickets};
  dim3 grid(n_jobs, n_heads);
  attention_prefill_tc_kernel<<<grid, FT_THREADS, FT_SMEM, stream>>>(mq, mk, mv, p);
  return launch_status();
}
