// Prefill attention on the 5th-generation tensor cores (tcgen05), bf16, head size 64 or 128.
//
// Same operation as attention_prefill.cu (reference loop: src/model/transformer.cpp:263-282): causal
// grouped-query attention of the prompts of a step over their cache pages.  A block takes 128 queries of
// one sequence and one query head and walks the pages (64 keys) the queries can see:
//
//   S_j = Q · K_jᵀ        tcgen05.mma, M = 128 queries on TMEM lanes, N = 64 keys on TMEM columns
//   softmax               a thread owns a query row's share of the page (all 64 keys at head size 128; 32 keys
//                         at head size 64, where two threads share a row, each with its own running maximum,
//                         sum and O that meet only at the end): tcgen05.ld, mask, maximum, exp2, sum — no
//                         shuffles; P_j goes back to TENSOR MEMORY as bf16 pairs, over the first half of the
//                         S columns the thread has just read (tcgen05.st)
//   O += P_j · V_j        tcgen05.mma with the A operand in TMEM (V is the MN-major B operand, straight from
//                         the cache page), ACCUMULATING in TMEM over the pages
//
// S_j lies in buffer j & 1, so S_{j+1} is computed while the softmax of S_j runs, and the softmax warps wait
// for nothing else: MMAs of one thread run in issue order, which is what lets S_{j+1} overwrite the buffer of
// P_{j-1} right after O += P_{j-1} V_{j-1} was issued.  No P tile in shared memory, no async-proxy fence, no
// hand-back of S.
//
// The accumulator is scaled lazily: P_j and O are kept relative to a reference maximum that follows the
// row's running maximum only when that has grown by more than 8 (in base 2), so P stays below 256 and the
// read-multiply-write of O in TMEM happens a few times per row instead of once per page (only then is
// O += P_{j-1} V_{j-1} waited for); the final division by the row sum makes the result the same.
//
// A causal prompt's query blocks differ 16-fold in the keys they see, and the kernel is as long as its longest
// block: with `split_pages` > 0 a block's key range is cut into parts of that many pages, each part a block of
// its own that leaves (reference maximum, sum, unnormalised output) per row in a workspace; the part that takes
// a (query block, head)'s last ticket adds the parts in key order and writes the output.
//
// A block has 64 KB (head size 128: 96 KB) of shared memory (Q, three (two) K/V stages) and 256 TMEM columns
// (S0, S1, O): two are resident per SM.  Roles: warp 0 = TMA producer (Q once, then K_j / V_j pages into the
// ring), warp 1 = TMEM allocation and MMA issue, warps 2.. = softmax and output (eight at head size 64, four at
// 128).  tcgen05.ld and .st are warp-wide instructions: no lane may skip them (rows past a sequence's end are
// computed and not stored).  Every wait is bounded (see sm100.cuh).
#include <cuda.h>
#include <math.h>

#include "common.cuh"
#include "sm100.cuh"

namespace llmi {

constexpr int FT_BM = 128, FT_PAGE = 64;
constexpr int FT_SUB = FT_PAGE * 64 * 2;              // 8 KB: 64 rows x 64 columns of bf16, one swizzled sub-tile
constexpr int FT_TMEM_COLS = 256;                     // S_j (then P_j) at columns 64 * (j & 1); O of key half h at 128 + HD * h
constexpr float FT_LAZY = 8.0f;                       // the reference maximum follows the running one in steps of 2^8

// Head size 64: two softmax threads per query row (HALVES = 2), each with 32 keys of a page and an O of 64 columns.
// Head size 128: one thread per row with all 64 keys and an O of 128 columns.  Either way S0, S1 and O fill 256
// TMEM columns and two blocks are resident per SM.
template <int HD>
struct FtCfg {
  static constexpr int NSUB = HD / 64;                        // 64-column sub-tiles of a Q, K or V tile
  static constexpr int HALVES = 128 / HD;
  static constexpr int KEYS = FT_PAGE / HALVES;               // keys of a page per softmax thread
  static constexpr int THREADS = 64 + 128 * HALVES;           // producer warp, MMA warp, 4 * HALVES softmax warps
  static constexpr int STAGES = HD == 64 ? 3 : 2;
  static constexpr int TILE = NSUB * FT_SUB;                  // one K or V page
  static constexpr int QBYTES = 2 * NSUB * FT_SUB;            // 128 query rows
  static constexpr int SMEM = QBYTES + STAGES * 2 * TILE + 1024 + 128;
};

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
  float* partials;          // [job (gridDim.y)][head][HD + 2][128]: per row m_ref, l, O[HD], when split
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


__device__ __forceinline__ void ft_mma_ts(uint32_t d, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d), "r"(a_tmem), "l"(b), "r"(idesc), "r"(acc)
      : "memory");
}
// 16 consecutive 32-bit columns of this thread's TMEM lane, written; no wait
__device__ __forceinline__ void ft_st16u(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
        "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}

template <int HD>
__global__ void __launch_bounds__(FtCfg<HD>::THREADS, 2)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, PrefillTcParams p) {
  using C = FtCfg<HD>;
  constexpr int STAGES = C::STAGES, NSUB = C::NSUB, HALVES = C::HALVES, KEYS = C::KEYS;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem = base;                                      // sub-tile u (dims 64u..): + u * 16 KB
  const uint32_t kv_smem = base + C::QBYTES;                         // stage s: K at + s * 2 * TILE, V a TILE further
  const uint32_t bars = kv_smem + STAGES * 2 * C::TILE;
  // barriers: q_full, kv_full[stages], kv_empty[stages], s_full[2], p_ready[2], o_done, tmem slot
  const uint32_t q_full = bars;
  auto kv_full = [&](int s) { return bars + 8u * (1 + s); };
  auto kv_empty = [&](int s) { return bars + 8u * (1 + STAGES + s); };
  auto s_full = [&](int b) { return bars + 8u * (1 + 2 * STAGES + b); };
  auto p_ready = [&](int b) { return bars + 8u * (3 + 2 * STAGES + b); };
  const uint32_t o_done = bars + 8u * (5 + 2 * STAGES);
  const uint32_t tmem_slot = o_done + 8u;

  pdl_launch_dependents();
  // The head is the FAST grid index and the job the slow one: blocks start in the order of their linear index, and a
  // long job that starts late is the kernel's tail (with the head as the slow index the longest job of the last head
  // started when the kernel was half over: 51 us for 2,048 tokens x 32 heads against 33 us this way).
  // Which sequence, which block of 128 queries and which part of its keys: jobs are counted from the last
  // block of the last sequence backwards (late blocks, which see more keys, come first), a block's parts in key order
  const int job = blockIdx.y;
  int seq = p.n_seqs - 1, mb = 0, part = 0, n_parts = 1, tile_id = p.n_tiles;
  int q_start = 0, q_len = 0, kv_len = 0, pos0 = 0, m0 = 0, rows_here = 0, first_q = 0, last_q = 0, pg_first = 0, n_pg = 0;
  {
    int x = job;
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
  const int head = blockIdx.x;
  const int kvh = head / (p.n_heads / p.n_kv_heads);
  const int32_t* pages = p.seq_pages + (size_t)seq * p.pages_stride;
  __shared__ int s_last;
  __shared__ float s_ml[2][FT_BM][2];      // (reference maximum, sum) of a row's two key halves

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
    mbar_init(q_full, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(kv_full(s), 1);
      mbar_init(kv_empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(s_full(b), 1);
      mbar_init(p_ready(b), 4 * HALVES);
    }
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
  const uint32_t tmem_s = tmem, tmem_o = tmem + 128;

  if (warp == 0) {
    if (lane == 0) {
      // ---- producer ----
      pdl_wait();   // q and the cache pages of this step come from the kernels before
      mbar_expect_tx(q_full, C::QBYTES);
#pragma unroll
      for (int u = 0; u < NSUB; ++u) ft_tma(q_smem + u * 2 * FT_SUB, &map_q, head * HD + 64 * u, q_start + m0, q_full);
      for (int j = 0; j < n_pg; ++j) {
        const int s = j % STAGES;
        if (j >= STAGES && !mbar_wait(kv_empty(s), ((j / STAGES) - 1) & 1, p.error_flag, 41)) break;
        const int row = (pages[pg_first + j] * p.n_kv_heads + kvh) * FT_PAGE;
        mbar_expect_tx(kv_full(s), 2 * C::TILE);
#pragma unroll
        for (int u = 0; u < NSUB; ++u) {
          ft_tma(kv_smem + s * 2 * C::TILE + u * FT_SUB, &map_k, 64 * u, row, kv_full(s));
          ft_tma(kv_smem + s * 2 * C::TILE + C::TILE + u * FT_SUB, &map_v, 64 * u, row, kv_full(s));
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer ----
      // S: A = Q (shared, K-major), B = K page (K-major), N = 64 keys, k over the head's dims (sub-tiles of 64).
      // O: A = P (TMEM: 128 lanes x 32 columns of bf16 pairs, over the first half of the S buffer it came from),
      // B = V page (MN-major), N = 64 dims per MMA (one per 64-column sub-tile of V).  MMAs of one thread run in
      // issue order: S_{j+1} may be issued into the buffer that P_{j-1} lies in right after O += P_{j-1} V_{j-1}.
      const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(64 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      const uint32_t idesc_o = idesc_s | (1u << 16);
      auto issue_s = [&](int j) {
        const uint32_t d = tmem_s + (uint32_t)(64 * (j & 1));
#pragma unroll
        for (int k4 = 0; k4 < HD / 16; ++k4) {
          const uint64_t a = ft_desc(q_smem + (k4 / 4) * 2 * FT_SUB), b = ft_desc(kv_smem + (j % STAGES) * 2 * C::TILE + (k4 / 4) * FT_SUB);
          ft_mma(d, a + 2 * (k4 % 4), b + 2 * (k4 % 4), idesc_s, k4 > 0);
        }
        ft_commit(s_full(j & 1));
      };
      bool ok = mbar_wait(q_full, 0, p.error_flag, 42) && mbar_wait(kv_full(0), 0, p.error_flag, 43);
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        issue_s(0);
      }
      for (int j = 0; j < n_pg && ok; ++j) {
        if (j + 1 < n_pg) {
          // S_{j+1} as soon as its page is here: the softmax of S_j runs meanwhile
          ok = mbar_wait(kv_full((j + 1) % STAGES), ((j + 1) / STAGES) & 1, p.error_flag, 44);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          issue_s(j + 1);
        }
        ok = mbar_wait(p_ready(j & 1), (j >> 1) & 1, p.error_flag, 46);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a = tmem_s + (uint32_t)(64 * (j & 1));
        const uint32_t v_tile = kv_smem + (j % STAGES) * 2 * C::TILE + C::TILE;
        // the keys of half h accumulate into their own O (their softmax threads keep their own reference maximum):
        // P of half h lies at columns 32h.. of the S buffer; 16 keys further: 8 columns of P, 16 rows of 128 bytes of V
#pragma unroll
        for (int h = 0; h < HALVES; ++h)
#pragma unroll
          for (int k4 = 0; k4 < KEYS / 16; ++k4)
#pragma unroll
            for (int u = 0; u < NSUB; ++u)
              ft_mma_ts(tmem_o + (uint32_t)(HD * h + 64 * u), a + (uint32_t)(32 * h + 8 * k4),
                        ft_desc(v_tile + u * FT_SUB) + (uint64_t)(((KEYS / 16) * h + k4) * ((16 * 128) >> 4)), idesc_o,
                        (j > 0 || k4 > 0) ? 1u : 0u);
        ft_commit(o_done);
        ft_commit(kv_empty(j % STAGES));
      }
    }
  } else {
    // ---- softmax and output: HALVES threads per query row, each with its share of a page's keys ----
    // The halves are independent streams (own running maximum, reference maximum, sum and O) that meet only at the
    // end: no exchange inside the page loop.
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;                 // keys KEYS*half .. of every page
    const int row = quad * 32 + lane;                 // row of the 128-query block = TMEM lane
    const int qrow = m0 + row;
    const bool row_ok = qrow < q_len;
    const int qpos = pos0 + qrow;
    const uint32_t t_lane = (uint32_t)(quad * 32) << 16;
    const uint32_t t_o = tmem_o + t_lane + (uint32_t)(HD * half);
    float m_run = -INFINITY, m_ref = -INFINITY, l_run = 0.f;   // maxima in base 2, scaled
    bool ok = true;
    for (int j = 0; j < n_pg && ok; ++j) {
      ok = mbar_wait(s_full(j & 1), (j >> 1) & 1, p.error_flag, 48);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t t_s = tmem_s + t_lane + (uint32_t)(64 * (j & 1) + KEYS * half);
      float sc[KEYS];
#pragma unroll
      for (int c = 0; c < KEYS; c += 16) ft_ld16(t_s + (uint32_t)c, sc + c);
      ft_ld_wait();
      const int page_key0 = (pg_first + j) * FT_PAGE;
      const int key0 = page_key0 + KEYS * half;
      const bool need_mask = (key0 + KEYS - 1 > first_q) || (p.window > 0);
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < KEYS; ++c) {
          const int key = key0 + c;
          if (key > qpos || (p.window > 0 && key < qpos - p.window + 1)) sc[c] = -INFINITY;
        }
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};      // four chains instead of one long one
#pragma unroll
      for (int c = 0; c < KEYS; c += 8) {
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
      uint32_t packed[KEYS / 2];
#pragma unroll
      for (int c = 0; c < KEYS; c += 2) {
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
        // O += P_{j-1} V_{j-1} (it may still run beside this softmax) is waited for on EVERY page, needed or not: a
        // wait on a phase's parity is right only for a thread that is at most one phase behind, and o_done completes a
        // phase per page.  (With the wait only where O is rescaled, a thread could reach the wait behind the loop two
        // phases behind, where it passes at once: when the MMAs lagged — head size 128, blocks that start beside busy
        // ones — the first query block, two pages, now and then read its O before the products had finished.)
        ok = mbar_wait(o_done, (j - 1) & 1, p.error_flag, 49);
        if (!ok) break;
        if (__any_sync(0xffffffffu, corr != 1.f)) {
          // this half's O is rescaled in place
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
          for (int c = 0; c < HD; c += 16) {
            float t[16];
            ft_ld16(t_o + (uint32_t)c, t);
            ft_ld_wait();
#pragma unroll
            for (int e = 0; e < 16; ++e) t[e] *= corr;
            ft_st16(t_o + (uint32_t)c, t);
          }
        }
      }
      // P -> TMEM, over the first half of the S columns this thread has just read: bf16 pairs, 16 columns at a time
#pragma unroll
      for (int c = 0; c < KEYS / 2; c += 16) ft_st16u(t_s + (uint32_t)c, packed + c);
      ft_st_wait();
      if (page_key0 + FT_PAGE > kv_len) {
        // The sequence ends inside this page: value rows behind its end are cleared so that their zero
        // probabilities cannot meet a NaN.  (The page is in shared memory: S_j was computed from it.)
        const uint32_t v_tile = kv_smem + (j % STAGES) * 2 * C::TILE + C::TILE;
        const int first_bad = kv_len - page_key0;
        for (int idx = (warp - 2) * 32 + lane; idx < (FT_PAGE - first_bad) * 8 * NSUB; idx += 128 * HALVES) {
          const int r = first_bad + (idx >> 3) / NSUB, u = (idx >> 3) % NSUB, ch = idx & 7;
          asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(v_tile + (uint32_t)(u * FT_SUB + r * 128 + (ch << 4))), "r"(0u) : "memory");
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> visible to the MMA's reads
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready(j & 1));
    }
    {
      // (a warp whose wait gave up still goes through the barriers below: nobody is left waiting for it)
      // (`fine` is the same in all lanes of a warp: the TMEM loads below are warp-wide instructions)
      const bool fine = __all_sync(0xffffffffu, ok && mbar_wait(o_done, (n_pg - 1) & 1, p.error_flag, 50));
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // A row's halves meet: (reference maximum, sum) through shared memory, the O's straight from TMEM; each of the
      // row's threads finishes DH of the output dims, 32 at a time.
      constexpr int DH = HD / HALVES;
      float M = m_ref, L = l_run, w_a = 1.f, w_b = 0.f;
      if (HALVES == 2) {
        s_ml[half][row][0] = m_ref;
        s_ml[half][row][1] = l_run;
        asm volatile("bar.sync 1, %0;" ::"n"(128 * HALVES) : "memory");          // the softmax warps
        const float m_a = s_ml[0][row][0], m_b = s_ml[1][row][0];
        M = fmaxf(m_a, m_b);
        w_a = (m_a == -INFINITY) ? 0.f : fast_exp2(m_a - M);
        w_b = (m_b == -INFINITY) ? 0.f : fast_exp2(m_b - M);
        L = s_ml[0][row][1] * w_a + s_ml[1][row][1] * w_b;
      }
      const uint32_t t_mine = tmem_o + t_lane + (uint32_t)(DH * half);          // this thread's dims in the first O
      const size_t slot_floats = (size_t)(HD + 2) * FT_BM;
      const size_t part_stride = (size_t)p.n_heads * slot_floats;
      bool write_out = fine, merge = false;
      if (n_parts > 1) {
        // this part's (maximum, sum, O) to the workspace; the part that comes last adds them all in key order
        float* mine = p.partials + ((size_t)job * p.n_heads + head) * slot_floats + row;
        if (half == 0) {
          mine[0] = M;
          mine[FT_BM] = L;
        }
#pragma unroll 1
        for (int c0 = 0; c0 < DH; c0 += 32) {
          float oa[32], ob[32];
          ft_ld16(t_mine + (uint32_t)c0, oa);
          ft_ld16(t_mine + (uint32_t)(c0 + 16), oa + 16);
          if (HALVES == 2) {
            ft_ld16(t_mine + (uint32_t)(HD + c0), ob);
            ft_ld16(t_mine + (uint32_t)(HD + c0 + 16), ob + 16);
          }
          ft_ld_wait();
#pragma unroll
          for (int c = 0; c < 32; ++c)
            mine[(size_t)(2 + DH * half + c0 + c) * FT_BM] = HALVES == 2 ? w_a * oa[c] + w_b * ob[c] : oa[c];
        }
        __threadfence();
        asm volatile("bar.sync 1, %0;" ::"n"(128 * HALVES) : "memory");
        int* ticket = p.tickets + tile_id * p.n_heads + head;
        if (threadIdx.x == 64) s_last = (atomicAdd(ticket, 1) == n_parts - 1);
        asm volatile("bar.sync 1, %0;" ::"n"(128 * HALVES) : "memory");
        merge = s_last != 0;
        write_out = fine && merge;
        if (merge) {
          __threadfence();
          const float* first = p.partials + ((size_t)(job - part) * p.n_heads + head) * slot_floats + row;
          M = -INFINITY;
          for (int z = 0; z < n_parts; ++z) M = fmaxf(M, __ldcg(first + z * part_stride));
          L = 0.f;
          for (int z = 0; z < n_parts; ++z) {
            const float mz = __ldcg(first + z * part_stride);
            L = fmaf(__ldcg(first + z * part_stride + FT_BM), (mz == -INFINITY) ? 0.f : fast_exp2(mz - M), L);
          }
          if (threadIdx.x == 64) *ticket = 0;
        }
      }
      if (write_out) {      // every lane takes part in the TMEM loads; only the rows that exist are stored
        const float inv = 1.f / L;
        __nv_bfloat16* dst = p.out + (size_t)(q_start + qrow) * p.ldo + (size_t)head * HD + DH * half;
#pragma unroll 1
        for (int c0 = 0; c0 < DH; c0 += 32) {
          float o[32];
          if (merge) {
            const float* first = p.partials + ((size_t)(job - part) * p.n_heads + head) * slot_floats + row;
#pragma unroll
            for (int c = 0; c < 32; ++c) o[c] = 0.f;
            for (int z = 0; z < n_parts; ++z) {
              const float* pz = first + z * part_stride;
              const float mz = __ldcg(pz);
              const float w = (mz == -INFINITY) ? 0.f : fast_exp2(mz - M);
#pragma unroll
              for (int c = 0; c < 32; ++c) o[c] = fmaf(w, __ldcg(pz + (size_t)(2 + DH * half + c0 + c) * FT_BM), o[c]);
            }
          } else {
            float ob[32];
            ft_ld16(t_mine + (uint32_t)c0, o);
            ft_ld16(t_mine + (uint32_t)(c0 + 16), o + 16);
            if (HALVES == 2) {
              ft_ld16(t_mine + (uint32_t)(HD + c0), ob);
              ft_ld16(t_mine + (uint32_t)(HD + c0 + 16), ob + 16);
            }
            ft_ld_wait();
            if (HALVES == 2) {
#pragma unroll
              for (int c = 0; c < 32; ++c) o[c] = w_a * o[c] + w_b * ob[c];
            }
          }
#pragma unroll
          for (int c = 0; c < 32 && row_ok; c += 8) {
            uint4 v;
            __nv_bfloat162 h0 = __floats2bfloat162_rn(o[c] * inv, o[c + 1] * inv), h1 = __floats2bfloat162_rn(o[c + 2] * inv, o[c + 3] * inv);
            __nv_bfloat162 h2 = __floats2bfloat162_rn(o[c + 4] * inv, o[c + 5] * inv), h3 = __floats2bfloat162_rn(o[c + 6] * inv, o[c + 7] * inv);
            v.x = *reinterpret_cast<uint32_t*>(&h0);
            v.y = *reinterpret_cast<uint32_t*>(&h1);
            v.z = *reinterpret_cast<uint32_t*>(&h2);
            v.w = *reinterpret_cast<uint32_t*>(&h3);
            *reinterpret_cast<uint4*>(dst + c0 + c) = v;
          }
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

LLMI_EXPORT int llmi_attention_prefill_tc_supported(int head_dim) { return head_dim == 64 || head_dim == 128; }

namespace llmi {
template <int HD>
static int ft_launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const PrefillTcParams& p, dim3 grid,
                     cudaStream_t stream) {
  using C = FtCfg<HD>;
  static PerDevice<bool> configured_on;
  bool& configured = configured_on.here();
  if (!configured) {
    if (cudaFuncSetAttribute(attention_prefill_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM) != cudaSuccess)
      return LLMI_ERR_LAUNCH;
    configured = true;
  }
  // a programmatic dependent: its blocks set themselves up (barriers, tensor memory, descriptors) while the kernel
  // before drains; the producer waits before its first copy, and nothing else reads or writes global memory earlier
  return launch_pdl(PDL_ATTENTION, attention_prefill_tc_kernel<HD>, grid, dim3(C::THREADS), C::SMEM, stream, mq, mk, mv, p);
}
}  // namespace llmi

// q: [n_tokens, >= n_heads*head_dim] rotated queries (row pitch ldq, 16-byte aligned rows); otherwise as llmi_attention_prefill.
// With split_pages > 0: partials holds n_jobs * n_heads * (head_dim + 2) * 128 floats.
LLMI_EXPORT int llmi_attention_prefill_tc(const void* q, long ldq, long n_tokens, void* out, long ldo, const void* k_cache,
                                          const void* v_cache, long n_cache_pages, const int32_t* seq_pages,
                                          int pages_stride, const int32_t* seq_q_start, const int32_t* seq_kv_len,
                                          int n_seqs, int n_blocks, int n_heads, int n_kv_heads, int head_dim, float scale,
                                          int window, int n_jobs, int split_pages, float* partials, long partials_floats,
                                          int* tickets, int n_tickets, int* error_flag, cudaStream_t stream) {
  if (n_seqs <= 0 || n_blocks <= 0 || n_heads <= 0 || n_kv_heads <= 0 || n_cache_pages <= 0 || n_tokens <= 0) return LLMI_ERR_BAD_SIZE;
  if (n_heads % n_kv_heads) return LLMI_ERR_BAD_SIZE;
  if (!llmi_attention_prefill_tc_supported(head_dim)) return LLMI_ERR_UNSUPPORTED;
  if (((uintptr_t)q & 15) || (ldq & 7) || ((uintptr_t)out & 15) || (ldo & 7) || ((uintptr_t)k_cache & 15) ||
      ((uintptr_t)v_cache & 15))
    return LLMI_ERR_ALIGN;
  const long rows = n_cache_pages * n_kv_heads * FT_PAGE;
  if (rows > 0x7fffffffL) return LLMI_ERR_BAD_SIZE;
  CUtensorMap mq, mk, mv;
  int rc = ft_make_map(&mq, q, n_tokens, (long)n_heads * head_dim, ldq, FT_BM);
  if (rc != LLMI_OK) return rc;
  rc = ft_make_map(&mk, k_cache, rows, head_dim, head_dim, FT_PAGE);
  if (rc != LLMI_OK) return rc;
  rc = ft_make_map(&mv, v_cache, rows, head_dim, head_dim, FT_PAGE);
  if (rc != LLMI_OK) return rc;
  // n_jobs: blocks along y — n_blocks without a split, else the sum over the query blocks of their parts (the caller
  // counts them with the same rule as the kernel); the workspace holds one slot per job and head
  if (split_pages > 0) {
    if (n_jobs < n_blocks || !partials || !tickets || (long)n_jobs * n_heads * (head_dim + 2) * FT_BM > partials_floats ||
        (long)n_blocks * n_heads > n_tickets)
      return LLMI_ERR_BAD_SIZE;
  } else {
    n_jobs = n_blocks;
  }
  PrefillTcParams p{(__nv_bfloat16*)out, ldo, seq_pages, seq_q_start, seq_kv_len, pages_stride, n_seqs, n_heads,
                    n_kv_heads, scale * 1.4426950408889634f, window, error_flag, n_blocks, split_pages, partials, tickets};
  if (n_jobs > 65535) return LLMI_ERR_BAD_SIZE;
  dim3 grid(n_heads, n_jobs);
  return head_dim == 64 ? ft_launch<64>(mq, mk, mv, p, grid, stream) : ft_launch<128>(mq, mk, mv, p, grid, stream);
}
