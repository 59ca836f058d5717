// y = x · Wᵀ on the 5th-generation tensor cores (tcgen05), bf16 inputs, fp32 accumulation in TMEM.
//
// The reference's matmul is a loop of dot products over weight rows (src/model/kernels.cpp:97-113),
// W stored [out, in] (include/llmi/model/kernels.hpp:15-17).  Here the same product is tiled for
// sm_100a: the WEIGHT tile is the 128-row operand of the MMA (out features on TMEM lanes) and the
// ACTIVATION tile is the N operand (16..256 tokens on TMEM columns), so that one kernel serves a
// 2,048-token prefill and a 1-token decode step alike: for few tokens the weights still stream
// through full 128-row MMAs and the step is bound by HBM, not by the token count.
//
//   warp 0      : TMA producer — cp.async.bulk.tensor tiles of W [128 x 64] and x [BN x 64] into a
//                 ring of shared-memory stages (128-byte swizzle), completion on mbarriers
//   warp 1      : allocates TMEM; one thread issues tcgen05.mma (4 per stage, K = 16 each) and
//                 tcgen05.commit to hand stages back and to signal the finished accumulator
//   warps 2..5  : epilogue — tcgen05.ld the accumulator (one TMEM lane quadrant per warp), add bias,
//                 and store / add into the output, which is token-major [tokens, out]
//
// Split-K: when a product has too few output tiles to fill the GPU (decode: o_proj, down_proj), the
// k range is cut over gridDim.z.  Each CTA writes its fp32 partial tile to a workspace and takes a
// ticket; the CTA that takes the last ticket of a tile adds the partials in split order and runs
// the epilogue.  Nothing waits for another CTA, and the order of additions is fixed.
//
// Every wait on an mbarrier is bounded: after about a second it records an error code in
// *error_flag and the CTA unwinds (frees TMEM, exits) instead of hanging.
#include <cuda.h>

#include "common.cuh"
#include "sm100.cuh"
#include "tc_common.cuh"

namespace llmi {

#ifndef LLMI_TC_SMALL_STAGES
#define LLMI_TC_SMALL_STAGES 4
#endif
#ifndef LLMI_TC_SMALL_CTAS
#define LLMI_TC_SMALL_CTAS 3
#endif

template <int BN>
struct TcConfig {
  static constexpr int A_BYTES = TC_BM * TC_BK * 2;
  static constexpr int B_BYTES = BN * TC_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // few-token tiles stream weights: 4 stages per CTA and 2-3 CTAs per SM keep more bytes in flight and
  // hide each CTA's start-up behind its neighbours; large tiles are compute-bound and take the whole SM
  static constexpr int STAGES = BN <= 32 ? LLMI_TC_SMALL_STAGES : (BN == 64 ? 4 : (BN == 128 ? 6 : 4));
  static constexpr int CTAS_PER_SM = BN <= 32 ? LLMI_TC_SMALL_CTAS : (BN == 64 ? 2 : 1);
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 8 * (2 * STAGES + 4) + 16 /*barriers, TMEM slot*/;
  static constexpr int ACC_COLS = BN;                       // one accumulator: 128 lanes x BN columns of fp32
  static constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;   // two of them, so that epilogue and MMAs overlap
};

// Work is cut into units (m tile, n tile, k split); `n_units` of them, m fastest.  The grid is
// persistent: block b takes units b, b + gridDim.x, ...  The ring of stages runs on across units,
// and the accumulator is double-buffered in TMEM, so the epilogue of one unit (TMEM -> registers ->
// global) overlaps the loads and MMAs of the next.
template <int BN>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, TcParams p,
               int m_tiles, int n_tiles) {
  using C = TcConfig<BN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = base + C::STAGES * C::STAGE_BYTES;   // full[S], empty[S], acc_full[2], acc_empty[2], tmem slot
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (C::STAGES + s); };
  auto acc_full = [&](int b) { return bars + 8u * (2 * C::STAGES + b); };
  auto acc_empty = [&](int b) { return bars + 8u * (2 * C::STAGES + 2 + b); };
  const uint32_t tmem_slot = bars + 8u * (2 * C::STAGES + 4);
  __shared__ int s_last;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kblocks = (p.k + TC_BK - 1) / TC_BK;
  const int per = (kblocks + p.splits - 1) / p.splits;
  const int n_out_tiles = m_tiles * n_tiles;
  const int n_units = n_out_tiles * p.splits;
  // A block with a single unit needs one accumulator; with several it takes two and alternates.
  const int acc_bufs = n_units > (int)gridDim.x ? 2 : 1;
  const uint32_t tmem_cols = (uint32_t)(acc_bufs * BN < 32 ? 32 : acc_bufs * BN);

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full(b), 1);
      mbar_init(acc_empty(b), 4);   // the four epilogue warps
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(tmem_cols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  uint32_t tmem_d;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_d) : "r"(tmem_slot));

  // unit -> (m tile, n tile, first k block, number of k blocks)
  auto unit_of = [&](int u, int& mt, int& nt, int& z, int& kb0, int& nkb) {
    const int tile = u % n_out_tiles;
    z = u / n_out_tiles;
    mt = tile % m_tiles;
    nt = tile / m_tiles;
    kb0 = z * per;
    nkb = max(0, min(kblocks, kb0 + per) - kb0);
  };

  pdl_launch_dependents();
  if (warp == 0) {
    if (lane == 0) {
      // ---- TMA producer ----
      // The weights do not depend on the kernel before this one: the weight tiles of the first stages are
      // requested at once.  The activations do: their tiles follow after pdl_wait().
      int total = 0;
      for (int u = blockIdx.x; u < n_units; u += gridDim.x) {
        int mt, nt, z, kb0, nkb;
        unit_of(u, mt, nt, z, kb0, nkb);
        total += nkb;
      }
      const int ahead = total < C::STAGES ? total : C::STAGES;   // k blocks requested before the wait
      int xk[C::STAGES], xn[C::STAGES];
      int it = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
        int mt, nt, z, kb0, nkb;
        unit_of(u, mt, nt, z, kb0, nkb);
        for (int i = 0; i < nkb; ++i, ++it) {
          const int s = it % C::STAGES;
          if (it >= C::STAGES && !mbar_wait(empty_bar(s), ((it / C::STAGES) - 1) & 1, p.error_flag, 1)) { ok = false; break; }
          mbar_expect_tx(full_bar(s), C::STAGE_BYTES);
          const uint32_t a_dst = base + s * C::STAGE_BYTES;
          tma_load_2d(a_dst, &map_w, (kb0 + i) * TC_BK, mt * TC_BM, full_bar(s));
          if (it < ahead) {
            xk[s] = (kb0 + i) * TC_BK;
            xn[s] = nt * BN;
            if (it == ahead - 1) {
              pdl_wait();
              for (int j = 0; j < ahead; ++j)
                tma_load_2d(base + j * C::STAGE_BYTES + C::A_BYTES, &map_x, xk[j], xn[j], full_bar(j));
            }
          } else {
            tma_load_2d(a_dst + C::A_BYTES, &map_x, (kb0 + i) * TC_BK, nt * BN, full_bar(s));
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer ----
      // instruction descriptor: D fp32, A and B bf16, both K-major, N = BN, M = 128
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
      int it = 0, j = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x, ++j) {
        int mt, nt, z, kb0, nkb;
        unit_of(u, mt, nt, z, kb0, nkb);
        const int b = j & (acc_bufs - 1);
        if (j >= acc_bufs && !mbar_wait(acc_empty(b), ((j / acc_bufs) - 1) & 1, p.error_flag, 4)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d_addr = tmem_d + (uint32_t)(b * C::ACC_COLS);
        for (int i = 0; i < nkb; ++i, ++it) {
          const int s = it % C::STAGES;
          ok = mbar_wait(full_bar(s), (it / C::STAGES) & 1, p.error_flag, 2);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = base + s * C::STAGE_BYTES;
          const uint64_t a_desc = umma_desc(a_addr), b_desc = umma_desc(a_addr + C::A_BYTES);
#pragma unroll
          for (int k4 = 0; k4 < TC_BK / 16; ++k4) {
            // 16 bf16 = 32 bytes further along K inside the swizzled row: +2 in 16-byte units
            umma_bf16(d_addr, a_desc + 2 * k4, b_desc + 2 * k4, idesc, (i > 0 || k4 > 0) ? 1u : 0u);
          }
          umma_commit(empty_bar(s));
        }
        if (ok) umma_commit(acc_full(b));
      }
    }
  } else {
    // ---- epilogue warps: TMEM lane quadrant = warp % 4 ----
    const int quad = warp & 3;
    pdl_wait();   // the output (read-modify-write), the workspace and the tickets belong to earlier kernels until now
    int j = 0;
    for (int u = blockIdx.x; u < n_units; u += gridDim.x, ++j) {
      int mt, nt, z, kb0, nkb;
      unit_of(u, mt, nt, z, kb0, nkb);
      const int b = j & (acc_bufs - 1);
      const uint32_t acc_parity = (uint32_t)(j / acc_bufs) & 1u;
      const int m = mt * TC_BM + quad * 32 + lane;
      const int n0 = nt * BN;
      const uint32_t t_base = tmem_d + ((uint32_t)(quad * 32) << 16) + (uint32_t)(b * C::ACC_COLS);
      const int tile = nt * m_tiles + mt;
      if (p.splits == 1 && p.mode == OUT_ADD_F32) {
        // Residual add: the old values are fetched one 16-token chunk ahead of the accumulator reads, so
        // that their round trip to L2 overlaps the chunk before (and, for the first chunk, the MMAs).
        const int nch = (min(BN, p.n_tok - n0) + 15) / 16;
        const bool row_ok = m < p.m_out;
        const float bias = (p.bias && row_ok) ? p.bias[m] : 0.f;
        float* o = (float*)p.out + (size_t)n0 * p.ldo + m;
        float nxt[16];
#pragma unroll
        for (int c = 0; c < 16; ++c) nxt[c] = (row_ok && n0 + c < p.n_tok) ? o[(size_t)c * p.ldo] : 0.f;
        if (!mbar_wait(acc_full(b), acc_parity, p.error_flag, 3)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        for (int ci = 0; ci < nch; ++ci) {
          float cur[16], v[16];
#pragma unroll
          for (int c = 0; c < 16; ++c) cur[c] = nxt[c];
          if (ci + 1 < nch) {
#pragma unroll
            for (int c = 0; c < 16; ++c)
              nxt[c] = (row_ok && n0 + (ci + 1) * 16 + c < p.n_tok) ? o[(size_t)((ci + 1) * 16 + c) * p.ldo] : 0.f;
          }
          tmem_ld16(t_base + ci * 16, v);
          if (ci == nch - 1) {   // the last read of this accumulator: hand it back
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty(b));
          }
#pragma unroll
          for (int c = 0; c < 16; ++c)
            if (row_ok && n0 + ci * 16 + c < p.n_tok) o[(size_t)(ci * 16 + c) * p.ldo] = cur[c] + (v[c] + bias);
        }
        continue;
      }
      if (!mbar_wait(acc_full(b), acc_parity, p.error_flag, 3)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (p.splits == 1) {
        for (int c0 = 0; c0 < BN; c0 += 16) {
          if (n0 + c0 >= p.n_tok) break;
          float v[16];
          tmem_ld16(t_base + c0, v);
          if (c0 + 16 >= BN || n0 + c0 + 16 >= p.n_tok) {   // the last read of this accumulator: hand it back
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty(b));
          }
          tc_epilogue_store<BN>(p, v, m, n0 + c0, p.n_tok - (n0 + c0));
        }
      } else {
        float* ws = p.workspace + ((size_t)z * n_out_tiles + tile) * (BN * TC_BM);
        for (int c0 = 0; c0 < BN; c0 += 16) {
          if (n0 + c0 >= p.n_tok) break;
          float v[16];
          if (nkb > 0) tmem_ld16(t_base + c0, v);
          else {
#pragma unroll
            for (int c = 0; c < 16; ++c) v[c] = 0.f;
          }
#pragma unroll
          for (int c = 0; c < 16; ++c) ws[(c0 + c) * TC_BM + quad * 32 + lane] = v[c];
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty(b));
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");   // the four epilogue warps
        if (threadIdx.x == 64) s_last = (atomicAdd(&p.tickets[tile], 1) == p.splits - 1);
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const bool last = s_last != 0;
        asm volatile("bar.sync 1, 128;" ::: "memory");   // s_last may be rewritten by the next unit
        if (last) {
          __threadfence();
          for (int c0 = 0; c0 < BN; c0 += 16) {
            if (n0 + c0 >= p.n_tok) break;
            float v[16];
#pragma unroll
            for (int c = 0; c < 16; ++c) v[c] = 0.f;
            // partials in split order, four splits' loads in flight at a time
            const size_t zs = (size_t)n_out_tiles * (BN * TC_BM);
            const float* src0 = p.workspace + (size_t)tile * (BN * TC_BM) + c0 * TC_BM + quad * 32 + lane;
            int zz = 0;
            for (; zz + 4 <= p.splits; zz += 4) {
              float t[4][16];
#pragma unroll
              for (int q = 0; q < 4; ++q)
#pragma unroll
                for (int c = 0; c < 16; ++c) t[q][c] = __ldcg(src0 + (zz + q) * zs + c * TC_BM);
#pragma unroll
              for (int q = 0; q < 4; ++q)
#pragma unroll
                for (int c = 0; c < 16; ++c) v[c] += t[q][c];
            }
            for (; zz < p.splits; ++zz) {
#pragma unroll
              for (int c = 0; c < 16; ++c) v[c] += __ldcg(src0 + zz * zs + c * TC_BM);
            }
            tc_epilogue_store<BN>(p, v, m, n0 + c0, p.n_tok - (n0 + c0));
          }
          if (threadIdx.x == 64) p.tickets[tile] = 0;
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(tmem_cols));
  }
}

// ------------------------------------------------------------------------------------------------
// The same product on PAIRS of SMs (cta_group::2) for long prompts.
//
// A 128x256 tile per SM needs 48 KB from L2 per 64-deep k block, and with 227 KB of shared memory only
// four such stages fit: not enough work in flight to cover the latency of the loads, which is what holds
// the single-SM kernel at ~58 % tensor-pipe activity.  Two SMs of a cluster share one 256-token tile: each
// loads its own 128 weight rows and HALF of the token tile, one thread of the leader issues
// tcgen05.mma.cta_group::2 (M = 256 over both SMs' TMEM, N = 256), so a stage is 32 KB per SM for the same
// MMA work and six stages fit.  No multicast load is used: each SM fetches what it needs itself, and its
// copies report to the leader's mbarrier (the .cta_group::2 form of cp.async.bulk.tensor).
//
//   full[s]      in the leader; 64 KB expected per stage (both SMs' A and B halves)
//   empty[s]     in each SM; signalled by the leader's tcgen05.commit, multicast to the pair
//   acc_full[b]  in each SM (multicast commit);  acc_empty[b] in the leader, 8 arrivals (4 warps x 2 SMs)
constexpr int TP_BN = 256;              // widest token tile; an accumulator's columns in TMEM
constexpr int TP_STAGES = 6;
constexpr int TP_STAGE_BYTES = 2 * TC_BM * TC_BK * 2;   // A half-tile + B half-tile, 16 KB each
constexpr int TP_OUT_BYTES = 16 * TC_BM * 4;             // residual-add epilogue: [16 tokens][128 rows] fp32 on its way out
constexpr int TP_SMEM = TP_STAGES * TP_STAGE_BYTES + 2 * TP_OUT_BYTES + 1024 + 8 * (2 * TP_STAGES + 4) + 16;

__global__ void __launch_bounds__(TC_THREADS)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    const __grid_constant__ CUtensorMap map_out, TcParams p, int m_tiles, int n_tiles, int bn,
                    int out_tma) {   // tiles of 256 weight rows x bn tokens (bn % 16 == 0, <= 256); out_tma: map_out describes the output
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t out_smem = base + TP_STAGES * TP_STAGE_BYTES;      // two buffers of TP_OUT_BYTES
  uint8_t* const out_ptr = smem_raw + (out_smem - smem_u32(smem_raw));   // the same place as a generic address
  const uint32_t bars = out_smem + 2 * TP_OUT_BYTES;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (TP_STAGES + s); };
  auto acc_full = [&](int b) { return bars + 8u * (2 * TP_STAGES + b); };
  auto acc_empty = [&](int b) { return bars + 8u * (2 * TP_STAGES + 2 + b); };
  const uint32_t tmem_slot = bars + 8u * (2 * TP_STAGES + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();          // 0: leader, 1: peer
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int kblocks = (p.k + TC_BK - 1) / TC_BK;
  const int n_units = m_tiles * n_tiles;

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    for (int s = 0; s < TP_STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full(b), 1);
      mbar_init(acc_empty(b), 8);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(512));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  // both CTAs' barriers exist before anything signals across the pair
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  uint32_t tmem_d;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_d) : "r"(tmem_slot));

  pdl_launch_dependents();
  if (warp == 0) {
    if (lane == 0) {
      // ---- TMA producer (both CTAs): own 128 weight rows and own half of the token tile ----
      pdl_wait();
      int it = 0;
      bool ok = true;
      for (int u = pair; u < n_units && ok; u += n_pairs) {
        const int mt = u % m_tiles, nt = u / m_tiles;
        for (int i = 0; i < kblocks; ++i, ++it) {
          const int s = it % TP_STAGES;
          if (it >= TP_STAGES && !mbar_wait(empty_bar(s), ((it / TP_STAGES) - 1) & 1, p.error_flag, 5)) { ok = false; break; }
          const uint32_t leader_full = map_to_rank(full_bar(s), 0);
          if (rank == 0) mbar_expect_tx(full_bar(s), 2 * (TC_BM * TC_BK * 2 + (bn >> 1) * TC_BK * 2));
          const uint32_t dst = base + s * TP_STAGE_BYTES;
          tma_load_2d_pair(dst, &map_w, i * TC_BK, mt * 256 + (int)rank * TC_BM, leader_full);
          tma_load_2d_pair(dst + TC_BM * TC_BK * 2, &map_x, i * TC_BK, nt * bn + (int)rank * (bn >> 1), leader_full);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      // ---- MMA issuer (leader only): D fp32, A and B bf16 K-major, M = 256 over the pair, N = bn ----
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
      int it = 0, j = 0;
      bool ok = true;
      for (int u = pair; u < n_units && ok; u += n_pairs, ++j) {
        const int b = j & 1;
        if (j >= 2 && !mbar_wait(acc_empty(b), ((j >> 1) - 1) & 1, p.error_flag, 6)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d_addr = tmem_d + (uint32_t)(b * TP_BN);
        for (int i = 0; i < kblocks; ++i, ++it) {
          const int s = it % TP_STAGES;
          ok = mbar_wait(full_bar(s), (it / TP_STAGES) & 1, p.error_flag, 7);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = base + s * TP_STAGE_BYTES;
          const uint64_t a_desc = umma_desc(a_addr), b_desc = umma_desc(a_addr + TC_BM * TC_BK * 2);
#pragma unroll
          for (int k4 = 0; k4 < TC_BK / 16; ++k4)
            umma_bf16_pair(d_addr, a_desc + 2 * k4, b_desc + 2 * k4, idesc, (i > 0 || k4 > 0) ? 1u : 0u);
          umma_commit_pair(empty_bar(s));
        }
        if (ok) umma_commit_pair(acc_full(b));
      }
    }
  } else {
    // ---- epilogue warps (both CTAs): this CTA's 128 rows x 256 tokens ----
    const int quad = warp & 3;
    pdl_wait();
    int j = 0, n_out = 0;       // n_out: chunks this CTA has sent out through shared memory (residual-add epilogue)
    for (int u = pair; u < n_units; u += n_pairs, ++j) {
      const int mt = u % m_tiles, nt = u / m_tiles;
      const int b = j & 1;
      const int m = mt * 256 + (int)rank * TC_BM + quad * 32 + lane;
      const int n0 = nt * bn;
      const uint32_t t_base = tmem_d + ((uint32_t)(quad * 32) << 16) + (uint32_t)(b * TP_BN);
      const uint32_t leader_empty = map_to_rank(acc_empty(b), 0);
      if (!mbar_wait(acc_full(b), (j >> 1) & 1, p.error_flag, 8)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int nch = (min(bn, p.n_tok - n0) + 15) / 16;
      if (out_tma) {
        // The tile goes out through shared memory, 16 tokens at a time ([16 tokens][128 rows] in the output's type,
        // gated: [16][64 features]; two buffers), and is stored by TMA — for the residual stream ADDED by TMA
        // (cp.reduce.async.bulk.tensor .add): nothing of the old values comes to the SM.  The epilogue is a stream of
        // shared-memory stores instead of a chain of read-modify-write round trips or of 2-byte stores to global memory
        // (gated, the stores of the threads cost 7 to 10 us a product that the next tile's MMAs did not hide; it is
        // not hidden at all when a pair has one tile only: the o and down projections of a 2,048-token prompt).
        // Rows and tokens past the ends of `out` are clipped by the copy.
        const float bias = (p.bias && m < p.m_out) ? p.bias[m] : 0.f;
        const int row_in_cta = quad * 32 + lane;
        for (int ci = 0; ci < nch; ++ci) {
          float v[16];
          tmem_ld16(t_base + ci * 16, v);
          if (ci == nch - 1) {
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_remote(leader_empty);
          }
          const uint32_t buf_off = (uint32_t)((n_out & 1) * TP_OUT_BYTES);
          const uint32_t buf = out_smem + buf_off;
          uint8_t* const bufp = out_ptr + buf_off;
          if (n_out >= 2) {
            // the copy that read this buffer two chunks ago has to be done with it
            if (warp == 2 && lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            asm volatile("bar.sync 1, 128;" ::: "memory");
          }
          if (p.mode == OUT_SWIGLU) {
            // rows alternate gate and up (src/model/transformer.cpp:290; src/model/kernels.cpp:148): the even lane finishes
            // tokens 0..7 of feature row / 2, the odd lane tokens 8..15
            const bool is_gate = (row_in_cta & 1) == 0;
            float g[8], u[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              const float recv = __shfl_xor_sync(0xffffffffu, is_gate ? v[c + 8] : v[c], 1);
              g[c] = is_gate ? v[c] : recv;
              u[c] = is_gate ? recv : v[c + 8];
            }
            __nv_bfloat16* o = (__nv_bfloat16*)bufp + (is_gate ? 0 : 8) * (TC_BM / 2) + (row_in_cta >> 1);
#pragma unroll
            for (int c = 0; c < 8; ++c) o[c * (TC_BM / 2)] = __float2bfloat16_rn(__fdividef(g[c], 1.0f + __expf(-g[c])) * u[c]);
          } else if (p.mode == OUT_STORE) {
            __nv_bfloat16* o = (__nv_bfloat16*)bufp + row_in_cta;
#pragma unroll
            for (int c = 0; c < 16; ++c) o[c * TC_BM] = __float2bfloat16_rn(v[c] + bias);
          } else {
            float* o = (float*)bufp + row_in_cta;
#pragma unroll
            for (int c = 0; c < 16; ++c) o[c * TC_BM] = v[c] + bias;
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (warp == 2 && lane == 0) {
            const int r0 = mt * 256 + (int)rank * TC_BM;
            const int c0 = p.mode == OUT_SWIGLU ? (r0 >> 1) : r0;
            if (p.mode == OUT_ADD_F32)
              asm volatile(
                  "cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];"
                  ::"l"(&map_out), "r"(c0), "r"(n0 + ci * 16), "r"(buf)
                  : "memory");
            else
              asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];"
                           ::"l"(&map_out), "r"(c0), "r"(n0 + ci * 16), "r"(buf)
                           : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
          ++n_out;
        }
      } else {
        for (int ci = 0; ci < nch; ++ci) {
          float v[16];
          tmem_ld16(t_base + ci * 16, v);
          if (ci == nch - 1) {
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_remote(leader_empty);
          }
          tc_epilogue_store<TP_BN>(p, v, m, n0 + ci * 16, p.n_tok - (n0 + ci * 16));
        }
      }
    }
    // the additions still on their way read this CTA's shared memory: they are done before anybody leaves
    if (warp == 2 && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }
  // nobody leaves while its partner may still signal it or read its shared memory
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(512));
  }
}

// Width of the token tile for a product on pairs of SMs.  The device's pairs (74 on a B200) take the (256 rows x bn tokens) tiles in
// rounds, and a last round that is nearly empty costs as much as a full one: 2,048 tokens x 6,144 rows are 192
// tiles of 256 tokens (2.6 rounds, paid as 3), but 216 tiles of 240 tokens (2.9 rounds of 240/256 the length).
// A narrower tile also needs more bytes from L2 per flop (128 weight rows + bn/2 token rows a stage and SM), which
// bounds the tile's time from below.
static int pair_token_tile(int n_tok, int m_out) {
  static int fixed = -1;
  if (fixed < 0) {
    const char* e = getenv("LLMI_TC_PAIR_BN");
    fixed = e ? atoi(e) : 0;
  }
  if (fixed >= 128 && fixed <= 256 && fixed % 16 == 0) return fixed;
  const long m_tiles = (m_out + 255) / 256;
  const long n_pairs = sm_count() / 2 > 0 ? sm_count() / 2 : 1;
  int best = TP_BN;
  double best_cost = 0;
  for (int bn = TP_BN; bn >= 128; bn -= 16) {
    const long units = m_tiles * ((n_tok + bn - 1) / bn);
    const long rounds = (units + n_pairs - 1) / n_pairs;
    const double by_loads = 0.93 * (256 + bn) / 2;
    const double cost = rounds * (bn > by_loads ? bn : by_loads);
    if (bn == TP_BN || cost < best_cost * 0.97) {
      best = bn;
      best_cost = cost;
    }
  }
  return best;
}

static int launch_tc_pair(const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap& mo, TcParams p, int m_tiles,
                          int n_tiles, int bn, int out_tma, cudaStream_t stream) {
  static PerDevice<bool> configured_on;
  bool& configured = configured_on.here();
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_tc_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TP_SMEM) != cudaSuccess)
      return LLMI_ERR_LAUNCH;
    configured = true;
  }
  const long n_units = (long)m_tiles * n_tiles;
  const long n_pairs = sm_count() / 2 > 0 ? sm_count() / 2 : 1;     // one resident pair of CTAs per pair of SMs
  const long pairs = n_units < n_pairs ? n_units : n_pairs;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * pairs));
  cfg.blockDim = dim3(TC_THREADS);
  cfg.dynamicSmemBytes = TP_SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = pdl_enabled(PDL_GEMM) ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel, mw, mx, mo, p, m_tiles, n_tiles, bn, out_tma) == cudaSuccess ? LLMI_OK : LLMI_ERR_LAUNCH;
}

// ------------------------------------------------------------------------------------------------
// The same product for 17 to a few hundred tokens with no more output tiles than SMs (a decode step at batch 17..128,
// a short prompt): the k range is cut over the CTAs of a CLUSTER, and the stages are WIDE.
//
// Such a product is a read of W, and with 128-row tiles it has few of them (2,048 output rows: 16 tiles), so k must be
// cut for every SM to stream.  Through a workspace, the CTA that comes last adds all the partial tiles alone (16 splits
// of a 128x64 tile: half a megabyte read by one CTA — the o and down projections took 18 and 29 us at 64 tokens).
// Here the S CTAs that share an output tile form a cluster, each CTA finishes 1/S of the tile's rows, and nothing of
// the partial sums goes through global memory.
//
// A thread that issues a tensor copy is busy with it for about half a microsecond whatever its size up to 32 KB, and
// one thread's copies do not overlap (a block alone on its SM whose one producer thread requests 16 KB tiles takes in
// 30 GB/s whatever the depth of its ring; with 32 KB tiles 45 to 50, with 64 KB tiles up to 108 when few blocks run;
// two threads that take the stages in turn: 43 to 49 GB/s with 16 KB tiles).  Here a stage holds TWO 64-wide k blocks
// of both operands, each fetched by ONE copy of a three-dimensional box (k within a block, row, k block), and four
// threads in four warps issue the copies: two take the weight boxes of the stages in turn, two the token boxes.  One
// block per SM with a ring of about 190 KB.
//
// The way out.  Loads from another CTA's shared memory by threads are slow (a CTA that read 48 KB of its three
// peers' partial tiles with 16-byte loads, all in flight at once, took 5.4 us: 9 GB/s), and so are stores of 2 or 4
// bytes a lane while the next kernel's weight tiles queue at the memory.  So:
//   1. every CTA leaves its partial tile P [128 rows][BN tokens] fp32 in its own shared memory (over the ring);
//   2. after a cluster barrier one thread per peer sends that peer's rows of P by a bulk copy (shared memory to the
//      peer's shared memory, completion on the peer's mbarrier) into the slot R[sender] there;
//   3. the CTA of rank r adds rows r*128/S.. of P and of the R slots in rank order — local reads only —, applies the
//      epilogue and lays the result out token-major in a staging tile;
//   4. one thread stores (or, for the residual stream, adds) the staging tile by TMA.
// Outputs whose base or pitch is not a multiple of 16 bytes take the stores of the threads instead of step 4.
template <int BN>
struct WideConfig {
  static constexpr int KBS = 2;                                  // 64-wide k blocks per stage
  static constexpr int A_KB = TC_BM * TC_BK * 2;                 // one k block of the weight tile: 16 KB
  static constexpr int B_KB = BN * TC_BK * 2;
  static constexpr int A_BYTES = KBS * A_KB, B_BYTES = KBS * B_KB;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = BN == 128 ? 3 : 4;
  static constexpr int RED_STRIDE = BN + 4;                      // floats per row of P (16-byte skew: no bank conflicts)
  static constexpr int RED_BYTES = TC_BM * RED_STRIDE * 4;       // P; the S slots of R together are as large
  static constexpr int STAGING_BYTES = BN * TC_BM * 4;           // at most (one CTA of a cluster of S fills 1/S of it)
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  // cluster of one: P, staging; larger: P, R, staging / 2 at most
  static constexpr int OUT_BYTES_1 = RED_BYTES + STAGING_BYTES, OUT_BYTES_S = 2 * RED_BYTES + STAGING_BYTES / 2;
  static constexpr int OUT_BYTES = OUT_BYTES_1 > OUT_BYTES_S ? OUT_BYTES_1 : OUT_BYTES_S;
  static constexpr int DATA_BYTES = RING_BYTES > OUT_BYTES ? RING_BYTES : OUT_BYTES;
  static constexpr int SMEM_BYTES = DATA_BYTES + 1024 + 8 * (2 * STAGES + 3) + 16;
  static constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
};
constexpr int TW_THREADS = 288;     // warp 0, 6: weight producers; 1: MMA; 2..5: epilogue; 7, 8: token producers

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
// this CTA's shared memory to a peer's (both addresses 16-byte aligned, bytes a multiple of 16); completes on the peer's barrier
__device__ __forceinline__ void bulk_send(uint32_t dst_cluster, uint32_t src, uint32_t bytes, uint32_t bar_cluster) {
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst_cluster), "r"(src), "r"(bytes), "r"(bar_cluster)
               : "memory");
}

// Steps 3 and 4 for a cluster of S, run by NT threads (whole warps, te = 0..NT-1, named barrier 2).
template <int BN, int NT, int S>
__device__ __forceinline__ void wide_way_out(const TcParams& p, const CUtensorMap* map_out, int out_tma, uint32_t base, uint8_t* smem_base,
                                             int rank, int mt, int nt, int te) {   // smem_base: the generic address of `base`
  using C = WideConfig<BN>;
  constexpr int RP = TC_BM / S;                 // rows of this CTA
  constexpr int GROUPS = NT / RP;               // groups of columns (tokens)
  constexpr int CPT = BN / GROUPS;              // columns per thread
  static_assert(CPT >= 4 && CPT % 4 == 0, "a thread takes whole 16-byte pieces");
  constexpr int NQ = CPT / 4;
  constexpr uint32_t SLICE_BYTES = RP * C::RED_STRIDE * 4;
  const int row = te % RP, cg = te / RP;
  const int m = mt * TC_BM + rank * RP + row;
  // own rows of P and of the slots, the own slot excepted (nobody sends to itself)
  float v[CPT];
#pragma unroll
  for (int c = 0; c < CPT; ++c) v[c] = 0.f;
  {
    float4 t[NQ][S];
#pragma unroll
    for (int r = 0; r < S; ++r) {
      const uint32_t src = r == rank ? base + (uint32_t)(rank * RP) * (C::RED_STRIDE * 4) : base + C::RED_BYTES + (uint32_t)r * SLICE_BYTES;
      const uint32_t addr = src + (uint32_t)(row * C::RED_STRIDE + cg * CPT) * 4u;
#pragma unroll
      for (int q = 0; q < NQ; ++q)
        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(t[q][r].x), "=f"(t[q][r].y), "=f"(t[q][r].z), "=f"(t[q][r].w) : "r"(addr + 16u * q));
    }
#pragma unroll
    for (int q = 0; q < NQ; ++q)
#pragma unroll
      for (int r = 0; r < S; ++r) {      // rank order
        v[4 * q] += t[q][r].x;
        v[4 * q + 1] += t[q][r].y;
        v[4 * q + 2] += t[q][r].z;
        v[4 * q + 3] += t[q][r].w;
      }
  }
  const int n_base = nt * BN + cg * CPT;
  if (!out_tma) {
#pragma unroll
    for (int ch = 0; ch < (CPT + 15) / 16; ++ch) {
      float w[16];
#pragma unroll
      for (int c = 0; c < 16; ++c) w[c] = ch * 16 + c < CPT ? v[ch * 16 + c] : 0.f;
      const int width = CPT - ch * 16 < 16 ? CPT - ch * 16 : 16;
      tc_epilogue_store<BN>(p, w, m, n_base + ch * 16, min(width, p.n_tok - (n_base + ch * 16)));
    }
    return;
  }
  // the staging tile: [BN tokens][RP rows] (gated: [BN][RP / 2] features), dense.  Plain stores, all values first: a
  // chain of exchange, exponential, division and store per token, each waiting for the one before, cost 5 us a tile.
  const uint32_t staging_off = S == 1 ? C::RED_BYTES : 2 * C::RED_BYTES;
  const uint32_t staging = base + staging_off;
  uint8_t* const stg = smem_base + staging_off;
  if (p.mode == OUT_SWIGLU) {
    // rows alternate gate and up (src/model/transformer.cpp:290; src/model/kernels.cpp:148): the even lane takes the
    // odd lane's up and finishes feature row / 2
    __nv_bfloat16* o = (__nv_bfloat16*)stg + (size_t)(cg * CPT) * (RP / 2) + (row >> 1);
    float up[CPT];
#pragma unroll
    for (int c = 0; c < CPT; ++c) up[c] = __shfl_down_sync(0xffffffffu, v[c], 1);
    if (!(row & 1)) {
#pragma unroll
      for (int c = 0; c < CPT; ++c) o[c * (RP / 2)] = __float2bfloat16_rn(__fdividef(v[c], 1.0f + __expf(-v[c])) * up[c]);
    }
  } else {
    const float b = (p.bias && m < p.m_out) ? p.bias[m] : 0.f;
    if (p.mode == OUT_STORE) {
      __nv_bfloat16* o = (__nv_bfloat16*)stg + (size_t)(cg * CPT) * RP + row;
#pragma unroll
      for (int c = 0; c < CPT; ++c) o[c * RP] = __float2bfloat16_rn(v[c] + b);
    } else {
      float* o = (float*)stg + (size_t)(cg * CPT) * RP + row;
#pragma unroll
      for (int c = 0; c < CPT; ++c) o[c * RP] = v[c] + b;
    }
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the staging tile is read by the async proxy
  asm volatile("bar.sync 2, %0;" ::"n"(NT) : "memory");
  if (te == 0) {
    const int m0 = mt * TC_BM + rank * RP;
    const int c0 = p.mode == OUT_SWIGLU ? (m0 >> 1) : m0, c1 = nt * BN;
    if (p.mode == OUT_ADD_F32)
      asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];"
                   ::"l"(map_out), "r"(c0), "r"(c1), "r"(staging) : "memory");
    else
      asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];"
                   ::"l"(map_out), "r"(c0), "r"(c1), "r"(staging) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // the staging tile has been read: the block may end
  }
}

// boxed3d: the operand maps are three-dimensional (k a multiple of 64); else two-dimensional, one copy per k block.
// out_tma: map_out describes the output for step 4 (box [BN tokens][128 / S rows], gated: half the rows).
template <int BN>
__global__ void __launch_bounds__(TW_THREADS)
gemm_tc_wide_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    const __grid_constant__ CUtensorMap map_out, TcParams p, int m_tiles, int S, int boxed3d,
                    int out_tma) {   // gridDim.x = tiles * S, cluster (S, 1, 1); S in {1, 2, 4}
  using C = WideConfig<BN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* const smem_base = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bars = base + C::DATA_BYTES;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (C::STAGES + s); };
  const uint32_t acc_full = bars + 8u * (2 * C::STAGES);
  const uint32_t recv_bar = bars + 8u * (2 * C::STAGES + 1);
  const uint32_t tmem_slot = bars + 8u * (2 * C::STAGES + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = (int)cluster_rank();
  const int tile = blockIdx.x / S;
  const int mt = tile % m_tiles, nt = tile / m_tiles;
  const int kblocks = (p.k + TC_BK - 1) / TC_BK;
  const int per = (kblocks + S - 1) / S;
  const int kb0 = rank * per;
  const int nkb = max(0, min(kblocks, kb0 + per) - kb0);
  const int nst = (nkb + C::KBS - 1) / C::KBS;          // stages; the last one may hold one k block that counts
  const uint32_t slice_bytes = (uint32_t)(TC_BM / S) * (C::RED_STRIDE * 4);

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    if (out_tma) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_out) : "memory");
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(acc_full, 1);
    mbar_init(recv_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (S > 1) mbar_expect_tx(recv_bar, (uint32_t)(S - 1) * slice_bytes);    // what the peers will send, long before they do
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(C::TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  uint32_t tmem_d;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_d) : "r"(tmem_slot));

  pdl_launch_dependents();
  if (warp == 0 || warp >= 6) {
    if (lane == 0) {
      // ---- producers.  The weights do not depend on the kernel before, the tokens do.  A stage's full barrier is in
      // its new phase once its empty barrier has completed, so token bytes that land before the weight producer has
      // announced the stage still count for the right phase.
      const bool tokens = warp >= 7;
      const int me = tokens ? warp - 7 : (warp == 0 ? 0 : 1);
      if (tokens) pdl_wait();
      for (int i = me; i < nst; i += 2) {
        const int s = i % C::STAGES;
        if (i >= C::STAGES && !mbar_wait(empty_bar(s), ((i / C::STAGES) - 1) & 1, p.error_flag, tokens ? 26 : 21)) break;
        const int kb = kb0 + i * C::KBS;           // (a k block past this CTA's range is fetched and not multiplied)
        const uint32_t dst = base + s * C::STAGE_BYTES + (tokens ? C::A_BYTES : 0);
        if (!tokens) mbar_expect_tx(full_bar(s), C::STAGE_BYTES);
        if (boxed3d) {
          if (tokens) tma_load_3d(dst, &map_x, 0, nt * BN, kb, full_bar(s));
          else tma_load_3d(dst, &map_w, 0, mt * TC_BM, kb, full_bar(s));
        } else {
#pragma unroll
          for (int j = 0; j < C::KBS; ++j) {
            if (tokens) tma_load_2d(dst + j * C::B_KB, &map_x, (kb + j) * TC_BK, nt * BN, full_bar(s));
            else tma_load_2d(dst + j * C::A_KB, &map_w, (kb + j) * TC_BK, mt * TC_BM, full_bar(s));
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer ----
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
      bool ok = true;
      for (int i = 0; i < nst; ++i) {
        const int s = i % C::STAGES;
        ok = mbar_wait(full_bar(s), (i / C::STAGES) & 1, p.error_flag, 22);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_addr = base + s * C::STAGE_BYTES;
        const int nk = min(C::KBS, nkb - i * C::KBS);
        for (int j = 0; j < nk; ++j) {
          const uint64_t a_desc = umma_desc(a_addr + j * C::A_KB), b_desc = umma_desc(a_addr + C::A_BYTES + j * C::B_KB);
#pragma unroll
          for (int k4 = 0; k4 < TC_BK / 16; ++k4)
            umma_bf16(tmem_d, a_desc + 2 * k4, b_desc + 2 * k4, idesc, (i > 0 || j > 0 || k4 > 0) ? 1u : 0u);
        }
        umma_commit(empty_bar(s));
      }
      if (nkb > 0 && ok) umma_commit(acc_full);   // arrives when every product above has finished
      else mbar_arrive(acc_full);
    }
  } else {
    // ---- epilogue warps (2..5), step 1: this CTA's partial tile into its own shared memory (over the ring) ----
    const int quad = warp & 3;
    pdl_wait();
    mbar_wait(acc_full, 0, p.error_flag, 23);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t row_addr = base + (uint32_t)((quad * 32 + lane) * C::RED_STRIDE) * 4u;
    const uint32_t t_base = tmem_d + ((uint32_t)(quad * 32) << 16);
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 16) {
      float v[16];
      if (nkb > 0) tmem_ld16(t_base + c0, v);
      else {
#pragma unroll
        for (int c = 0; c < 16; ++c) v[c] = 0.f;
      }
#pragma unroll
      for (int q = 0; q < 4; ++q)
        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + (uint32_t)(c0 + 4 * q) * 4u), "f"(v[4 * q]),
                     "f"(v[4 * q + 1]), "f"(v[4 * q + 2]), "f"(v[4 * q + 3])
                     : "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // P is read by the bulk copies below
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  bool received = true;
  if (S > 1) {
    // every CTA's partial tile is in place and its ring is free
    cluster_sync_all();
    // ---- step 2: one thread per peer sends that peer's rows ----
    if (lane == 0 && warp >= 1 && warp <= S && warp - 1 != rank) {
      const uint32_t peer = (uint32_t)(warp - 1);
      bulk_send(map_to_rank(base + C::RED_BYTES + (uint32_t)rank * slice_bytes, peer), base + peer * slice_bytes, slice_bytes,
                map_to_rank(recv_bar, peer));
    }
    received = mbar_wait(recv_bar, 0, p.error_flag, 27);
    // Nobody may leave while a copy that it sent still reads its shared memory: every peer says here that it has
    // received, and the wait is at the end, behind the way out.
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  } else {
    __syncthreads();
  }
  // ---- steps 3 and 4 (the producer and MMA warps have nothing left to do: all but warp 0 help where the tile is wide enough)
  if (received) {
    if constexpr (BN >= 64) {
      if (warp >= 1) {
        const int te = threadIdx.x - 32;
        if (S == 1) wide_way_out<BN, 256, 1>(p, &map_out, out_tma, base, smem_base, rank, mt, nt, te);
        else if (S == 2) wide_way_out<BN, 256, 2>(p, &map_out, out_tma, base, smem_base, rank, mt, nt, te);
        else wide_way_out<BN, 256, 4>(p, &map_out, out_tma, base, smem_base, rank, mt, nt, te);
      }
    } else {
      if (warp >= 2 && warp < 6) {
        const int te = threadIdx.x - 64;
        if (S == 1) wide_way_out<BN, 128, 1>(p, &map_out, out_tma, base, smem_base, rank, mt, nt, te);
        else if (S == 2) wide_way_out<BN, 128, 2>(p, &map_out, out_tma, base, smem_base, rank, mt, nt, te);
        else wide_way_out<BN, 128, 4>(p, &map_out, out_tma, base, smem_base, rank, mt, nt, te);
      }
    }
  }
  if (S > 1) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  else __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(C::TMEM_COLS));
  }
}

// Cluster size for a product of `tiles` output tiles and `kblocks` 64-wide k blocks: the larger of 4 and 2 that leaves
// every CTA at least four k blocks and does not ask for more CTAs than SMs (one block per SM), else 1.  Clusters of
// eight such blocks have few places on the device (measured, 2,048 x 2,048 at 128 tokens: 24.4 us in clusters of
// eight, 14.1 us in clusters of four).
static int wide_cluster(long tiles, int kblocks) {
  for (int s = 4; s >= 2; s >>= 1)
    if (tiles * s <= sm_count() && kblocks / s >= 4) return s;
  return 1;
}

template <int BN>
static int launch_tc_wide(const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap& mo, TcParams p, int m_tiles, int n_tiles,
                          int S, int boxed3d, int out_tma, cudaStream_t stream) {
  using C = WideConfig<BN>;
  static PerDevice<bool> configured_on;
  bool& configured = configured_on.here();
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_tc_wide_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess)
      return LLMI_ERR_LAUNCH;
    configured = true;
  }
  const long tiles = (long)m_tiles * n_tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(tiles * S));
  cfg.blockDim = dim3(TW_THREADS);
  cfg.dynamicSmemBytes = C::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)S;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = pdl_enabled(PDL_GEMM) ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return cudaLaunchKernelEx(&cfg, gemm_tc_wide_kernel<BN>, mw, mx, mo, p, m_tiles, S, boxed3d, out_tma) == cudaSuccess ? LLMI_OK
                                                                                                               : LLMI_ERR_LAUNCH;
}

// ------------------------------------------------------------------------------------------- host

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)sym;
  }
  return fn;
}

// A [rows, k] bf16 matrix with row pitch ld (elements), tiles of [box_rows, 64], 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* ptr, long rows, long k, long ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return LLMI_ERR_DRIVER;
  const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? LLMI_OK : LLMI_ERR_DRIVER;
}

// The same matrix (k a multiple of 64) seen as (k within a 64-wide block, row, k block): boxes of [kbs][box_rows][64].
static int make_map_3d(CUtensorMap* map, const void* ptr, long rows, long k, long ld, int box_rows, int kbs) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return LLMI_ERR_DRIVER;
  const cuuint64_t dims[3] = {(cuuint64_t)TC_BK, (cuuint64_t)rows, (cuuint64_t)(k / TC_BK)};
  const cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)TC_BK * 2};
  const cuuint32_t box[3] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows, (cuuint32_t)kbs};
  const cuuint32_t elem[3] = {1, 1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? LLMI_OK : LLMI_ERR_DRIVER;
}

template <int BN>
static int launch_tc(const CUtensorMap& mw, const CUtensorMap& mx, TcParams p, int m_tiles, int n_tiles,
                     cudaStream_t stream) {
  using C = TcConfig<BN>;
  static PerDevice<bool> configured_on;
  bool& configured = configured_on.here();
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess)
      return LLMI_ERR_LAUNCH;
    configured = true;
  }
  const long n_units = (long)m_tiles * n_tiles * p.splits;
  const long resident = (long)sm_count() * C::CTAS_PER_SM;
  const int grid = (int)(n_units < resident ? n_units : resident);
  return launch_pdl(PDL_GEMM, gemm_tc_kernel<BN>, grid, TC_THREADS, C::SMEM_BYTES, stream, mw, mx, p, m_tiles, n_tiles);
}

}  // namespace llmi

using namespace llmi;

// Width of the token tile.  Up to 128 tokens: the tokens are one tile.  Beyond that, 128 while that makes no more
// tiles than the device has SMs — few tiles want their k range cut over a cluster, which the cluster kernel does
// for tiles up to 128 wide (the o projection of a 256-token prompt, 2,048 x 2,048: 16 tiles of 256 tokens cut 8
// ways through a workspace took 53 us, of which the CTA that came last spent most adding eight partial tiles
// alone) — else 256.
static int tc_bn(int n_tok, int m_out) {
  if (n_tok <= 128) return n_tok <= 16 ? 16 : n_tok <= 32 ? 32 : n_tok <= 64 ? 64 : 128;
  const long tiles128 = (long)((m_out + TC_BM - 1) / TC_BM) * ((n_tok + 127) / 128);
  return tiles128 <= sm_count() ? 128 : 256;
}
static int tc_ctas_per_sm(int bn) { return bn <= 32 ? LLMI_TC_SMALL_CTAS : (bn == 64 ? 2 : 1); }

// How many k-splits a product of this shape gets (a function of the shape only): enough blocks to
// fill every SM's resident slots once, each with at least four k-blocks to stream.
LLMI_EXPORT int llmi_gemm_tc_splits(int n_tok, int m_out, int k) {
  const int bn = tc_bn(n_tok, m_out);
  const long tiles = (long)((m_out + TC_BM - 1) / TC_BM) * ((n_tok + bn - 1) / bn);
  const int kblocks = (k + TC_BK - 1) / TC_BK;
  const long slots = (long)sm_count() * tc_ctas_per_sm(bn);
  if (tiles * 2 > slots || kblocks < 8) return 1;
  int s = (int)(slots / tiles);
  if (s > kblocks / 4) s = kblocks / 4;
  if (s > 16) s = 16;
  return s < 1 ? 1 : s;
}

// The output as [n_tok][cols] of bf16 or fp32 with boxes of [box_tok tokens][box_cols]: the way out by TMA of the
// cluster kernel and of the kernel on pairs of SMs.  LLMI_ERR_ALIGN if its base or pitch is not a multiple of 16 bytes (the caller then lets the threads store).
static int make_out_map(CUtensorMap* map, void* out, long n_tok, long cols, long ldo, int elem_bytes, int box_cols, int box_tok) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return LLMI_ERR_DRIVER;
  if (((uintptr_t)out & 15) || ((ldo * elem_bytes) & 15) || ((box_cols * elem_bytes) & 15)) return LLMI_ERR_ALIGN;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)n_tok};
  const cuuint64_t strides[1] = {(cuuint64_t)ldo * elem_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_tok};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(map, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, out, dims, strides,
                        box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? LLMI_OK : LLMI_ERR_DRIVER;
}

// The wide-stage cluster kernel takes the products of 17 to a few hundred tokens whose 128-row tiles are no more than the
// SMs (one block per SM): its cluster size, 0 if the product is not its own.  (LLMI_TC_WIDE=0 switches it off.)
static int tc_wide_cluster(int n_tok, int m_out, int k) {
  static int enabled = -1;
  if (enabled < 0) {
    const char* e = getenv("LLMI_TC_WIDE");
    enabled = (e && e[0] == '0') ? 0 : 1;
  }
  const int bn = tc_bn(n_tok, m_out);
  if (!enabled || bn < 32 || bn > 128) return 0;
  const long tiles = (long)((m_out + TC_BM - 1) / TC_BM) * ((n_tok + bn - 1) / bn);
  if (tiles > sm_count()) return 0;
  return wide_cluster(tiles, (k + TC_BK - 1) / TC_BK);
}

// 64-wide k blocks that one CTA accumulates before partial sums are added across CTAs (the whole k range when
// nothing is cut): two products of the same weights add in the same order exactly when this number agrees.
LLMI_EXPORT int llmi_gemm_tc_k_per_cta(int n_tok, int m_out, int k) {
  const int kblocks = (k + TC_BK - 1) / TC_BK;
  const int W = tc_wide_cluster(n_tok, m_out, k);
  const int cuts = W ? W : llmi_gemm_tc_splits(n_tok, m_out, k);
  return (kblocks + cuts - 1) / cuts;
}

// Bytes of fp32 workspace and number of int tickets the product needs (both 0 without split-K).
LLMI_EXPORT long llmi_gemm_tc_workspace(int n_tok, int m_out, int k, int* n_tickets) {
  const int s = llmi_gemm_tc_splits(n_tok, m_out, k);
  const int bn = tc_bn(n_tok, m_out);
  const long tiles = (long)((m_out + TC_BM - 1) / TC_BM) * ((n_tok + bn - 1) / bn);
  if (n_tickets) *n_tickets = s > 1 ? (int)tiles : 0;
  return s > 1 ? (long)s * tiles * bn * TC_BM * 4 : 0;
}

// y[n_tok, m_out] (mode) = x[n_tok, k] · w[m_out, k]ᵀ + bias; bf16 inputs; pitches in elements.
// mode 3 (gated): w's rows alternate gate and up rows of a feed-forward, y is [n_tok, m_out / 2] bf16 and
// receives silu(gate) * up.
// Requirements (else LLMI_ERR_ALIGN): x, w 16-byte aligned; ldx, ldw multiples of 8 elements.
LLMI_EXPORT int llmi_gemm_tc(const void* x, long ldx, const void* w, long ldw, const float* bias, void* y, long ldy,
                             int n_tok, int m_out, int k, int mode, float* workspace, long workspace_bytes,
                             int* tickets, int n_tickets, int* error_flag, cudaStream_t stream) {
  if (n_tok <= 0 || m_out <= 0 || k <= 0) return LLMI_ERR_BAD_SIZE;
  if (mode < 0 || mode > 3) return LLMI_ERR_UNSUPPORTED;
  if (mode == OUT_SWIGLU && ((m_out & 1) || bias)) return LLMI_ERR_UNSUPPORTED;
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15) || (ldx & 7) || (ldw & 7)) return LLMI_ERR_ALIGN;
  const int bn = tc_bn(n_tok, m_out);
  int need_tickets = 0;
  const long need_ws = llmi_gemm_tc_workspace(n_tok, m_out, k, &need_tickets);
  int splits = llmi_gemm_tc_splits(n_tok, m_out, k);
  if (splits > 1 && (need_ws > workspace_bytes || need_tickets > n_tickets || !workspace || !tickets)) splits = 1;
  CUtensorMap mw, mx;
  int rc;
  const int W = tc_wide_cluster(n_tok, m_out, k);
  if (W) {
    const int boxed3d = (k % TC_BK) == 0;
    rc = boxed3d ? make_map_3d(&mw, w, m_out, k, ldw, TC_BM, 2) : make_map(&mw, w, m_out, k, ldw, TC_BM);
    if (rc != LLMI_OK) return rc;
    rc = boxed3d ? make_map_3d(&mx, x, n_tok, k, ldx, bn, 2) : make_map(&mx, x, n_tok, k, ldx, bn);
    if (rc != LLMI_OK) return rc;
    TcParams pk{m_out, n_tok, k, y, ldy, bias, mode, 1, nullptr, nullptr, error_flag};
    const int m_tiles = (m_out + TC_BM - 1) / TC_BM, n_tiles = (n_tok + bn - 1) / bn;
    // the way out by TMA: a CTA of a cluster of W stores [bn tokens][128 / W rows] (gated: half as many features)
    CUtensorMap mo = mw;
    const int gated = mode == OUT_SWIGLU;
    const int out_rc = make_out_map(&mo, y, n_tok, gated ? m_out / 2 : m_out, ldy, (mode == OUT_STORE || gated) ? 2 : 4,
                                         (TC_BM / W) >> gated, bn);
    if (out_rc == LLMI_ERR_DRIVER) return out_rc;
    const int out_tma = out_rc == LLMI_OK;
    if (bn == 32) return launch_tc_wide<32>(mw, mx, mo, pk, m_tiles, n_tiles, W, boxed3d, out_tma, stream);
    if (bn == 64) return launch_tc_wide<64>(mw, mx, mo, pk, m_tiles, n_tiles, W, boxed3d, out_tma, stream);
    return launch_tc_wide<128>(mw, mx, mo, pk, m_tiles, n_tiles, W, boxed3d, out_tma, stream);
  }
  rc = make_map(&mw, w, m_out, k, ldw, TC_BM);
  if (rc != LLMI_OK) return rc;
  // long prompts: pairs of SMs share a 256-token tile (each loads 128 of its rows)
  static int pair_ok = -1;
  if (pair_ok < 0) {
    const char* e = getenv("LLMI_TC_PAIR");
    pair_ok = (e && e[0] == '0') ? 0 : 1;
  }
  // The pair kernel's tiles leave by TMA, 16 tokens at a time ([16][128 rows] in the output's type, gated [16][64]):
  // the output must then be 16-byte aligned with a pitch of whole 16 bytes.  If it is not, the threads store — except
  // into the residual stream, which the pair kernel only adds to by TMA (such a product takes the single-SM kernel).
  // pairs of SMs: from 256 tokens on, where the shape has more 128-wide tiles than SMs (bn == 256)
  if (pair_ok && n_tok >= 256 && (bn == 256 || n_tok >= 512) && splits == 1) {
    const int gated = mode == OUT_SWIGLU;
    CUtensorMap mo = mw;
    const int out_rc = make_out_map(&mo, y, n_tok, gated ? m_out / 2 : m_out, ldy, (mode == OUT_STORE || gated) ? 2 : 4,
                                         TC_BM >> gated, 16);
    if (out_rc == LLMI_ERR_DRIVER) return out_rc;
    if (out_rc == LLMI_OK || mode != OUT_ADD_F32) {
      const int pbn = pair_token_tile(n_tok, m_out);
      rc = make_map(&mx, x, n_tok, k, ldx, pbn / 2);
      if (rc != LLMI_OK) return rc;
      TcParams pp{m_out, n_tok, k, y, ldy, bias, mode, 1, workspace, tickets, error_flag};
      return launch_tc_pair(mw, mx, mo, pp, (m_out + 255) / 256, (n_tok + pbn - 1) / pbn, pbn, out_rc == LLMI_OK, stream);
    }
  }
  rc = make_map(&mx, x, n_tok, k, ldx, bn);
  if (rc != LLMI_OK) return rc;
  TcParams p{m_out, n_tok, k, y, ldy, bias, mode, splits, workspace, tickets, error_flag};
  const int m_tiles = (m_out + TC_BM - 1) / TC_BM, n_tiles = (n_tok + bn - 1) / bn;
  if ((long)m_tiles * n_tiles * splits > 0x7fffffffL) return LLMI_ERR_BAD_SIZE;
  switch (bn) {
    case 16: return launch_tc<16>(mw, mx, p, m_tiles, n_tiles, stream);
    case 32: return launch_tc<32>(mw, mx, p, m_tiles, n_tiles, stream);
    case 64: return launch_tc<64>(mw, mx, p, m_tiles, n_tiles, stream);
    case 128: return launch_tc<128>(mw, mx, p, m_tiles, n_tiles, stream);
    default: return launch_tc<256>(mw, mx, p, m_tiles, n_tiles, stream);
  }
}
