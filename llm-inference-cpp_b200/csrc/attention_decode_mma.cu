// Decode attention for GROUPED queries on the tensor cores (mma.sync), bf16, head size 64 or 128.
//
// Same operation and the same frame as attention_decode.cu (reference loop: src/model/transformer.cpp:263-282
// with T = 1): persistent blocks over (sequence, kv head, split) items, a producer warp that keeps a ring of
// cache pages full, four consumer warps that take 16 keys of every page each, an epilogue warp for the items
// that are cut into splits, partial results merged in split order through a workspace and tickets.  What
// differs is the arithmetic.  The kernel of attention_decode.cu computes every query head's dot products on
// the CUDA cores, so its work grows with the group size g = heads / kv heads while the bytes it reads do not:
// at g = 3 it reaches half the memory bandwidth, at g = 8 a seventh.  Here the g query heads that share a kv
// head are the ROWS of one MMA tile (16 rows, the ones past g are zero):
//
//   S[16 heads x 16 keys] = Q[16 x hd] · K_pageᵀ     mma.sync m16n8k16, K fragments by ldmatrix
//   softmax per row in the accumulator layout (base 2, one ex2 per key), P packed to bf16 in registers
//   O[16 heads x hd]     += P[16 x 16] · V_page        V fragments by ldmatrix.trans
//
// so the work per page does not depend on g.  The pages come by TMA with the 128-byte swizzle that ldmatrix
// wants (the cache of a layer seen as a matrix [pages * kv heads * 64 rows, hd]).  With `fuse` the kernel also
// does the step's position encoding, as attention_decode.cu does (rope_store.cu's arithmetic: the same bits).
#include <cuda.h>
#include <math.h>

#include "common.cuh"
#include "sm100.cuh"

namespace llmi {

constexpr int DM_PAGE = 64;
constexpr int DM_CONSUMERS = 4;
constexpr int DM_THREADS = (DM_CONSUMERS + 2) * 32;

struct DecodeMmaParams {
  const __nv_bfloat16* q;   // [tokens, >= n_heads*HD] (fused: the un-rotated [q | k | v] rows), row pitch ldq
  long ldq;
  __nv_bfloat16* out;       // [tokens, n_heads*HD], row pitch ldo
  long ldo;
  const int32_t* seq_pages;   // [n_seqs, pages_stride]
  const int32_t* seq_kv_len;  // [n_seqs] length after this step (0: padding)
  const int32_t* seq_q_start; // [n_seqs] row of the sequence's token
  int pages_stride;
  int n_kv_heads;
  int group;                 // query heads per kv head (<= G)
  float scale_log2;          // softmax scale * log2(e)
  int window;
  int pages_per_split;
  int max_splits;
  float* partials;           // [n_seqs, n_kv_heads, max_splits, group, HD + 2]
  int* tickets;              // [n_seqs * n_kv_heads], zero between launches
  int* error_flag;
  int fuse;
  const float* inv_freq;     // [HD / 2] when rotary_dim > 0
  int rotary_dim;
  int n_heads;
  int write_kv;
  __nv_bfloat16* k_cache_w;  // the caches, writable (fused append)
  __nv_bfloat16* v_cache_w;
};

template <int HD>
struct DmCfg {
  static constexpr int NSUB = HD / 64;                    // 64-column sub-tiles of a page tile
  static constexpr int SUB_BYTES = DM_PAGE * 64 * 2;      // 8 KB
  static constexpr int TILE_BYTES = NSUB * SUB_BYTES;
  static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  static constexpr int STAGES = HD <= 64 ? 4 : 3;
  static constexpr int BAR_BYTES = 8 * (2 * STAGES + 4) + 32;
  static constexpr int ROT_BYTES = STAGES * HD * 4;       // per stage: sin[HD/2], cos[HD/2] of the item that starts there
  // the warps' partial results (values, max, sum) and two buffers of merged results on their way to the epilogue
  // warp: [4 + 2][group][HD + 2] floats
  static constexpr int smem_bytes(int group) {
    return STAGES * STAGE_BYTES + 1024 + BAR_BYTES + ROT_BYTES + (DM_CONSUMERS + 2) * group * (HD + 2) * 4;
  }
};

__device__ __forceinline__ void dm_mma(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t dm_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 dm_unpack(uint32_t w) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
}
__device__ __forceinline__ void dm_tma(uint32_t dst, const CUtensorMap* map, int col, int row, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(col), "r"(row)
      : "memory");
}

struct DmItem {
  int seq, kvh, part, n_parts, lo, pos, pg0, n_pages, tok;
};

template <int HD>
__global__ void __launch_bounds__(DM_THREADS, 2)
attention_decode_mma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            DecodeMmaParams p, int n_items) {
  using C = DmCfg<HD>;
  extern __shared__ uint8_t smem_raw[];
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.group;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = base + C::STAGES * C::STAGE_BYTES;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (C::STAGES + s); };
  auto rfull_bar = [&](int b) { return bars + 8u * (2 * C::STAGES + b); };
  auto rempty_bar = [&](int b) { return bars + 8u * (2 * C::STAGES + 2 + b); };
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw)) + C::STAGES * C::STAGE_BYTES + C::BAR_BYTES;
  float* rot_tab = reinterpret_cast<float*>(gen);
  float* s_warp = rot_tab + C::STAGES * HD;                         // [4 warps][group][HD + 2]: values, max, sum
  float* r_buf = s_warp + DM_CONSUMERS * G * (HD + 2);           // [2][group][HD + 2]
  const bool rotate = p.fuse && p.rotary_dim > 0;
  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), DM_CONSUMERS);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(rfull_bar(b), 1);
      mbar_init(rempty_bar(b), 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // The first non-empty item at or after `item` in this block's sequence of items (stride gridDim.x).
  auto next_item = [&](int item, DmItem& d) -> int {
    for (; item < n_items; item += gridDim.x) {
      const int split = item % p.max_splits;
      const int sh = item / p.max_splits;
      d.kvh = sh % p.n_kv_heads;
      d.seq = sh / p.n_kv_heads;
      const int kv_len = p.seq_kv_len[d.seq];
      if (kv_len <= 0) continue;                                   // padding sequence
      d.pos = kv_len - 1;
      d.lo = (p.window > 0 && kv_len - p.window > 0) ? kv_len - p.window : 0;
      const int first_page = d.lo / DM_PAGE, last_page = d.pos / DM_PAGE;
      const int first_split = first_page / p.pages_per_split, last_split = last_page / p.pages_per_split;
      if (split < first_split || split > last_split) continue;
      d.part = split - first_split;
      d.n_parts = last_split - first_split + 1;
      d.pg0 = max(first_page, split * p.pages_per_split);
      d.n_pages = min(last_page + 1, (split + 1) * p.pages_per_split) - d.pg0;
      d.tok = p.seq_q_start[d.seq];
      return item;
    }
    return n_items;
  };

  if (warp == DM_CONSUMERS) {
    // ---- producer (lane 0 issues the copies; the whole warp appends a sequence-head's new k and v) ----
    int it = 0;
    DmItem d;
    bool ok = true, waited = false;
    for (int item = next_item(blockIdx.x, d); item < n_items && ok; item = next_item(item + gridDim.x, d)) {
      const int32_t* pages = p.seq_pages + (size_t)d.seq * p.pages_stride;
      for (int i = 0; i < d.n_pages && ok; ++i, ++it) {
        const int s = it % C::STAGES;
        const bool newest = (d.pg0 + i + 1) * DM_PAGE > d.pos;   // the page of the newest position
        if (newest && !waited) {     // written by the kernel before (or, fused, made of what it wrote)
          pdl_wait();
          waited = true;
        }
        constexpr int HALF = HD / 2;
        if (rotate && (i == 0 || newest)) {
          // the slot of the item's first stage gets the sines and cosines: it must be free
          if (i == 0 && it >= C::STAGES && lane == 0 &&
              !mbar_wait(empty_bar(s), ((it / C::STAGES) - 1) & 1, p.error_flag, 75))
            ok = false;
          ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
          if (!ok) break;
        }
        float sn[(HALF + 31) / 32], cs[(HALF + 31) / 32];
        if (rotate && (i == 0 || newest)) {
#pragma unroll
          for (int u = 0; u < (HALF + 31) / 32; ++u) {
            const int j = lane + 32 * u;
            if (j < HALF) {
              sincosf((float)d.pos * p.inv_freq[j], &sn[u], &cs[u]);
              if (i == 0) {
                rot_tab[s * HD + j] = sn[u];
                rot_tab[s * HD + HALF + j] = cs[u];
              }
            }
          }
          __syncwarp();      // lane 0's arrive on the stage's barrier below publishes the table
        }
        if (newest && p.fuse && p.write_kv) {
          const __nv_bfloat16* row = p.q + (size_t)d.tok * p.ldq;
          const __nv_bfloat16* ksrc = row + (size_t)(p.n_heads + d.kvh) * HD;
          const __nv_bfloat16* vsrc = row + (size_t)(p.n_heads + p.n_kv_heads + d.kvh) * HD;
          const size_t dst = (((size_t)pages[d.pos / DM_PAGE] * p.n_kv_heads + d.kvh) * DM_PAGE + (d.pos % DM_PAGE)) * HD;
#pragma unroll
          for (int u = 0; u < (HALF + 31) / 32; ++u) {
            const int j = lane + 32 * u;
            if (j < HALF) {
              if (rotate) {
                const float a = __bfloat162float(ksrc[j]), b = __bfloat162float(ksrc[j + HALF]);
                p.k_cache_w[dst + j] = __float2bfloat16_rn(rot_lo(a, b, cs[u], sn[u]));
                p.k_cache_w[dst + j + HALF] = __float2bfloat16_rn(rot_hi(a, b, cs[u], sn[u]));
              } else {
                p.k_cache_w[dst + j] = ksrc[j];
                p.k_cache_w[dst + j + HALF] = ksrc[j + HALF];
              }
              p.v_cache_w[dst + j] = vsrc[j];
              p.v_cache_w[dst + j + HALF] = vsrc[j + HALF];
            }
          }
          __threadfence();                                    // the copy below reads these rows through the async proxy
          asm volatile("fence.proxy.async;" ::: "memory");
          __syncwarp();
        }
        if (lane == 0) {
          if (it >= C::STAGES && !mbar_wait(empty_bar(s), ((it / C::STAGES) - 1) & 1, p.error_flag, 71)) ok = false;
          if (ok) {
            const int row = (pages[d.pg0 + i] * p.n_kv_heads + d.kvh) * DM_PAGE;
            mbar_expect_tx(full_bar(s), C::STAGE_BYTES);
#pragma unroll
            for (int u = 0; u < C::NSUB; ++u) {
              dm_tma(base + s * C::STAGE_BYTES + u * C::SUB_BYTES, &map_k, u * 64, row, full_bar(s));
              dm_tma(base + s * C::STAGE_BYTES + C::TILE_BYTES + u * C::SUB_BYTES, &map_v, u * 64, row, full_bar(s));
            }
          }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      }
    }
    return;
  }

  if (warp == DM_CONSUMERS + 1) {
    // ---- epilogue warp: items cut into several splits pass through here ----
    int n_split_items = 0;
    DmItem d;
    pdl_wait();
    for (int item = next_item(blockIdx.x, d); item < n_items; item = next_item(item + gridDim.x, d)) {
      if (d.n_parts == 1) continue;
      const int b = n_split_items & 1;
      if (!mbar_wait(rfull_bar(b), (n_split_items >> 1) & 1, p.error_flag, 73)) return;
      ++n_split_items;
      float* part = p.partials + ((((size_t)d.seq * p.n_kv_heads + d.kvh) * p.max_splits + d.part) * G) * (HD + 2);
      const float* rb = r_buf + (size_t)b * G * (HD + 2);
      for (int i = lane; i < G * (HD + 2); i += 32) part[i] = rb[i];
      __syncwarp();
      if (lane == 0) mbar_arrive(rempty_bar(b));      // the consumers may fill this buffer again
      __threadfence();
      __syncwarp();
      int last = 0;
      if (lane == 0) last = (atomicAdd(&p.tickets[d.seq * p.n_kv_heads + d.kvh], 1) == d.n_parts - 1);
      last = __shfl_sync(0xffffffffu, last, 0);
      if (!last) continue;
      __threadfence();
      // The final merge, in split order, two heads at a time.  The splits go by in chunks of NZ: lane z loads the
      // (max, sum) of the chunk's split z while every lane loads its dims of all NZ splits' values, so a chunk of
      // two heads costs one round trip to L2; running maximum and rescaling between chunks as in the main loop.
      const float* parts = p.partials + (((size_t)d.seq * p.n_kv_heads + d.kvh) * p.max_splits) * G * (HD + 2);
      constexpr int DPL = HD / 32;                // output dims per lane
      constexpr int NZ = DPL <= 2 ? 16 : 8;       // registers: 2 heads * NZ * DPL values
      for (int g0 = 0; g0 < G; g0 += 2) {
        float M[2] = {-INFINITY, -INFINITY}, L[2] = {0.f, 0.f}, A[2][DPL];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int u = 0; u < DPL; ++u) A[h][u] = 0.f;
        for (int z0 = 0; z0 < d.n_parts; z0 += NZ) {
          const int nz = min(NZ, d.n_parts - z0);
          float mz[2], lz[2], v[2][NZ][DPL];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int g = min(g0 + h, G - 1);
            const float* pl = parts + ((size_t)(z0 + min(lane, nz - 1)) * G + g) * (HD + 2);
            mz[h] = lane < nz ? __ldcg(&pl[HD]) : -INFINITY;
            lz[h] = lane < nz ? __ldcg(&pl[HD + 1]) : 0.f;
#pragma unroll
            for (int z = 0; z < NZ; ++z) {
              if (z < NZ / 2 || nz > NZ / 2) {      // (warp-uniform) the second half only when there are that many
                const float* pz = parts + ((size_t)(z0 + min(z, nz - 1)) * G + g) * (HD + 2);
#pragma unroll
                for (int u = 0; u < DPL; ++u) v[h][z][u] = __ldcg(&pz[lane + 32 * u]);
              } else {
#pragma unroll
                for (int u = 0; u < DPL; ++u) v[h][z][u] = 0.f;
              }
            }
          }
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const float Mc = fmaxf(M[h], warp_max(mz[h]));
            const float keep = (M[h] == -INFINITY) ? 0.f : fast_exp2(M[h] - Mc);
            M[h] = Mc;
            L[h] *= keep;
#pragma unroll
            for (int u = 0; u < DPL; ++u) A[h][u] *= keep;
            const float wl = (mz[h] == -INFINITY) ? 0.f : fast_exp2(mz[h] - Mc);
            const float ll = lz[h] * wl;
#pragma unroll
            for (int z = 0; z < NZ; ++z) {
              const float w = __shfl_sync(0xffffffffu, wl, z);      // 0 for the lanes past the chunk's splits
              L[h] += __shfl_sync(0xffffffffu, ll, z);
#pragma unroll
              for (int u = 0; u < DPL; ++u) A[h][u] = fmaf(w, v[h][z][u], A[h][u]);
            }
          }
        }
#pragma unroll
        for (int h = 0; h < 2; ++h)
          if (g0 + h < G) {
#pragma unroll
            for (int u = 0; u < DPL; ++u)
              p.out[(size_t)d.tok * p.ldo + (size_t)(d.kvh * G + g0 + h) * HD + lane + 32 * u] =
                  __float2bfloat16_rn(A[h][u] / L[h]);
          }
      }
      __syncwarp();
      if (lane == 0) p.tickets[d.seq * p.n_kv_heads + d.kvh] = 0;
    }
    return;
  }

  // ---- consumers: warp w takes keys 16w .. 16w+15 of every page; the group's heads are the MMA's rows ----
  const int gq = lane >> 2, t = lane & 3;                 // accumulator rows gq and gq + 8, columns 2t and 2t + 1
  const int ctid = threadIdx.x;                           // 0..127
  int it = 0, n_split_items = 0;
  bool ok = true;
  DmItem d;
  pdl_wait();   // q comes from the kernels before
  for (int item = next_item(blockIdx.x, d); item < n_items && ok; item = next_item(item + gridDim.x, d)) {
    uint32_t qa[HD / 16][4];
    float o[HD / 8][4];
#pragma unroll
    for (int dc = 0; dc < HD / 8; ++dc)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[dc][e] = 0.f;
    float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};     // maxima scaled, in base 2
    {
      // Q fragments (A operand) of the item, straight from global memory, on their way while the first page
      // arrives: rows = the group's heads.  With the fused rotation a thread holds both halves of every pair it
      // needs (dims d and d + HD/2 sit in k chunks HD/32 apart, same thread); the sines and cosines come from the
      // producer warp (slot of the item's first stage) with the first page.
      const __nv_bfloat16* q0 = p.q + (size_t)d.tok * p.ldq + (size_t)(d.kvh * G + gq) * HD;
      const __nv_bfloat16* q1 = q0 + (size_t)8 * HD;
      const bool v0 = gq < G, v1 = gq + 8 < G;
#pragma unroll
      for (int kc = 0; kc < HD / 16; ++kc) {
        qa[kc][0] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + kc * 16 + 2 * t) : 0u;
        qa[kc][1] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + kc * 16 + 2 * t) : 0u;
        qa[kc][2] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + kc * 16 + 8 + 2 * t) : 0u;
        qa[kc][3] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + kc * 16 + 8 + 2 * t) : 0u;
      }
    }
    for (int i = 0; i < d.n_pages; ++i, ++it) {
      const int s = it % C::STAGES;
      ok = mbar_wait(full_bar(s), (it / C::STAGES) & 1, p.error_flag, 72);
      if (!ok) break;
      if (i == 0) {
        if (rotate) {
          const float* tab = rot_tab + s * HD;
#pragma unroll
          for (int kc = 0; kc < HD / 32; ++kc) {           // chunks of the first half; partners HD/32 chunks on
#pragma unroll
            for (int e = 0; e < 4; ++e) {                   // e: (row gq | gq+8) x (columns 2t.. | 8+2t..)
              const int dim = kc * 16 + (e >> 1) * 8 + 2 * t;
              const float2 a = dm_unpack(qa[kc][e]), b = dm_unpack(qa[kc + HD / 32][e]);
              const float s0 = tab[dim], c0 = tab[HD / 2 + dim], s1 = tab[dim + 1], c1 = tab[HD / 2 + dim + 1];
              qa[kc][e] = dm_pack(rot_lo(a.x, b.x, c0, s0), rot_lo(a.y, b.y, c1, s1));
              qa[kc + HD / 32][e] = dm_pack(rot_hi(a.x, b.x, c0, s0), rot_hi(a.y, b.y, c1, s1));
            }
          }
        }
      }
      const uint32_t k_tile = base + s * C::STAGE_BYTES, v_tile = k_tile + C::TILE_BYTES;
      const int page_pos0 = (d.pg0 + i) * DM_PAGE;
      const bool inside = page_pos0 >= d.lo && page_pos0 + DM_PAGE - 1 <= d.pos;   // every key of the page counts
      if (!inside) {
        // value rows of keys that do not count are cleared: their zero probabilities must not meet a NaN
        for (int idx = lane; idx < 16 * (HD / 8); idx += 32) {
          const int row = warp * 16 + idx / (HD / 8), ch = idx % (HD / 8);
          const int kpos = page_pos0 + row;
          if (kpos < d.lo || kpos > d.pos)
            asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(v_tile + (ch / 8) * C::SUB_BYTES + (uint32_t)(row * 128 + ((ch & 7) << 4))), "r"(0u)
                         : "memory");
        }
        __syncwarp();
      }
      // S = Q Kᵀ: 16 heads x this warp's 16 keys
      float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int kc = 0; kc < HD / 16; ++kc) {
        const int mtx = lane >> 3, r = lane & 7;
        const int row = warp * 16 + (mtx >> 1) * 8 + r, kch = (kc % 4) * 2 + (mtx & 1);
        uint32_t b0, b1, b2, b3;
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                     : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3)
                     : "r"(k_tile + (kc / 4) * C::SUB_BYTES + (uint32_t)(row * 128 + ((kch ^ (row & 7)) << 4))));
        dm_mma(sc[0], qa[kc], b0, b1);
        dm_mma(sc[1], qa[kc], b2, b3);
      }
      if (!inside) {
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int kpos = page_pos0 + warp * 16 + n * 8 + 2 * t + (e & 1);
            if (kpos < d.lo || kpos > d.pos) sc[n][e] = -INFINITY;
          }
      }
      float mx0 = fmaxf(fmaxf(sc[0][0], sc[0][1]), fmaxf(sc[1][0], sc[1][1]));
      float mx1 = fmaxf(fmaxf(sc[0][2], sc[0][3]), fmaxf(sc[1][2], sc[1][3]));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(mrow[0], mx0 * p.scale_log2), mn1 = fmaxf(mrow[1], mx1 * p.scale_log2);
      const float c0 = (mn0 == -INFINITY) ? 1.f : fast_exp2(mrow[0] - mn0);
      const float c1 = (mn1 == -INFINITY) ? 1.f : fast_exp2(mrow[1] - mn1);
      mrow[0] = mn0;
      mrow[1] = mn1;
      if (__any_sync(0xffffffffu, c0 != 1.f || c1 != 1.f)) {
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
      uint32_t pa[4];
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        const float p0 = fast_exp2(fmaf(sc[n][0], p.scale_log2, nm0));   // 2^(-inf) = 0 for masked keys
        const float p1 = fast_exp2(fmaf(sc[n][1], p.scale_log2, nm0));
        const float p2 = fast_exp2(fmaf(sc[n][2], p.scale_log2, nm1));
        const float p3 = fast_exp2(fmaf(sc[n][3], p.scale_log2, nm1));
        lrow[0] += p0 + p1;
        lrow[1] += p2 + p3;
        pa[n * 2 + 0] = dm_pack(p0, p1);
        pa[n * 2 + 1] = dm_pack(p2, p3);
      }
      // O += P V: 16 heads x HD dims over this warp's 16 keys
#pragma unroll
      for (int dc = 0; dc < HD / 8; dc += 2) {
        const int mtx = lane >> 3, r = lane & 7;
        const int key = warp * 16 + (mtx & 1) * 8 + r;
        const int dchunk = dc + (mtx >> 1);
        uint32_t r0, r1, r2, r3;
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                     : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                     : "r"(v_tile + (dchunk / 8) * C::SUB_BYTES + (uint32_t)(key * 128 + (((dchunk & 7) ^ (key & 7)) << 4))));
        dm_mma(o[dc], pa, r0, r1);
        dm_mma(o[dc + 1], pa, r2, r3);
      }
      fence_reads_before_async_writes();
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_bar(s));
    }
    if (!ok) break;
    // this warp's (max, sum, values) per head to shared memory; the row sums first over the four threads of a row
    lrow[0] += __shfl_xor_sync(0xffffffffu, lrow[0], 1);
    lrow[0] += __shfl_xor_sync(0xffffffffu, lrow[0], 2);
    lrow[1] += __shfl_xor_sync(0xffffffffu, lrow[1], 1);
    lrow[1] += __shfl_xor_sync(0xffffffffu, lrow[1], 2);
    float* mine = s_warp + (size_t)warp * G * (HD + 2);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int row = gq + 8 * h;
      if (row < G) {
#pragma unroll
        for (int dc = 0; dc < HD / 8; ++dc) {
          mine[row * (HD + 2) + dc * 8 + 2 * t] = o[dc][2 * h];
          mine[row * (HD + 2) + dc * 8 + 2 * t + 1] = o[dc][2 * h + 1];
        }
        if (t == 0) {
          mine[row * (HD + 2) + HD] = mrow[h];
          mine[row * (HD + 2) + HD + 1] = lrow[h];
        }
      }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");   // the four consumer warps

    // merge the four consumer warps (fixed order); a whole sequence-head is written at once, a split goes to
    // the epilogue warp
    const int b = n_split_items & 1;
    if (d.n_parts > 1) {
      if (n_split_items >= 2) ok = mbar_wait(rempty_bar(b), ((n_split_items >> 1) - 1) & 1, p.error_flag, 74);
      if (!ok) break;
    }
    float* rb = r_buf + (size_t)b * G * (HD + 2);
    for (int idx = ctid; idx < G * HD; idx += DM_CONSUMERS * 32) {
      const int g = idx / HD, dd = idx - g * HD;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < DM_CONSUMERS; ++w) M = fmaxf(M, s_warp[((size_t)w * G + g) * (HD + 2) + HD]);
      float L = 0.f, A = 0.f;
#pragma unroll
      for (int w = 0; w < DM_CONSUMERS; ++w) {
        const float* sw = s_warp + ((size_t)w * G + g) * (HD + 2);
        const float f = (sw[HD] == -INFINITY) ? 0.f : fast_exp2(sw[HD] - M);
        L += sw[HD + 1] * f;
        A += sw[dd] * f;
      }
      if (d.n_parts == 1) {
        p.out[(size_t)d.tok * p.ldo + (size_t)(d.kvh * G + g) * HD + dd] = __float2bfloat16_rn(A / L);
      } else {
        rb[g * (HD + 2) + dd] = A;
        if (dd == 0) {
          rb[g * (HD + 2) + HD] = M;
          rb[g * (HD + 2) + HD + 1] = L;
        }
      }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");   // r_buf is complete; the warps' buffers are free again
    if (d.n_parts > 1) {
      if (ctid == 0) mbar_arrive(rfull_bar(b));
      ++n_split_items;
    }
  }
}

typedef CUresult (*DmEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The cache of one layer as a matrix [pages * kv_heads * 64 rows, head_dim]: tiles of [64 rows, 64 cols].
static int dm_cache_map(CUtensorMap* map, const void* ptr, long rows, int head_dim) {
  static DmEncodeFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return LLMI_ERR_DRIVER;
    fn = (DmEncodeFn)sym;
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

// Blocks of the kernel that are resident on the device at once for a group size (0: the launch cannot be set up).
template <int HD>
static int dm_resident(int group) {
  using C = DmCfg<HD>;
  struct PerGroup { int n[17] = {}; };
  static PerDevice<PerGroup> resident_on;
  int* resident = resident_on.here().n;
  static PerDevice<bool> configured_on;
  bool& configured = configured_on.here();
  if (!configured) {
    if (cudaFuncSetAttribute(attention_decode_mma_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             C::smem_bytes(16)) != cudaSuccess)
      return 0;
    configured = true;
  }
  if (!resident[group]) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attention_decode_mma_kernel<HD>, DM_THREADS,
                                                      C::smem_bytes(group)) != cudaSuccess || per_sm < 1)
      per_sm = 1;
    resident[group] = per_sm * sm_count();
  }
  return resident[group];
}

template <int HD>
static int dm_launch(const CUtensorMap& mk, const CUtensorMap& mv, const DecodeMmaParams& p, int n_seqs, cudaStream_t stream) {
  using C = DmCfg<HD>;
  const int resident = dm_resident<HD>(p.group);
  if (resident <= 0) return LLMI_ERR_LAUNCH;
  const long n_items = (long)n_seqs * p.n_kv_heads * p.max_splits;
  if (n_items > 0x7fffffffL) return LLMI_ERR_BAD_SIZE;
  const int grid = coprime_grid(n_items, resident, p.max_splits);
  return launch_pdl(PDL_ATTENTION, attention_decode_mma_kernel<HD>, grid, DM_THREADS, C::smem_bytes(p.group), stream, mk, mv,
                    p, (int)n_items);
}

}  // namespace llmi

using namespace llmi;

// 1 if the (head size, group size) pair has a compiled tensor-core decode kernel.
LLMI_EXPORT int llmi_attention_decode_mma_supported(int head_dim, int group) {
  return (head_dim == 64 || head_dim == 128) && group >= 1 && group <= 16;
}

// Blocks of the kernel that are resident on the device at once (0: no such kernel).
LLMI_EXPORT int llmi_attention_decode_mma_resident(int head_dim, int group) {
  if (!llmi_attention_decode_mma_supported(head_dim, group)) return 0;
  return head_dim == 64 ? dm_resident<64>(group) : dm_resident<128>(group);
}

// As llmi_attention_decode (fuse = 0: q rotated, cache complete) or llmi_attention_decode_fused (fuse = 1: `q` is the
// step's un-rotated [q | k | v] rows; rotary_dim is head_dim or 0), for any group size up to 16.  n_cache_pages: pages
// of the cache tensors (their first extent).  The workspace and the tickets are those of llmi_attention_decode.
LLMI_EXPORT int llmi_attention_decode_mma(const void* q, long ldq, void* out, long ldo, void* k_cache, void* v_cache,
                                          long n_cache_pages, const int32_t* seq_pages, int pages_stride,
                                          const int32_t* seq_kv_len, const int32_t* seq_q_start, int n_seqs, int n_heads,
                                          int n_kv_heads, int head_dim, float scale, int window, int max_pages,
                                          int pages_per_split, int fuse, const float* inv_freq, int rotary_dim,
                                          int write_kv, float* partials, long partials_floats, int* tickets, int n_tickets,
                                          int* error_flag, cudaStream_t stream) {
  if (n_seqs <= 0 || n_heads <= 0 || n_kv_heads <= 0 || max_pages <= 0 || pages_per_split <= 0 || n_cache_pages <= 0)
    return LLMI_ERR_BAD_SIZE;
  if (n_heads % n_kv_heads) return LLMI_ERR_BAD_SIZE;
  const int group = n_heads / n_kv_heads;
  if (!llmi_attention_decode_mma_supported(head_dim, group)) return LLMI_ERR_UNSUPPORTED;
  if (fuse && rotary_dim != 0 && (rotary_dim != head_dim || !inv_freq)) return LLMI_ERR_UNSUPPORTED;
  if (((uintptr_t)q & 15) || (ldq & 7) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15)) return LLMI_ERR_ALIGN;
  const int splits = (max_pages + pages_per_split - 1) / pages_per_split;
  if ((long)n_seqs * n_heads * splits * (head_dim + 2) > partials_floats || (long)n_seqs * n_kv_heads > n_tickets)
    return LLMI_ERR_BAD_SIZE;
  const long rows = n_cache_pages * n_kv_heads * DM_PAGE;
  if (rows > 0x7fffffffL) return LLMI_ERR_BAD_SIZE;
  CUtensorMap mk, mv;
  int rc = dm_cache_map(&mk, k_cache, rows, head_dim);
  if (rc != LLMI_OK) return rc;
  rc = dm_cache_map(&mv, v_cache, rows, head_dim);
  if (rc != LLMI_OK) return rc;
  DecodeMmaParams p{(const __nv_bfloat16*)q, ldq, (__nv_bfloat16*)out, ldo, seq_pages, seq_kv_len, seq_q_start, pages_stride,
                    n_kv_heads, group, scale * 1.4426950408889634f, window, pages_per_split, splits, partials, tickets,
                    error_flag, fuse ? 1 : 0, inv_freq, fuse ? rotary_dim : 0, n_heads, write_kv ? 1 : 0,
                    (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache};
  return head_dim == 64 ? dm_launch<64>(mk, mv, p, n_seqs, stream) : dm_launch<128>(mk, mv, p, n_seqs, stream);
}
