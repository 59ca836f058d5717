// Decode attention: one new token per sequence attends over its sequence's cache pages (bf16).
//
// Reference loop: src/model/transformer.cpp:263-282 with T = 1 (scores over s = 0..pos, softmax,
// weighted sum of values; kv head = query head / group).  A decode step reads every cached key and
// value exactly once and does a handful of FLOPs per byte, so the kernel is built around HBM:
//
//  * the cache keeps one (page, kv head) tile of 64 positions contiguous, so a tile of K or V is ONE
//    bulk copy (cp.async.bulk, 64*head_dim*2 bytes) into a ring of shared-memory stages, completed on
//    mbarriers; a producer warp keeps the ring full while four consumer warps compute;
//  * the positions of a sequence are cut into splits of `pages_per_split` pages (a function of
//    position only) and a block works on one (split, kv head, sequence); all `G` query heads that
//    share the kv head use the tile while it is in shared memory;
//  * the grid is persistent (as many blocks as fit on the device); a block walks through its items and
//    its copy ring runs on across items, so HBM stays busy while an item is merged and written;
//  * each item leaves (max, sum, weighted values) of its split in a workspace and takes a ticket;
//    the block that takes a sequence-head's last ticket merges the splits in split order and writes
//    the output.  Nothing waits for another block.
//
// Two other forms of the same kernel (template parameters): VP, with a second producer thread for the value tiles
// and a deeper ring, two blocks per SM, for steps whose sequence-heads about fill those blocks as whole items; and
// CL, launched as one cluster of 2, 4 or 8 blocks per sequence-head (one block per split) whose results meet in the
// first block's shared memory instead of the workspace, for few sequence-heads of few pages.  The host chooses
// (ops/kernels.py: decode_pages_per_split, decode_cluster); all forms give the same bits for the same split.
//
// Softmax runs in fp32 with a running maximum, in base 2 (scores are scaled by scale*log2(e) and the
// exponential is one ex2 instruction); the merge order is fixed, so a sequence's result does not depend
// on its batch-mates.  `window` > 0 keeps keys pos-window+1..pos.
//
// With `fuse` the kernel also does the step's position encoding (rope_store.cu's work for one token per
// sequence): one kernel less in a decode layer.  The arithmetic is rope_store.cu's, so are the bits.
//
// Launched as a programmatic dependent, the kernel starts while the kernels before it still run: of
// everything it reads, they write only q and the cache row of each sequence's newest position, so the
// producer fetches older pages at once and waits (griddepcontrol.wait) only before the newest page;
// the consumers wait before they read q.
#include <math.h>

#include "common.cuh"
#include "sm100.cuh"

namespace llmi {

constexpr int DEC_PAGE = 64;          // positions per cache page (the cache's page size)
constexpr int DEC_CONSUMERS = 4;      // consumer warps; each takes 16 keys of a page
constexpr int DEC_THREADS = (DEC_CONSUMERS + 2) * 32;   // + producer warp + epilogue warp
// The variant for few sequence-heads has one warp more, whose first lane asks for the value tiles (a thread is busy
// with a copy for about half a microsecond and its copies do not overlap: with two issuing threads a block streams
// fast enough for a sequence-head to need fewer splits, or none).  Seven warps of its 92 registers fit an SM twice,
// six warps of 72 three times: with more sequence-heads than two blocks per SM hold, three blocks with one
// producer each are the faster ones (measured, 32 kv heads of 64 at 4,096 positions, this variant against the
// other: batch 8 46.9 / 49.6 us, batch 24 to 48 3 to 10 % slower).
template <bool VP> struct DecThreads { static constexpr int value = DEC_THREADS + (VP ? 32 : 0); };

struct DecodeParams {
  const __nv_bfloat16* q;   // [tokens, >= n_heads*HD], row pitch ldq
  long ldq;
  __nv_bfloat16* out;       // [tokens, n_heads*HD], row pitch ldo
  long ldo;
  const __nv_bfloat16* k_cache;
  const __nv_bfloat16* v_cache;
  const int32_t* seq_pages;   // [n_seqs, pages_stride]
  const int32_t* seq_kv_len;  // [n_seqs] length after this step (0: padding)
  const int32_t* seq_q_start; // [n_seqs] row of the sequence's token
  int pages_stride;
  int n_kv_heads;
  float scale_log2;          // softmax scale * log2(e)
  int window;
  int pages_per_split;
  int max_splits;            // gridDim.x
  float* partials;           // [n_seqs, n_kv_heads, max_splits, G, HD + 2]
  int* tickets;              // [n_seqs * n_kv_heads], zero between launches
  int* error_flag;
  // Fused position encoding (optional: fuse == 0 leaves q and the cache as the caller prepared them).
  // q then points at the step's un-rotated [q | k | v] rows; the kernel rotates q as it reads it, and the
  // block that holds a sequence-head's newest page rotates the new k and appends it and the new v to that
  // page before it fetches the page.  rotary_dim is head_dim (whole-head rotate-half) or 0 (append only).
  int fuse;
  const float* inv_freq;     // [head_dim / 2] when rotary_dim > 0
  int rotary_dim;
  int n_heads;
  int write_kv;              // 0: the call reads a cache that another call has written
  __nv_bfloat16* k_cache_w;  // the same caches, writable
  __nv_bfloat16* v_cache_w;
};

// (VP: the variant with a second producer thread; registers leave it two blocks per SM, so its ring may be deeper)
template <int HD, bool VP = false>
struct DecCfg {
  static constexpr int TILE_BYTES = DEC_PAGE * HD * 2;
  static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  static constexpr int STAGES = (VP && HD <= 64) ? 6 : (HD <= 128 ? 4 : 3);
  static constexpr int LPR = HD / 8;          // lanes per key row (16 bytes each)
  static constexpr int RPI = 32 / LPR;        // rows per warp instruction
  static constexpr int NI = 16 / RPI;         // instructions per warp per page (16 keys per warp)
  static constexpr int BAR_BYTES = 8 * (2 * STAGES + 4) + 32;
  static constexpr int ROT_BYTES = STAGES * HD * 4;       // per stage: sin[HD/2], cos[HD/2] of the item that starts there
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 128 /*align*/ + BAR_BYTES + ROT_BYTES;
};

__device__ __forceinline__ void bf16x8_to_f32(const uint4& raw, float* f) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 v = __bfloat1622float2(p[e]);
    f[2 * e] = v.x;
    f[2 * e + 1] = v.y;
  }
}

constexpr int DEC_MAX_CLUSTER = 8;

struct DecItem {
  int seq, kvh, part, n_parts, lo, pos, pg0, n_pages, tok;
};

// Work is cut into items (sequence, kv head, split).  The grid is persistent: block b takes items
// b, b + gridDim.x, ... and its ring of stages runs on across item borders.  Four consumer warps
// share an item's pages (16 keys of a page each); a producer warp keeps the ring full; an epilogue
// warp takes a finished item's merged (max, sum, values) from shared memory and does the slow,
// latency-bound part — partial to the workspace, fence, ticket, and the final merge if it drew the
// last ticket — while the consumers are already on the next item.
//
// CL: the kernel is launched as clusters of p.max_splits blocks (2, 4 or 8), one block per item and one cluster
// per sequence-head, all resident at once.  A block sends its split's (values, maximum, sum) into the shared memory
// of the cluster's first block, which adds them in split order and writes the head's output: no partial results
// in global memory, no fence, no ticket, no round trips to L2 behind the last page.  For few sequence-heads, where
// the kernel is as long as that chain, not as its bytes (batch 1, 4,096 positions: 10 us for 33 MB).
template <int HD, int G, bool VP, bool CL = false>
__global__ void __launch_bounds__(DecThreads<VP>::value)
attention_decode_kernel(DecodeParams p, int n_items) {
  using C = DecCfg<HD, VP>;
  static_assert(C::LPR >= 2 && C::LPR <= 32 && C::NI >= 1, "head size not supported by this layout");
  static_assert(!(VP && CL), "the cluster form has one producer thread");
  extern __shared__ uint8_t smem_raw[];
  __shared__ float s_m[DEC_CONSUMERS][G], s_l[DEC_CONSUMERS][G];
  __shared__ float s_acc[DEC_CONSUMERS][G][HD];
  __shared__ float r_buf[2][G][HD + 2];     // merged results on their way to the epilogue warp
  __shared__ float cl_recv[CL ? DEC_MAX_CLUSTER : 1][CL ? G : 1][CL ? HD + 2 : 1];   // first block of a cluster: the splits' results
  __shared__ __align__(8) uint64_t cl_bar_word;
  const uint32_t cl_bar = smem_u32(&cl_bar_word);

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t base = (smem_u32(smem_raw) + 127u) & ~127u;
  const uint32_t bars = base + C::STAGES * C::STAGE_BYTES;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (C::STAGES + s); };
  auto rfull_bar = [&](int b) { return bars + 8u * (2 * C::STAGES + b); };
  auto rempty_bar = [&](int b) { return bars + 8u * (2 * C::STAGES + 2 + b); };
  float* rot_tab = reinterpret_cast<float*>(smem_raw + (base - smem_u32(smem_raw)) + C::STAGES * C::STAGE_BYTES + C::BAR_BYTES);
  const bool rotate = p.fuse && p.rotary_dim > 0;
  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), DEC_CONSUMERS);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(rfull_bar(b), 1);
      mbar_init(rempty_bar(b), 1);
    }
    if (CL) mbar_init(cl_bar, cluster_size());     // every block of the cluster arrives once, the first included
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (CL) cluster_sync_all();     // nobody arrives on the first block's barrier before it is set up

  // The first non-empty item at or after `item` in this block's sequence of items (stride gridDim.x);
  // returns n_items when there is none.  Every warp role walks the same sequence.
  auto next_item = [&](int item, DecItem& d) -> int {
    for (; item < n_items; item += gridDim.x) {
      const int split = item % p.max_splits;
      const int sh = item / p.max_splits;
      d.kvh = sh % p.n_kv_heads;
      d.seq = sh / p.n_kv_heads;
      const int kv_len = p.seq_kv_len[d.seq];
      if (kv_len <= 0) continue;                                   // padding sequence
      d.pos = kv_len - 1;
      d.lo = (p.window > 0 && kv_len - p.window > 0) ? kv_len - p.window : 0;
      const int first_page = d.lo / DEC_PAGE, last_page = d.pos / DEC_PAGE;
      const int first_split = first_page / p.pages_per_split, last_split = last_page / p.pages_per_split;
      if (split < first_split || split > last_split) continue;     // nothing of the sequence in this split
      d.part = split - first_split;
      d.n_parts = last_split - first_split + 1;
      d.pg0 = max(first_page, split * p.pages_per_split);
      d.n_pages = min(last_page + 1, (split + 1) * p.pages_per_split) - d.pg0;
      d.tok = p.seq_q_start[d.seq];
      return item;
    }
    return n_items;
  };

  if (warp == DEC_CONSUMERS) {
    // ---- producer (lane 0 issues the copies; the whole warp appends a sequence-head's new k and v) ----
    int it = 0;
    DecItem d;
    bool ok = true, waited = false;
    for (int item = next_item(blockIdx.x, d); item < n_items && ok; item = next_item(item + gridDim.x, d)) {
      const int32_t* pages = p.seq_pages + (size_t)d.seq * p.pages_stride;
      for (int i = 0; i < d.n_pages && ok; ++i, ++it) {
        const int s = it % C::STAGES;
        const bool newest = (d.pg0 + i + 1) * DEC_PAGE > d.pos;   // the page of the newest position
        if (newest && !waited) {     // written by the kernel before (or, fused, made of what it wrote)
          pdl_wait();
          waited = true;
        }
        constexpr int HALF = HD / 2;
        if (rotate && (i == 0 || newest)) {
          // sines and cosines of this sequence's position: for the consumers (q), left in the slot of the
          // item's first stage, and for the new key below.  The slot is free: its stage's last reader released it.
          if (i == 0 && it >= C::STAGES && lane == 0 &&
              !mbar_wait(empty_bar(s), ((it / C::STAGES) - 1) & 1, p.error_flag, 15))
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
          const size_t dst = (((size_t)pages[d.pos / DEC_PAGE] * p.n_kv_heads + d.kvh) * DEC_PAGE + (d.pos % DEC_PAGE)) * HD;
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
          // the bulk copy below reads these rows through the async proxy
          __threadfence();
          asm volatile("fence.proxy.async;" ::: "memory");
          __syncwarp();
        }
        if (lane == 0) {
          if (it >= C::STAGES && !mbar_wait(empty_bar(s), ((it / C::STAGES) - 1) & 1, p.error_flag, 11)) ok = false;
          if (ok) {
            const size_t tile = ((size_t)pages[d.pg0 + i] * p.n_kv_heads + d.kvh) * (size_t)(DEC_PAGE * HD);
            mbar_expect_tx(full_bar(s), C::STAGE_BYTES);
            bulk_load(base + s * C::STAGE_BYTES, p.k_cache + tile, C::TILE_BYTES, full_bar(s));
            // (with the value tiles' own producer, only the newest page's value tile is asked for here)
            if (!VP || newest) bulk_load(base + s * C::STAGE_BYTES + C::TILE_BYTES, p.v_cache + tile, C::TILE_BYTES, full_bar(s));
          }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      }
    }
    return;
  }

  if (VP && warp == DEC_CONSUMERS + 2) {
    // ---- the value tiles' producer: the same walk over items and stages, the value tile of every page but a
    // sequence-head's newest one (that page is written in this step: its tiles follow the producer warp's wait and
    // append).  A stage's full barrier is in its new phase once its empty barrier has completed, so these bytes
    // count for the right phase even when they land before the producer warp has announced the stage.
    if (lane == 0) {
      int it = 0;
      DecItem d;
      bool ok = true;
      for (int item = next_item(blockIdx.x, d); item < n_items && ok; item = next_item(item + gridDim.x, d)) {
        const int32_t* pages = p.seq_pages + (size_t)d.seq * p.pages_stride;
        for (int i = 0; i < d.n_pages; ++i, ++it) {
          if ((d.pg0 + i + 1) * DEC_PAGE > d.pos) continue;          // the newest page
          const int s = it % C::STAGES;
          if (it >= C::STAGES && !mbar_wait(empty_bar(s), ((it / C::STAGES) - 1) & 1, p.error_flag, 16)) { ok = false; break; }
          const size_t tile = ((size_t)pages[d.pg0 + i] * p.n_kv_heads + d.kvh) * (size_t)(DEC_PAGE * HD);
          bulk_load(base + s * C::STAGE_BYTES + C::TILE_BYTES, p.v_cache + tile, C::TILE_BYTES, full_bar(s));
        }
      }
    }
    return;
  }

  if (warp == DEC_CONSUMERS + 1) {
    // ---- epilogue warp: items cut into several splits pass through here ----
    if (CL) return;               // (a cluster's results meet in its first block's shared memory instead)
    int n_split_items = 0;
    DecItem d;
    pdl_wait();
    for (int item = next_item(blockIdx.x, d); item < n_items; item = next_item(item + gridDim.x, d)) {
      if (d.n_parts == 1) continue;
      const int b = n_split_items & 1;
      if (!mbar_wait(rfull_bar(b), (n_split_items >> 1) & 1, p.error_flag, 13)) return;
      ++n_split_items;
      float* part = p.partials + ((((size_t)d.seq * p.n_kv_heads + d.kvh) * p.max_splits + d.part) * G) * (HD + 2);
      for (int i = lane; i < G * (HD + 2); i += 32) part[i] = (&r_buf[b][0][0])[i];
      __syncwarp();
      if (lane == 0) mbar_arrive(rempty_bar(b));      // the consumers may fill this buffer again
      __threadfence();
      __syncwarp();
      int last = 0;
      if (lane == 0) last = (atomicAdd(&p.tickets[d.seq * p.n_kv_heads + d.kvh], 1) == d.n_parts - 1);
      last = __shfl_sync(0xffffffffu, last, 0);
      if (!last) continue;
      __threadfence();
      // The final merge, in split order.  Lane z holds split z's (max, sum); the weights go round by
      // shuffle, and the values of four splits are loaded together, so the merge costs a few round
      // trips to L2 rather than one per split.
      const float* parts = p.partials + (((size_t)d.seq * p.n_kv_heads + d.kvh) * p.max_splits) * G * (HD + 2);
      constexpr int DPL = (HD + 31) / 32;   // output dims per lane
      for (int g = 0; g < G; ++g) {
        float L = 0.f, A[DPL];
#pragma unroll
        for (int u = 0; u < DPL; ++u) A[u] = 0.f;
        constexpr int NZ = DPL <= 2 ? 16 : 8;      // splits merged in one go (registers: NZ * DPL values)
        if (d.n_parts <= NZ) {
          // few splits: every load of the merge is issued before any is used — one round trip to L2
          float mz[NZ], lz[NZ], v[NZ][DPL];
#pragma unroll
          for (int z = 0; z < NZ; ++z) {
            if (z < 8 || d.n_parts > 8) {        // (warp-uniform) the second eight only when there are that many
              const float* pz = parts + ((size_t)min(z, d.n_parts - 1) * G + g) * (HD + 2);
              mz[z] = __ldcg(&pz[HD]);
              lz[z] = __ldcg(&pz[HD + 1]);
#pragma unroll
              for (int u = 0; u < DPL; ++u) v[z][u] = (lane + 32 * u < HD) ? __ldcg(&pz[lane + 32 * u]) : 0.f;
            } else {
              mz[z] = -INFINITY;
              lz[z] = 0.f;
#pragma unroll
              for (int u = 0; u < DPL; ++u) v[z][u] = 0.f;
            }
          }
          float M = -INFINITY;
#pragma unroll
          for (int z = 0; z < NZ; ++z)
            if (z < d.n_parts) M = fmaxf(M, mz[z]);
#pragma unroll
          for (int z = 0; z < NZ; ++z) {
            const float w = (z < d.n_parts && mz[z] != -INFINITY) ? fast_exp2(mz[z] - M) : 0.f;
            L = fmaf(lz[z], w, L);
#pragma unroll
            for (int u = 0; u < DPL; ++u) A[u] = fmaf(w, v[z][u], A[u]);
          }
        } else {
          float M = -INFINITY;
          for (int z = lane; z < d.n_parts; z += 32) M = fmaxf(M, __ldcg(&parts[((size_t)z * G + g) * (HD + 2) + HD]));
          M = warp_max(M);
          for (int z0 = 0; z0 < d.n_parts; z0 += 32) {
            const int z = z0 + lane;
            float wz = 0.f, lw = 0.f;
            if (z < d.n_parts) {
              const float* pz = parts + ((size_t)z * G + g) * (HD + 2);
              const float mz = __ldcg(&pz[HD]);
              wz = (mz == -INFINITY) ? 0.f : fast_exp2(mz - M);
              lw = __ldcg(&pz[HD + 1]) * wz;
            }
            const int nz = min(32, d.n_parts - z0);
            for (int j0 = 0; j0 < nz; j0 += 4) {
              float v[4][DPL];
#pragma unroll
              for (int jj = 0; jj < 4; ++jj) {
                const float* pj = parts + ((size_t)(z0 + min(j0 + jj, nz - 1)) * G + g) * (HD + 2);
#pragma unroll
                for (int u = 0; u < DPL; ++u) v[jj][u] = (lane + 32 * u < HD) ? __ldcg(&pj[lane + 32 * u]) : 0.f;
              }
#pragma unroll
              for (int jj = 0; jj < 4; ++jj) {
                const int j = min(j0 + jj, nz - 1);
                const float w = (j0 + jj < nz) ? __shfl_sync(0xffffffffu, wz, j) : 0.f;
                L += (j0 + jj < nz) ? __shfl_sync(0xffffffffu, lw, j) : 0.f;
#pragma unroll
                for (int u = 0; u < DPL; ++u) A[u] = fmaf(w, v[jj][u], A[u]);
              }
            }
          }
        }
#pragma unroll
        for (int u = 0; u < DPL; ++u)
          if (lane + 32 * u < HD)
            p.out[(size_t)d.tok * p.ldo + (size_t)(d.kvh * G + g) * HD + lane + 32 * u] = __float2bfloat16_rn(A[u] / L);
      }
      __syncwarp();
      if (lane == 0) p.tickets[d.seq * p.n_kv_heads + d.kvh] = 0;
    }
    return;
  }

  // ---- consumers: lane = (row group r, 16-byte chunk c) of a key row ----
  const int c = lane % C::LPR, r = lane / C::LPR;
  const int ctid = threadIdx.x;   // 0..127
  int it = 0, n_split_items = 0;
  bool ok = true, sent = false;
  DecItem d, dn;
  int item = next_item(blockIdx.x, d);
  uint4 q_raw[G], q_next[G];
  constexpr int HALF_CHUNKS = C::LPR / 2;
  pdl_wait();   // q comes from the kernels before
  if (item < n_items) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const __nv_bfloat16* qh = p.q + (size_t)d.tok * p.ldq + (size_t)(d.kvh * G + g) * HD;
      q_raw[g] = *reinterpret_cast<const uint4*>(qh + c * 8);
    }
  }
  while (item < n_items && ok) {
    const int item_next = next_item(item + gridDim.x, dn);
    if (item_next < n_items) {     // the next item's q is fetched while this item's pages are worked on
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const __nv_bfloat16* qh = p.q + (size_t)dn.tok * p.ldq + (size_t)(dn.kvh * G + g) * HD;
        q_next[g] = *reinterpret_cast<const uint4*>(qh + c * 8);
      }
    }
    float q[G][8];
    float m[G], l[G], acc[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      m[g] = -INFINITY;
      l[g] = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[g][e] = 0.f;
    }
    for (int i = 0; i < d.n_pages; ++i, ++it) {
      const int s = it % C::STAGES;
      ok = mbar_wait(full_bar(s), (it / C::STAGES) & 1, p.error_flag, 12);
      if (!ok) break;
      if (i == 0) {
#pragma unroll
        for (int g = 0; g < G; ++g) bf16x8_to_f32(q_raw[g], q[g]);
        if (rotate) {
          // rotate-half on this lane's 8 dims: (a, b) = (first-half value, second-half value) of each pair; the
          // partner chunk in the other half of the head is held by the lane HALF_CHUNKS away; sines and cosines
          // come from the producer warp (in the slot of this first stage); the result is rounded to bf16 as
          // the separate kernel would have stored it
          const float* tab = rot_tab + s * HD + (c % HALF_CHUNKS) * 8;
#pragma unroll
          for (int g = 0; g < G; ++g) {
            uint4 pair;
            pair.x = __shfl_xor_sync(0xffffffffu, q_raw[g].x, HALF_CHUNKS);
            pair.y = __shfl_xor_sync(0xffffffffu, q_raw[g].y, HALF_CHUNKS);
            pair.z = __shfl_xor_sync(0xffffffffu, q_raw[g].z, HALF_CHUNKS);
            pair.w = __shfl_xor_sync(0xffffffffu, q_raw[g].w, HALF_CHUNKS);
            float other[8];
            bf16x8_to_f32(pair, other);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const float sn = tab[e], cs = tab[HD / 2 + e];
              const float r = c < HALF_CHUNKS ? rot_lo(q[g][e], other[e], cs, sn) : rot_hi(other[e], q[g][e], cs, sn);
              q[g][e] = __bfloat162float(__float2bfloat16_rn(r));
            }
          }
        }
      }
      const uint32_t k_tile = base + s * C::STAGE_BYTES, v_tile = k_tile + C::TILE_BYTES;
      const int page_pos0 = (d.pg0 + i) * DEC_PAGE;
      const bool inside = page_pos0 >= d.lo && page_pos0 + DEC_PAGE - 1 <= d.pos;   // every key of the page counts
      float sc[C::NI][G];
      float pmax[G];
#pragma unroll
      for (int g = 0; g < G; ++g) pmax[g] = -INFINITY;
#pragma unroll
      for (int j = 0; j < C::NI; ++j) {
        const int row = warp * 16 + j * C::RPI + r;
        uint4 raw;
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(raw.x), "=r"(raw.y), "=r"(raw.z), "=r"(raw.w)
                     : "r"(k_tile + (uint32_t)(row * HD + c * 8) * 2));
        float kf[8];
        bf16x8_to_f32(raw, kf);
        const int kpos = page_pos0 + row;
        const bool valid = inside || (kpos >= d.lo && kpos <= d.pos);
#pragma unroll
        for (int g = 0; g < G; ++g) {
          float dot = 0.f;
#pragma unroll
          for (int e = 0; e < 8; ++e) dot = fmaf(q[g][e], kf[e], dot);
#pragma unroll
          for (int o = 1; o < C::LPR; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
          sc[j][g] = valid ? dot * p.scale_log2 : -INFINITY;
          pmax[g] = fmaxf(pmax[g], sc[j][g]);
        }
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
#pragma unroll
        for (int o = C::LPR; o < 32; o <<= 1) pmax[g] = fmaxf(pmax[g], __shfl_xor_sync(0xffffffffu, pmax[g], o));
        const float m_new = fmaxf(m[g], pmax[g]);
        if (m_new != m[g]) {             // warp-uniform: every lane holds the same maxima
          const float corr = fast_exp2(m[g] - m_new);     // 2^(-inf) = 0 on the first page
          m[g] = m_new;
          l[g] *= corr;
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[g][e] *= corr;
        }
      }
#pragma unroll
      for (int j = 0; j < C::NI; ++j) {
        const int row = warp * 16 + j * C::RPI + r;
        uint4 raw;
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(raw.x), "=r"(raw.y), "=r"(raw.z), "=r"(raw.w)
                     : "r"(v_tile + (uint32_t)(row * HD + c * 8) * 2));
        float vf[8];
        bf16x8_to_f32(raw, vf);
        if (!inside) {
          const int kpos = page_pos0 + row;
          if (kpos < d.lo || kpos > d.pos) {   // whatever lies outside the sequence's positions counts as zero
#pragma unroll
            for (int e = 0; e < 8; ++e) vf[e] = 0.f;
          }
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float pr = (m[g] == -INFINITY) ? 0.f : fast_exp2(sc[j][g] - m[g]);   // masked keys: 2^(-inf) = 0
          l[g] += pr;
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[g][e] = fmaf(pr, vf[e], acc[g][e]);
        }
      }
      fence_reads_before_async_writes();
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_bar(s));
    }
    if (!ok) break;
    // fold the row groups of the warp: lanes with the same chunk c hold the same totals afterwards
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
      for (int o = C::LPR; o < 32; o <<= 1) {
        l[g] += __shfl_xor_sync(0xffffffffu, l[g], o);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[g][e] += __shfl_xor_sync(0xffffffffu, acc[g][e], o);
      }
      if (r == 0) {
#pragma unroll
        for (int e = 0; e < 8; ++e) s_acc[warp][g][c * 8 + e] = acc[g][e];
        if (c == 0) {
          s_m[warp][g] = m[g];
          s_l[warp][g] = l[g];
        }
      }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");   // the four consumer warps

    // merge the four consumer warps (fixed order); a whole sequence-head is written at once, a split
    // goes to the epilogue warp
    const int b = n_split_items & 1;
    if (!CL && d.n_parts > 1) {
      if (n_split_items >= 2) ok = mbar_wait(rempty_bar(b), ((n_split_items >> 1) - 1) & 1, p.error_flag, 14);
      if (!ok) break;
    }
    for (int idx = ctid; idx < G * HD; idx += DEC_CONSUMERS * 32) {
      const int g = idx / HD, dd = idx - g * HD;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < DEC_CONSUMERS; ++w) M = fmaxf(M, s_m[w][g]);
      float L = 0.f, A = 0.f;
#pragma unroll
      for (int w = 0; w < DEC_CONSUMERS; ++w) {
        const float f = (s_m[w][g] == -INFINITY) ? 0.f : fast_exp2(s_m[w][g] - M);
        L += s_l[w][g] * f;
        A += s_acc[w][g][dd] * f;
      }
      if (CL) {
        // to the cluster's first block, into the row of this block's rank
        const uint32_t dst = map_to_rank(smem_u32(&cl_recv[cluster_rank()][g][0]), 0);
        st_cluster_f32(dst + 4u * dd, A);
        if (dd == 0) {
          st_cluster_f32(dst + 4u * HD, M);
          st_cluster_f32(dst + 4u * (HD + 1), L);
        }
      } else if (d.n_parts == 1) {
        p.out[(size_t)d.tok * p.ldo + (size_t)(d.kvh * G + g) * HD + dd] = __float2bfloat16_rn(A / L);
      } else {
        r_buf[b][g][dd] = A;
        if (dd == 0) {
          r_buf[b][g][HD] = M;
          r_buf[b][g][HD + 1] = L;
        }
      }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");   // r_buf is complete; s_m / s_acc are free again
    if (CL) {
      sent = true;
    } else if (d.n_parts > 1) {
      if (ctid == 0) mbar_arrive(rfull_bar(b));
      ++n_split_items;
    }
    item = item_next;
    d = dn;
#pragma unroll
    for (int g = 0; g < G; ++g) q_raw[g] = q_next[g];
  }
  if (CL) {
    // One item a block.  A block whose split holds nothing of its sequence (or whose sequence is padding, or whose
    // wait gave up) sends an empty result, so that the first block always hears from the whole cluster.
    const uint32_t rank = cluster_rank(), n_ranks = cluster_size();
    if (!sent) {
      const uint32_t dst = map_to_rank(smem_u32(&cl_recv[rank][0][0]), 0);
      for (int idx = ctid; idx < G * (HD + 2); idx += DEC_CONSUMERS * 32) {
        const int dd = idx % (HD + 2);
        st_cluster_f32(dst + 4u * idx, dd == HD ? -INFINITY : 0.f);
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    if (ctid == 0) mbar_arrive_remote(map_to_rank(cl_bar, 0));   // (after the bar.sync: the block's stores come first)
    if (rank != 0) return;
    if (!mbar_wait_cluster(cl_bar, 0, p.error_flag, 17)) return;
    // the sequence-head of this cluster (the first block's own split may be empty: not from `d`)
    const int sh = blockIdx.x / p.max_splits;
    const int kvh = sh % p.n_kv_heads, seq = sh / p.n_kv_heads;
    if (p.seq_kv_len[seq] <= 0) return;                            // padding sequence
    const int tok = p.seq_q_start[seq];
    for (int idx = ctid; idx < G * HD; idx += DEC_CONSUMERS * 32) {
      const int g = idx / HD, dd = idx - g * HD;
      float M = -INFINITY;
      for (uint32_t z = 0; z < n_ranks; ++z) M = fmaxf(M, cl_recv[z][g][HD]);
      float L = 0.f, A = 0.f;
      for (uint32_t z = 0; z < n_ranks; ++z) {                     // in split order
        const float mz = cl_recv[z][g][HD];
        const float w = (mz == -INFINITY) ? 0.f : fast_exp2(mz - M);
        L = fmaf(cl_recv[z][g][HD + 1], w, L);
        A = fmaf(w, cl_recv[z][g][dd], A);
      }
      p.out[(size_t)tok * p.ldo + (size_t)(kvh * G + g) * HD + dd] = __float2bfloat16_rn(A / L);
    }
  }
}

// Blocks of this kernel that fit on the device at once.
template <int HD, int G, bool VP = false>
int decode_resident() {
  using C = DecCfg<HD, VP>;
  static PerDevice<int> resident_on;
  int& resident = resident_on.here();
  if (!resident) {
    cudaFuncSetAttribute(attention_decode_kernel<HD, G, VP>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attention_decode_kernel<HD, G, VP>, DecThreads<VP>::value,
                                                      C::SMEM_BYTES) != cudaSuccess || per_sm < 1)
      per_sm = 1;
    resident = per_sm * sm_count();
  }
  return resident;
}

template <int HD, int G, bool VP>
int launch_decode_variant(const DecodeParams& p, int n_seqs, cudaStream_t stream) {
  using C = DecCfg<HD, VP>;
  static PerDevice<bool> configured_on;
  bool& configured = configured_on.here();
  if (!configured) {
    if (cudaFuncSetAttribute(attention_decode_kernel<HD, G, VP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             C::SMEM_BYTES) != cudaSuccess)
      return LLMI_ERR_LAUNCH;
    configured = true;
  }
  const long n_items = (long)n_seqs * p.n_kv_heads * p.max_splits;
  if (n_items > 0x7fffffffL) return LLMI_ERR_BAD_SIZE;
  const int resident = decode_resident<HD, G, VP>();
  const int grid = coprime_grid(n_items, resident, p.max_splits);
  return launch_pdl(PDL_ATTENTION, attention_decode_kernel<HD, G, VP>, grid, DecThreads<VP>::value, C::SMEM_BYTES, stream, p,
                    (int)n_items);
}

// The cluster form: clusters of `cluster` blocks, one block per item.
template <int HD>
int launch_decode_cluster(const DecodeParams& p, int n_seqs, int cluster, cudaStream_t stream) {
  using C = DecCfg<HD, false>;
  static PerDevice<bool> configured_on;
  bool& configured = configured_on.here();
  if (!configured) {
    if (cudaFuncSetAttribute(attention_decode_kernel<HD, 1, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             C::SMEM_BYTES) != cudaSuccess)
      return LLMI_ERR_LAUNCH;
    configured = true;
  }
  const long n_items = (long)n_seqs * p.n_kv_heads * cluster;
  if (n_items > 0x7fffffffL) return LLMI_ERR_BAD_SIZE;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)n_items);
  cfg.blockDim = dim3(DecThreads<false>::value);
  cfg.dynamicSmemBytes = C::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = pdl_enabled(PDL_ATTENTION) ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return cudaLaunchKernelEx(&cfg, attention_decode_kernel<HD, 1, false, true>, p, (int)n_items) == cudaSuccess ? LLMI_OK
                                                                                                              : LLMI_ERR_LAUNCH;
}

// How many clusters of `cluster` blocks of the cluster form the device holds at once (0: none, or no such kernel).
template <int HD>
int decode_clusters_resident(int cluster) {
  using C = DecCfg<HD, false>;
  cudaFuncSetAttribute(attention_decode_kernel<HD, 1, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(cluster * 1024));
  cfg.blockDim = dim3(DecThreads<false>::value);
  cfg.dynamicSmemBytes = C::SMEM_BYTES;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, attention_decode_kernel<HD, 1, false, true>, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

// The variant with a producer of its own for the value tiles: ungrouped queries (the grouped ones have the tensor-core
// kernel) and between half as many and as many sequence-heads as its blocks hold at once.
template <int HD, int G>
bool decode_two_producers(int n_seqs, int n_kv_heads) {
  if (G != 1) return false;
  static int enabled = -1;
  if (enabled < 0) {
    const char* e = getenv("LLMI_DECODE_VALUE_PRODUCER");
    enabled = (e && e[0] == '0') ? 0 : 1;
  }
  // (with fewer than half as many sequence-heads as blocks the items are short either way, and the other variant's
  // third block per SM counts for more: batch 4 of 32 kv heads 1.397 against 1.415 ms a step)
  const long pairs = (long)n_seqs * n_kv_heads, resident = decode_resident<HD, 1, true>();
  return enabled && pairs <= resident && 2 * pairs >= resident;
}

template <int HD, int G>
int launch_decode(const DecodeParams& p, int n_seqs, int n_live, int cluster, cudaStream_t stream) {
  if (cluster) {
    // (the clusters' blocks number the splits: those beyond the page tables' width find nothing to do)
    if (G != 1 || (cluster != 2 && cluster != 4 && cluster != 8) || p.max_splits > cluster) return LLMI_ERR_BAD_SIZE;
    DecodeParams q = p;
    q.max_splits = cluster;
    return launch_decode_cluster<HD>(q, n_seqs, cluster, stream);
  }
  // (n_live: how many of the n_seqs sequences are not padding, when the caller knows; it decides the variant only)
  if (G == 1 && decode_two_producers<HD, G>(n_live > 0 && n_live < n_seqs ? n_live : n_seqs, p.n_kv_heads))
    return launch_decode_variant<HD, 1, true>(p, n_seqs, stream);
  return launch_decode_variant<HD, G, false>(p, n_seqs, stream);
}

static int dispatch_decode(const DecodeParams& p, int n_seqs, int n_live, int cluster, int head_dim, int group,
                           cudaStream_t stream) {
#define LLMI_DEC(HD, G) \
  if (head_dim == HD && group == G) return launch_decode<HD, G>(p, n_seqs, n_live, cluster, stream)
  LLMI_DEC(64, 1); LLMI_DEC(64, 2); LLMI_DEC(64, 3); LLMI_DEC(64, 4); LLMI_DEC(64, 8);
  LLMI_DEC(128, 1); LLMI_DEC(128, 2); LLMI_DEC(128, 3); LLMI_DEC(128, 4); LLMI_DEC(128, 8);
  LLMI_DEC(32, 1); LLMI_DEC(32, 2); LLMI_DEC(32, 4);
#undef LLMI_DEC
  return LLMI_ERR_UNSUPPORTED;
}

}  // namespace llmi

using namespace llmi;

// 1 if the (head size, group size) pair has a compiled decode kernel.
LLMI_EXPORT int llmi_attention_decode_supported(int head_dim, int group) {
  if (head_dim == 64 || head_dim == 128) return group == 1 || group == 2 || group == 3 || group == 4 || group == 8;
  if (head_dim == 32) return group == 1 || group == 2 || group == 4;
  return 0;
}

// Blocks of the (head size, group) kernel that are resident on the device at once (0: no such kernel).
LLMI_EXPORT int llmi_attention_decode_resident(int head_dim, int group);

// Floats of workspace for n_seqs sequences of at most max_pages pages each.
LLMI_EXPORT long llmi_attention_decode_workspace(int n_seqs, int n_heads, int head_dim, int max_pages,
                                                 int pages_per_split) {
  const long splits = (max_pages + pages_per_split - 1) / pages_per_split;
  return (long)n_seqs * n_heads * splits * (head_dim + 2);
}

LLMI_EXPORT int llmi_attention_decode(const void* q, long ldq, void* out, long ldo, const void* k_cache,
                                      const void* v_cache, const int32_t* seq_pages, int pages_stride,
                                      const int32_t* seq_kv_len, const int32_t* seq_q_start, int n_seqs, int n_heads,
                                      int n_kv_heads, int head_dim, float scale, int window, int max_pages,
                                      int pages_per_split, float* partials, long partials_floats, int* tickets,
                                      int n_tickets, int* error_flag, int n_live, int cluster, cudaStream_t stream) {
  if (n_seqs <= 0 || n_heads <= 0 || n_kv_heads <= 0 || max_pages <= 0 || pages_per_split <= 0) return LLMI_ERR_BAD_SIZE;
  if (n_heads % n_kv_heads) return LLMI_ERR_BAD_SIZE;
  const int group = n_heads / n_kv_heads;
  if (!llmi_attention_decode_supported(head_dim, group)) return LLMI_ERR_UNSUPPORTED;
  if (((uintptr_t)q & 15) || (ldq & 7) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15)) return LLMI_ERR_ALIGN;
  const int splits = (max_pages + pages_per_split - 1) / pages_per_split;
  if (llmi_attention_decode_workspace(n_seqs, n_heads, head_dim, max_pages, pages_per_split) > partials_floats ||
      (long)n_seqs * n_kv_heads > n_tickets)
    return LLMI_ERR_BAD_SIZE;
  DecodeParams p{(const __nv_bfloat16*)q, ldq, (__nv_bfloat16*)out, ldo, (const __nv_bfloat16*)k_cache,
                 (const __nv_bfloat16*)v_cache, seq_pages, seq_kv_len, seq_q_start, pages_stride, n_kv_heads,
                 scale * 1.4426950408889634f, window, pages_per_split, splits, partials, tickets, error_flag,
                 0, nullptr, 0, n_heads, 0, nullptr, nullptr};
  return dispatch_decode(p, n_seqs, n_live, cluster, head_dim, group, stream);
}

// The same with the step's position encoding fused in: `qkv` holds the un-rotated [q | k | v] rows of the
// step's tokens (one per sequence); q is rotated as it is read, and the new k (rotated) and v are appended
// to the cache before the page they land in is fetched.  rotary_dim: head_dim (rotate-half over the whole
// head, inv_freq[head_dim/2]) or 0 (append only).  write_kv 0: the cache already holds the new entries.
LLMI_EXPORT int llmi_attention_decode_fused(const void* qkv, long ldq, void* out, long ldo, void* k_cache, void* v_cache,
                                            const int32_t* seq_pages, int pages_stride, const int32_t* seq_kv_len,
                                            const int32_t* seq_q_start, int n_seqs, int n_heads, int n_kv_heads,
                                            int head_dim, float scale, int window, int max_pages, int pages_per_split,
                                            const float* inv_freq, int rotary_dim, int write_kv, float* partials,
                                            long partials_floats, int* tickets, int n_tickets, int* error_flag,
                                            int n_live, int cluster, cudaStream_t stream) {
  if (n_seqs <= 0 || n_heads <= 0 || n_kv_heads <= 0 || max_pages <= 0 || pages_per_split <= 0) return LLMI_ERR_BAD_SIZE;
  if (n_heads % n_kv_heads) return LLMI_ERR_BAD_SIZE;
  const int group = n_heads / n_kv_heads;
  if (!llmi_attention_decode_supported(head_dim, group)) return LLMI_ERR_UNSUPPORTED;
  if (rotary_dim != 0 && (rotary_dim != head_dim || !inv_freq)) return LLMI_ERR_UNSUPPORTED;
  if (((uintptr_t)qkv & 15) || (ldq & 7) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15)) return LLMI_ERR_ALIGN;
  const int splits = (max_pages + pages_per_split - 1) / pages_per_split;
  if (llmi_attention_decode_workspace(n_seqs, n_heads, head_dim, max_pages, pages_per_split) > partials_floats ||
      (long)n_seqs * n_kv_heads > n_tickets)
    return LLMI_ERR_BAD_SIZE;
  DecodeParams p{(const __nv_bfloat16*)qkv, ldq, (__nv_bfloat16*)out, ldo, (const __nv_bfloat16*)k_cache,
                 (const __nv_bfloat16*)v_cache, seq_pages, seq_kv_len, seq_q_start, pages_stride, n_kv_heads,
                 scale * 1.4426950408889634f, window, pages_per_split, splits, partials, tickets, error_flag,
                 1, inv_freq, rotary_dim, n_heads, write_kv ? 1 : 0, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache};
  return dispatch_decode(p, n_seqs, n_live, cluster, head_dim, group, stream);
}

// Blocks of the kernel that a step of n_seqs sequences would run that are resident at once, and whether that is the
// variant with two producer threads (its items may be longer: see ops/kernels.py decode_pages_per_split).
LLMI_EXPORT int llmi_attention_decode_plan(int head_dim, int group, int n_seqs, int n_kv_heads, int* two_producers) {
  if (two_producers) *two_producers = 0;
#define LLMI_DEC(HD) \
  if (head_dim == HD && group == 1 && decode_two_producers<HD, 1>(n_seqs, n_kv_heads)) { \
    if (two_producers) *two_producers = 1; \
    return decode_resident<HD, 1, true>(); \
  }
  LLMI_DEC(64); LLMI_DEC(128); LLMI_DEC(32);
#undef LLMI_DEC
  return llmi_attention_decode_resident(head_dim, group);
}

// Clusters of `cluster` blocks of the cluster form (ungrouped queries only) that the device holds at once; 0 if none.
LLMI_EXPORT int llmi_attention_decode_clusters_resident(int head_dim, int group, int cluster) {
  if (group != 1 || (cluster != 2 && cluster != 4 && cluster != 8)) return 0;
  if (head_dim == 64) return decode_clusters_resident<64>(cluster);
  if (head_dim == 128) return decode_clusters_resident<128>(cluster);
  if (head_dim == 32) return decode_clusters_resident<32>(cluster);
  return 0;
}

LLMI_EXPORT int llmi_attention_decode_resident(int head_dim, int group) {
#define LLMI_DEC(HD, G) \
  if (head_dim == HD && group == G) return decode_resident<HD, G>()
  LLMI_DEC(64, 1); LLMI_DEC(64, 2); LLMI_DEC(64, 3); LLMI_DEC(64, 4); LLMI_DEC(64, 8);
  LLMI_DEC(128, 1); LLMI_DEC(128, 2); LLMI_DEC(128, 3); LLMI_DEC(128, 4); LLMI_DEC(128, 8);
  LLMI_DEC(32, 1); LLMI_DEC(32, 2); LLMI_DEC(32, 4);
#undef LLMI_DEC
  return 0;
}

// ------------------------------------------------------------------------------------------------
// The same decode attention for callers that cannot allocate device memory (see llmi_no_alloc.h).
// Its scratch — the per-split partial results, the tickets and an error word — lives in the array
// below, which every GPU that loads this library holds until the process exits.

namespace {

constexpr long STATIC_PARTIALS_FLOATS = 1L << 20;   // 4 MiB of partial results
constexpr int STATIC_TICKETS = 1 << 14;             // 64 KiB of tickets
constexpr int STATIC_MAX_DEVICES = 64;

struct DecodeStaticScratch {
  float partials[STATIC_PARTIALS_FLOATS];
  int tickets[STATIC_TICKETS];
  int error;
};

static __device__ __align__(256) DecodeStaticScratch g_decode_static_scratch;

// The device address of the array, per device.  In host code the name g_decode_static_scratch is only a
// stand-in for the symbol, not an address a kernel could use: the address comes from cudaGetSymbolAddress,
// asked once per device with that device current.
DecodeStaticScratch* g_decode_static_ptr[STATIC_MAX_DEVICES] = {};

}  // namespace

LLMI_EXPORT int llmi_attention_decode_static(const void* q, long ldq, void* out, long ldo, const void* k_cache,
                                             const void* v_cache, const int32_t* seq_pages, int pages_stride,
                                             const int32_t* seq_kv_len, const int32_t* seq_q_start, int n_seqs,
                                             int n_heads, int n_kv_heads, int head_dim, float scale, int window,
                                             int max_pages, int pages_per_split, int* error_out, cudaStream_t stream) {
  if (n_seqs <= 0 || n_heads <= 0 || n_kv_heads <= 0 || max_pages <= 0 || pages_per_split <= 0) return LLMI_ERR_BAD_SIZE;
  if (n_heads % n_kv_heads) return LLMI_ERR_BAD_SIZE;
  const int group = n_heads / n_kv_heads;
  if (!llmi_attention_decode_supported(head_dim, group)) return LLMI_ERR_UNSUPPORTED;
  if (((uintptr_t)q & 15) || (ldq & 7) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15)) return LLMI_ERR_ALIGN;
  // the built-in scratch has a fixed size: a problem that needs more is refused, never truncated
  if (llmi_attention_decode_workspace(n_seqs, n_heads, head_dim, max_pages, pages_per_split) > STATIC_PARTIALS_FLOATS ||
      (long)n_seqs * n_kv_heads > STATIC_TICKETS)
    return LLMI_ERR_STATIC_SCRATCH;

  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= STATIC_MAX_DEVICES) return LLMI_ERR_DRIVER;
  if (!g_decode_static_ptr[dev]) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_decode_static_scratch) != cudaSuccess || !ptr) return LLMI_ERR_DRIVER;
    g_decode_static_ptr[dev] = (DecodeStaticScratch*)ptr;
  }
  DecodeStaticScratch* sc = g_decode_static_ptr[dev];
  // The array keeps what the last call left.  The tickets of this call's sequences and the error word must
  // start at zero (a call that was cut short may have left them otherwise); the partials are written before
  // they are read and need no clearing.
  if (cudaMemsetAsync(sc->tickets, 0, sizeof(int) * (size_t)n_seqs * n_kv_heads, stream) != cudaSuccess ||
      cudaMemsetAsync(&sc->error, 0, sizeof(int), stream) != cudaSuccess)
    return LLMI_ERR_LAUNCH;
  const int splits = (max_pages + pages_per_split - 1) / pages_per_split;
  DecodeParams p{(const __nv_bfloat16*)q, ldq, (__nv_bfloat16*)out, ldo, (const __nv_bfloat16*)k_cache,
                 (const __nv_bfloat16*)v_cache, seq_pages, seq_kv_len, seq_q_start, pages_stride, n_kv_heads,
                 scale * 1.4426950408889634f, window, pages_per_split, splits, sc->partials, sc->tickets, &sc->error,
                 0, nullptr, 0, n_heads, 0, nullptr, nullptr};
  const int rc = dispatch_decode(p, n_seqs, 0, 0, head_dim, group, stream);
  if (rc != LLMI_OK) return rc;
  if (error_out && cudaMemcpyAsync(error_out, &sc->error, sizeof(int), cudaMemcpyDeviceToDevice, stream) != cudaSuccess)
    return LLMI_ERR_LAUNCH;
  return LLMI_OK;
}
