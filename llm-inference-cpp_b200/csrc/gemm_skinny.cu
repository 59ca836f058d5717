// y = x · Wᵀ for a handful of tokens (decode at small batch): a weight-streaming product.
//
// Same operation as the reference's matmul (src/model/kernels.cpp:97-113; W is [out, in]) and as gemm_tc.cu,
// for the case where it is nothing but a read of W from HBM: 1..32 tokens (up to 64 for small matrices).
// The big kernel's 128-row weight
// tiles leave too few blocks for such products unless k is split across blocks, and the cross-block reduce,
// the TMEM allocation and the ticket cost more than the product itself (a 8 MB weight matrix is 1.2 us of
// HBM time).  Here a block owns 16 output rows over the WHOLE k range, so nothing crosses blocks:
//
//   * a producer warp streams W[16 rows, 256 k] and x[tokens, 256 k] by TMA (128-byte swizzle) into a ring
//     of shared-memory stages — 72 KB in flight per block, three blocks per SM;
//   * four consumer warps each take one 64-wide k slice of every stage: ldmatrix + mma.sync m16n8k16
//     (bf16 in, fp32 accumulators in registers: 16 rows x 8 tokens per tile);
//   * at the end of a row tile the four partial sums are added in warp order through shared memory and
//     the epilogue (bias, store / fp32 store / residual add / silu(gate)·up on interleaved rows) writes
//     token-major output.
// Two optional extras fold the RMSNorm between two products of a decode layer into them (a norm of 8 rows is
// all launch and latency).  The product BEFORE the norm (residual add) also writes, for the x it has just
// updated, h = bf16(norm_weight * x) and the sum of x^2 over its 16 rows, per tile and token; the product
// AFTER the norm takes h as its input, adds the tiles' sums in tile order, and multiplies its accumulators
// by 1/sqrt(sum/k + eps) before the bias: y = scale * (h . W) is the normalised product with the scale
// applied in fp32 at the end instead of before the rounding of h.
// The token rows are fetched as they are (a TMA box of exactly n_tok rows, packed [slice][token][64 k]): what a
// block can take in through TMA is the bound (about 59 GB/s an SM), and at one token eight padded rows would be
// a third of it.  The MMA's B fragment still spans 8 (16, 32) rows; the rows past n_tok are whatever follows
// in shared memory and feed output columns that nobody stores.
// Blocks are persistent over row tiles and the ring runs on across tiles.  The k order of the additions is
// fixed (it does not depend on the number of tokens), and programmatic dependent launch lets the first
// weight tiles be requested before the kernel that produces x has finished.
#include <cuda.h>

#include "common.cuh"
#include "sm100.cuh"

namespace llmi {

constexpr int SK_ROWS = 16;          // output rows per tile
constexpr int SK_BK = 256;           // k per stage: four 64-wide slices, one per consumer warp
// stages of the ring: six, three for the widest token tile (64 tokens: 40 KB a stage)
template <int NT> struct SkStages { static constexpr int value = NT >= 8 ? 3 : (NT == 1 ? 9 : 6); };
constexpr int SK_CONSUMERS = 4;
constexpr int SK_THREADS = (SK_CONSUMERS + 1) * 32;

constexpr int SK_SS_STRIDE = 64;     // floats per tile in the sums of squares (tokens <= 64)

constexpr int SK_STORE = 0, SK_STORE_F32 = 1, SK_ADD_F32 = 2, SK_SWIGLU = 3;

struct SkinnyParams {
  int m_out, n_tok, k;
  void* out;
  long ldo;
  const float* bias;
  int mode;
  int* error_flag;
  int x_rows;                 // rows of the token box: n_tok
  // the norm AFTER this product (mode SK_ADD_F32 only): null or
  const float* emit_w;        // [m_out] weight of that norm
  __nv_bfloat16* emit_h;      // [n_tok, emit_ldh]: bf16(emit_w * x_new)
  long emit_ldh;
  float* emit_ss;             // [m_tiles, SK_SS_STRIDE]: sum over the tile's rows of x_new^2, per token
  // the norm BEFORE this product: null or
  const float* in_ss;         // [in_tiles, SK_SS_STRIDE] as written by the product before
  int in_tiles;
  float in_eps;
};

// One copy fetches [4 k slices][rows][64 k]: the matrix is seen as a 3-D tensor (k within a slice, row, slice).
__device__ __forceinline__ void sk_tma(uint32_t dst, const CUtensorMap* map, int row, int slice, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(0), "r"(row), "r"(slice)
      : "memory");
}
__device__ __forceinline__ void sk_mma(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// NT = token tiles of 8 (tokens <= 8 * NT)
template <int NT>
__global__ void __launch_bounds__(SK_THREADS)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, SkinnyParams p,
                   int m_tiles) {
  constexpr int NPAD = NT * 8;
  constexpr int SK_STAGES = SkStages<NT>::value;
  constexpr int W_SLICE = SK_ROWS * 128;          // 16 rows x 64 k of bf16
  constexpr int X_SLICE = NPAD * 128;
  constexpr int W_BYTES = 4 * W_SLICE, X_BYTES = 4 * X_SLICE;
  constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
  extern __shared__ uint8_t smem_raw[];
  __shared__ float s_part[SK_CONSUMERS][32][NT * 4];
  __shared__ float s_scale[NPAD];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = base + SK_STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (SK_STAGES + s); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kstages = (p.k + SK_BK - 1) / SK_BK;
  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    for (int s = 0; s < SK_STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), SK_CONSUMERS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  pdl_launch_dependents();

  if (warp == SK_CONSUMERS) {
    // ---- producer ----
    if (lane == 0) {
      int my_tiles = 0;
      for (int t = blockIdx.x; t < m_tiles; t += gridDim.x) ++my_tiles;
      const int total = my_tiles * kstages;
      const int ahead = total < SK_STAGES ? total : SK_STAGES;   // stages whose weights are requested before the wait
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < m_tiles && ok; t += gridDim.x) {
        for (int ks = 0; ks < kstages; ++ks, ++it) {
          const int s = it % SK_STAGES;
          if (it >= SK_STAGES && !mbar_wait(empty_bar(s), ((it / SK_STAGES) - 1) & 1, p.error_flag, 31)) { ok = false; break; }
          mbar_expect_tx(full_bar(s), W_BYTES + 4 * p.x_rows * 128);
          const uint32_t dst = base + s * STAGE_BYTES;
          sk_tma(dst, &map_w, t * SK_ROWS, ks * 4, full_bar(s));
          if (it < ahead) {
            if (it == ahead - 1) {
              pdl_wait();   // x comes from the kernel before; the weights requested so far did not have to wait for it
              for (int j = 0; j < ahead; ++j) {
                const int ksj = j % kstages;      // the first stages belong to this block's first tile(s)
                sk_tma(base + j * STAGE_BYTES + W_BYTES, &map_x, 0, ksj * 4, full_bar(j));
              }
            }
          } else {
            sk_tma(dst + W_BYTES, &map_x, 0, ks * 4, full_bar(s));
          }
        }
      }
    }
    return;
  }

  // ---- consumers ----
  pdl_wait();   // the output (residual add) and the bias of a previous layer's step are safe to touch from here
  if (p.in_ss) {
    // scale of each token's row: the tiles' sums of squares added in tile order (one partial sum per thread
    // over every (128 / NPAD)-th tile, then those in thread order), as the norm kernel would: 1/sqrt(mean + eps)
    constexpr int PARTS = SK_CONSUMERS * 32 / NPAD;
    float* red = &s_part[0][0][0];        // free until the first tile's end
    const int tok = threadIdx.x % NPAD, part = threadIdx.x / NPAD;
    float a = 0.f;
    for (int t = part; t < p.in_tiles; t += PARTS) a += __ldcg(&p.in_ss[(size_t)t * SK_SS_STRIDE + tok]);
    red[part * NPAD + tok] = a;
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (threadIdx.x < NPAD) {
      float sum = 0.f;
      for (int q = 0; q < PARTS; ++q) sum += red[q * NPAD + threadIdx.x];
      s_scale[threadIdx.x] = 1.0f / sqrtf(sum / (float)p.k + p.in_eps);
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
  }
  int it = 0;
  bool ok = true;
  const int g = lane >> 2, tq = lane & 3;
  for (int t = blockIdx.x; t < m_tiles && ok; t += gridDim.x) {
    float acc[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[n][e] = 0.f;
    // residual add: the old values of this tile's outputs are asked for now and used after the k loop (nobody else
    // writes them), so the tile does not end with a round trip to L2
    constexpr int OLD = NPAD * SK_ROWS / (SK_CONSUMERS * 32);
    float old[OLD], norm_w[OLD];
    if (p.mode == SK_ADD_F32) {
#pragma unroll
      for (int r = 0; r < OLD; ++r) {
        const int idx = threadIdx.x + r * SK_CONSUMERS * 32;
        const int tok = idx >> 4, m = t * SK_ROWS + (idx & 15);
        const bool live = tok < p.n_tok && m < p.m_out;
        old[r] = live ? __ldcg((const float*)p.out + (size_t)tok * p.ldo + m) : 0.f;
        norm_w[r] = (live && p.emit_w) ? p.emit_w[m] : 0.f;      // the weight of the norm behind this product, likewise
      }
    }
    for (int ks = 0; ks < kstages; ++ks, ++it) {
      const int s = it % SK_STAGES;
      ok = mbar_wait(full_bar(s), (it / SK_STAGES) & 1, p.error_flag, 32);
      if (!ok) break;
      const uint32_t w_slice = base + s * STAGE_BYTES + warp * W_SLICE;
      const uint32_t x_base = base + s * STAGE_BYTES + W_BYTES;
      const int x_row0 = warp * p.x_rows;                  // this warp's slice starts at this row of the packed box
#pragma unroll
      for (int c = 0; c < 4; ++c) {       // four k16 chunks of this warp's 64-wide slice
        uint32_t a[4];
        {
          const int mtx = lane >> 3, r = lane & 7;
          const int row = (mtx & 1) * 8 + r, kch = c * 2 + (mtx >> 1);
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                       : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3])
                       : "r"(w_slice + (uint32_t)(row * 128 + ((kch ^ (row & 7)) << 4))));
        }
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          uint32_t b0, b1;
          {
            const int mtx = (lane >> 3) & 1, r = lane & 7;       // lanes 16..31 repeat the addresses of 0..15 (x2)
            const int row = x_row0 + n * 8 + r, kch = c * 2 + mtx;     // the swizzle follows the physical row
            asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];"
                         : "=r"(b0), "=r"(b1)
                         : "r"(x_base + (uint32_t)(row * 128 + ((kch ^ (row & 7)) << 4))));
          }
          sk_mma(acc[n], a, b0, b1);
        }
      }
      fence_reads_before_async_writes();
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_bar(s));
    }
    if (!ok) break;
    // add the four warps' partial sums in warp order, then the epilogue, token-major
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) s_part[warp][lane][n * 4 + e] = acc[n][e];
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const int m0 = t * SK_ROWS;
    if (p.mode == SK_SWIGLU) {
      // rows alternate gate and up: 8 features per tile
      for (int idx = threadIdx.x; idx < NPAD * 8; idx += SK_CONSUMERS * 32) {
        const int tok = idx >> 3, f = idx & 7;
        if (tok >= p.n_tok || m0 + 2 * f + 1 >= p.m_out) continue;
        const float sc = p.in_ss ? s_scale[tok] : 1.0f;
        float gu[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int row = 2 * f + h;                       // accumulator element (row, tok) lives in lane (row%8)*4 + (tok%8)/2
          const int ln = (row & 7) * 4 + ((tok & 7) >> 1), e = (row >> 3) * 2 + (tok & 1), n = tok >> 3;
          float v = 0.f;
#pragma unroll
          for (int w = 0; w < SK_CONSUMERS; ++w) v += s_part[w][ln][n * 4 + e];
          gu[h] = v * sc;
        }
        ((__nv_bfloat16*)p.out)[(size_t)tok * p.ldo + (m0 >> 1) + f] =
            __float2bfloat16_rn(__fdividef(gu[0], 1.0f + __expf(-gu[0])) * gu[1]);
      }
    } else {
      // NPAD * 16 is a multiple of the 128 consumer threads: every thread makes the same number of rounds, and
      // the 16 rows of one token sit in 16 neighbouring lanes (the sum of squares below relies on both)
#pragma unroll
      for (int r = 0; r < OLD; ++r) {
        const int idx = threadIdx.x + r * SK_CONSUMERS * 32;
        const int tok = idx >> 4, row = idx & 15;
        const int m = m0 + row;
        const bool live = tok < p.n_tok && m < p.m_out;
        const int ln = (row & 7) * 4 + ((tok & 7) >> 1), e = (row >> 3) * 2 + (tok & 1), n = tok >> 3;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < SK_CONSUMERS; ++w) v += s_part[w][ln][n * 4 + e];
        if (p.in_ss) v *= s_scale[tok];
        float xn = 0.f;
        if (live) {
          if (p.bias) v += p.bias[m];
          const size_t o = (size_t)tok * p.ldo + m;
          if (p.mode == SK_STORE) ((__nv_bfloat16*)p.out)[o] = __float2bfloat16_rn(v);
          else if (p.mode == SK_STORE_F32) ((float*)p.out)[o] = v;
          else {
            xn = old[r] + v;
            ((float*)p.out)[o] = xn;
          }
        }
        if (p.emit_w) {      // only with SK_ADD_F32
          if (live) p.emit_h[(size_t)tok * p.emit_ldh + m] = __float2bfloat16_rn(norm_w[r] * xn);
          float sq = xn * xn;
#pragma unroll
          for (int o = 8; o >= 1; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
          if (row == 0) p.emit_ss[(size_t)t * SK_SS_STRIDE + tok] = sq;
        }
      }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");   // s_part is free for the next tile
  }
}

typedef CUresult (*SkEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int sk_make_map(CUtensorMap* map, const void* ptr, long rows, long k, long ld, int box_rows) {
  static SkEncodeFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return LLMI_ERR_DRIVER;
    fn = (SkEncodeFn)sym;
  }
  // (k within a 64-wide slice, row, slice): k must be a multiple of 64, so that no slice runs over a row's end
  const cuuint64_t dims[3] = {64, (cuuint64_t)rows, (cuuint64_t)(k / 64)};
  const cuuint64_t strides[2] = {(cuuint64_t)ld * 2, 128};
  const cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 4};
  const cuuint32_t elem[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS
             ? LLMI_OK
             : LLMI_ERR_DRIVER;
}

template <int NT>
static int launch_skinny(const CUtensorMap& mw, const CUtensorMap& mx, const SkinnyParams& p, int m_tiles,
                         cudaStream_t stream) {
  constexpr int SK_STAGES = SkStages<NT>::value;
  constexpr int SMEM = SK_STAGES * (4 * SK_ROWS * 128 + 4 * NT * 8 * 128) + 1024 + 8 * 2 * SK_STAGES + 16;
  static PerDevice<int> resident_on;
  int& resident = resident_on.here();
  if (!resident) {
    if (cudaFuncSetAttribute(gemm_skinny_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
      return LLMI_ERR_LAUNCH;
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemm_skinny_kernel<NT>, SK_THREADS, SMEM) != cudaSuccess ||
        per_sm < 1)
      per_sm = 1;
    resident = per_sm * sm_count();
  }
  const int grid = m_tiles < resident ? m_tiles : resident;
  return launch_pdl(PDL_GEMM, gemm_skinny_kernel<NT>, grid, SK_THREADS, SMEM, stream, mw, mx, p, m_tiles);
}

}  // namespace llmi

using namespace llmi;

// Most tokens the weight-streaming product takes.
LLMI_EXPORT int llmi_gemm_skinny_max_tokens() { return 64; }

// y[n_tok, m_out] (mode) = x[n_tok, k] · w[m_out, k]ᵀ + bias for n_tok <= 64 and k % 64 == 0; bf16 inputs; pitches in elements;
// modes as llmi_gemm_tc (0 store, 1 fp32 store, 2 fp32 add, 3 gated with alternating gate/up rows).
// emit_w/emit_h/emit_ss (mode 2 only, or all null): also write h = bf16(emit_w * y_new) and the per-tile sums of
// y_new^2, emit_ss[ceil(m_out/16), 64].  in_ss/in_tiles/in_eps (or null): x is such an h; the accumulators are
// multiplied by 1/sqrt(sum of the tiles' sums / k + in_eps) before the bias.
LLMI_EXPORT int llmi_gemm_skinny(const void* x, long ldx, const void* w, long ldw, const float* bias, void* y, long ldy,
                                 int n_tok, int m_out, int k, int mode, const float* emit_w, void* emit_h, long emit_ldh,
                                 float* emit_ss, const float* in_ss, int in_tiles, float in_eps, int* error_flag,
                                 cudaStream_t stream) {
  if (n_tok <= 0 || n_tok > 64 || m_out <= 0 || k <= 0) return LLMI_ERR_BAD_SIZE;
  if (mode < 0 || mode > 3) return LLMI_ERR_UNSUPPORTED;
  if (mode == SK_SWIGLU && ((m_out & 1) || bias)) return LLMI_ERR_UNSUPPORTED;
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15) || (ldx & 7) || (ldw & 7)) return LLMI_ERR_ALIGN;
  if (k % 64) return LLMI_ERR_UNSUPPORTED;   // the 3-D view of the matrices needs whole 64-wide k slices
  if (emit_w && (mode != SK_ADD_F32 || !emit_h || !emit_ss)) return LLMI_ERR_UNSUPPORTED;
  if (in_ss && in_tiles <= 0) return LLMI_ERR_BAD_SIZE;
  const int nt = n_tok <= 8 ? 1 : (n_tok <= 16 ? 2 : (n_tok <= 32 ? 4 : 8));
  CUtensorMap mw, mx;
  int rc = sk_make_map(&mw, w, m_out, k, ldw, SK_ROWS);
  if (rc != LLMI_OK) return rc;
  rc = sk_make_map(&mx, x, n_tok, k, ldx, n_tok);
  if (rc != LLMI_OK) return rc;
  SkinnyParams p{m_out, n_tok, k, y, ldy, bias, mode, error_flag, n_tok, emit_w, (__nv_bfloat16*)emit_h, emit_ldh, emit_ss,
                 in_ss, in_tiles, in_eps};
  const int m_tiles = (m_out + SK_ROWS - 1) / SK_ROWS;
  if (nt == 1) return launch_skinny<1>(mw, mx, p, m_tiles, stream);
  if (nt == 2) return launch_skinny<2>(mw, mx, p, m_tiles, stream);
  if (nt == 4) return launch_skinny<4>(mw, mx, p, m_tiles, stream);
  return launch_skinny<8>(mw, mx, p, m_tiles, stream);
}
