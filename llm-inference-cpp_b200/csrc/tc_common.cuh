// Pieces shared by the tcgen05 matrix-product kernels (gemm_tc.cu): tile constants, the
// shared-memory operand descriptor, MMA / commit / TMEM-load wrappers, the parameter block and the epilogue
// of one thread.
#pragma once
#include <cuda.h>

#include "common.cuh"
#include "sm100.cuh"

namespace llmi {

constexpr int TC_BM = 128;
constexpr int TC_BK = 64;  // 64 bf16 = 128 bytes = one swizzle row
constexpr int TC_THREADS = 192;

constexpr int OUT_STORE = 0, OUT_STORE_F32 = 1, OUT_ADD_F32 = 2, OUT_SWIGLU = 3;

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows 128 bytes apart,
// 8-row groups 1024 bytes apart (stride byte offset), descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);   // start address, 16-byte units
  d |= (uint64_t)1 << 16;                        // leading byte offset (unused with swizzle)
  d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset
  d |= (uint64_t)1 << 46;                        // version
  d |= (uint64_t)2 << 61;                        // SWIZZLE_128B
  return d;
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

struct TcParams {
  int m_out, n_tok, k;      // W [m_out, k], x [n_tok, k]
  void* out;                // [n_tok, m_out] row pitch ldo (elements)
  long ldo;
  const float* bias;        // [m_out] or null
  int mode;
  int splits;               // gridDim.z
  float* workspace;         // [splits][tiles][BN][128] fp32 when splits > 1
  int* tickets;             // [tiles], zero before and after the launch
  int* error_flag;
};

// The epilogue of one thread: v holds 16 consecutive tokens (n_base..) of out feature m.  Called by all
// 32 lanes of a warp together (the gated mode exchanges values between neighbouring lanes).
template <int BN>
__device__ __forceinline__ void tc_epilogue_store(const TcParams& p, float* v, int m, int n_base, int n_valid) {
  if (p.mode == OUT_SWIGLU) {
    // Rows come in pairs (2f: gate of feature f, 2f+1: up of feature f), so neighbouring lanes hold the
    // two halves of silu(gate) * up (src/model/transformer.cpp:290; src/model/kernels.cpp:148).  The even
    // lane finishes tokens 0..7 of the pair, the odd lane tokens 8..15.
    const bool is_gate = (m & 1) == 0;
    __nv_bfloat16* o = (__nv_bfloat16*)p.out + (size_t)n_base * p.ldo + (m >> 1);
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      // the even lane sends its gate of token c+8 and gets the up of token c; the odd lane the reverse
      const float recv = __shfl_xor_sync(0xffffffffu, is_gate ? v[c + 8] : v[c], 1);
      const float g = is_gate ? v[c] : recv, u = is_gate ? recv : v[c + 8];
      const int tok = is_gate ? c : c + 8;
      if (tok < n_valid && m < p.m_out)
        o[(size_t)tok * p.ldo] = __float2bfloat16_rn(__fdividef(g, 1.0f + __expf(-g)) * u);   // bf16 result: fast exp and divide suffice
    }
    return;
  }
  if (m >= p.m_out) return;
  const float b = p.bias ? p.bias[m] : 0.f;
  if (p.mode == OUT_ADD_F32) {
    // One-way additions at the L2 (a reduction, nothing comes back): nobody else adds to these elements during the
    // launch, so the result is the one of read, add, store — without the read's round trip, which costs microseconds
    // while the next kernel's weight tiles already queue at the memory.
    float* o = (float*)p.out + (size_t)n_base * p.ldo + m;
#pragma unroll
    for (int c = 0; c < 16; ++c)
      if (c < n_valid) asm volatile("red.global.add.f32 [%0], %1;" ::"l"(o + (size_t)c * p.ldo), "f"(v[c] + b) : "memory");
    return;
  }
#pragma unroll
  for (int c = 0; c < 16; ++c) {
    if (c >= n_valid) break;
    const float val = v[c] + b;
    const size_t idx = (size_t)(n_base + c) * p.ldo + m;
    if (p.mode == OUT_STORE) ((__nv_bfloat16*)p.out)[idx] = __float2bfloat16_rn(val);
    else ((float*)p.out)[idx] = val;
  }
}

__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t leader_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(leader_bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {   // arrives on `bar` in both CTAs of the pair
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"((uint16_t)3)
               : "memory");
}

}  // namespace llmi
