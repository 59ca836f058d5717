// mbarrier and bulk-copy helpers shared by the sm_100a kernels that pipeline through shared memory.
// Every wait is bounded: after about a second it records a code in *error_flag and returns false,
// so that a fault in a pipeline unwinds the block instead of hanging the GPU.
#pragma once
#include <stdint.h>

namespace llmi {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait.  Returns false (and records `code`) if the phase did not complete in ~1 s.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* error_flag, int code) {
  uint32_t done = 0;
  uint64_t t0 = 0;
  for (uint32_t spins = 0;; ++spins) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
    if ((spins & 1023u) == 1023u) {
      const uint64_t now = global_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > 1000000000ull) {
        if (error_flag) atomicCAS(error_flag, 0, code);
        return false;
      }
    }
  }
}

// Plain (untiled) bulk copy global -> shared; both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// A buffer that threads have READ (ld.shared, ldmatrix: the generic proxy) and that a bulk or tensor copy (the async
// proxy) will fill again: every reading thread calls this before it says that the buffer is free.  The arrive on the
// mbarrier alone does not order the reads before a write of the other proxy.  (Measured on the weight-streaming product
// without it: with two blocks on an SM, 9 to 16 tokens and two or three stages a row tile, one row tile in three
// thousand came out with a few rows wrong in 3 to 90 % of the launches — rows of the tile that the next copy brought.)
__device__ __forceinline__ void fence_reads_before_async_writes() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- thread-block clusters ----
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_size() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
// the address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t cluster_addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr));
  return v;
}
// an arrive on an mbarrier of another CTA of the cluster (its address from map_to_rank); what this thread wrote, or
// saw written, before is visible to whoever waits on that barrier with mbar_wait_cluster
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void st_cluster_f32(uint32_t cluster_addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(cluster_addr), "f"(v) : "memory");
}
// mbar_wait for a barrier that other CTAs of the cluster arrive on after plain stores into this CTA's shared memory
// (acquire at cluster scope); bounded like mbar_wait
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, int* error_flag, int code) {
  uint32_t done = 0;
  uint64_t t0 = 0;
  for (uint32_t spins = 0;; ++spins) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
    if ((spins & 1023u) == 1023u) {
      const uint64_t now = global_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > 1000000000ull) {
        if (error_flag) atomicCAS(error_flag, 0, code);
        return false;
      }
    }
  }
}
// every thread of every CTA of the cluster arrives and waits (what was written to shared memory before is
// visible to the cluster's other CTAs after)
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

}  // namespace llmi
