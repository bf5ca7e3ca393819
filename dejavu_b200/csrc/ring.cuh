// Shared-memory staging of weight rows with bulk asynchronous copies (cp.async.bulk, the 1-D form of TMA)
// completed on mbarriers. One thread issues a copy of several KB and goes on; the copy engine keeps the bytes
// in flight, so the amount of HBM traffic a multiprocessor has outstanding is bounded by shared memory
// (~200 KB), not by registers. Every copy here reads this GPU's own memory into the issuing block's own shared
// memory; no copy is addressed to more than one block.
#pragma once
#include "common.cuh"

namespace djv {

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
// makes the initialised barriers visible to the copy engine (call once, before the block-wide barrier)
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// one arrival that also announces `bytes` of copies that will complete on the barrier
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait for phase `parity` of the barrier. A copy from this GPU's own memory always completes, so the
// limit (one second of %globaltimer) is never reached in a healthy run; it exists so that no spin in this
// library is unbounded. Returns false when it ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, unsigned parity) {
  if (mbar_try_wait(bar, parity)) return true;
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (;;) {
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    if (t - t0 > 1000ull * 1000 * 1000) return false;
  }
}
// global -> this block's shared memory, `bytes` a multiple of 16, both addresses 16-byte aligned
__device__ __forceinline__ void bulk_load(void *smem_dst, const void *gmem_src, unsigned bytes, uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// orders earlier generic-proxy accesses to shared memory before later copies into the same locations
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

}  // namespace djv
