// mbarrier + bulk-copy (TMA) PTX wrappers shared by the GEMM and the row kernels, and the bounded wait every kernel of this
// library uses: a wait that runs out records TF_ERR_DEVICE_TIMEOUT in the device status words (read by tf_device_status) and
// returns false, so the kernel can leave its loops and return normally.
#pragma once

#include "common.cuh"

namespace tf {

// Device address of the two status words ([0] status, [1] detail) on the current device, looked up once per device.
// nullptr when the lookup fails (the caller reports TF_ERR_CUDA).
int* device_status_words();

#ifdef __CUDACC__

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Untiled bulk copy global -> shared (both addresses 16-byte aligned, bytes a multiple of 16), completion counted on `bar`.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// Bounded wait on an mbarrier phase. `status` points at the device status words; `abort_flag` is a shared-memory word all roles
// of the CTA poll, so that one role's timeout ends the others' waits too. Returns false when the limit ran out here or elsewhere.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int where,
                                                  unsigned long long limit_ns) {
  // fast path: a few plain polls first (each try_wait already blocks for a short hardware-defined time); the timer is only read
  // once a wait turns out to be long, because reading %globaltimer costs hundreds of clocks on the issuing thread
  for (int i = 0; i < 16; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (uint32_t spins = 1;; ++spins) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spins & 0x3F) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > limit_ns) {
        *abort_flag = 1;
        if (atomicCAS(&status[0], 0, TF_ERR_DEVICE_TIMEOUT) == 0) status[1] = where * 65536 + (int)blockIdx.x;
        return false;
      }
    }
  }
}

#endif  // __CUDACC__

}  // namespace tf
