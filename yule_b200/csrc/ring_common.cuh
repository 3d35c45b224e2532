// ring_common.cuh — mbarrier and bulk-copy helpers of the kernels that stage weights through a shared-memory
// ring (qmv_q4k_ring.cu, qmv_q6k_ring.cu, decode_mega.cu).  Include inside namespace yule { namespace { … } }.
#pragma once

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait for a stage.  False: the copy did not complete within the budget (status recorded), or some
// other wait of this context had already given up (status set): nobody waits out a second budget.
__device__ __forceinline__ bool ring_wait(uint32_t bar, uint32_t parity, int *status, long long budget) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t it = 1;; it++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 255u) == 0u) {
            if (status && *reinterpret_cast<volatile int *>(status) != 0) return false;
            if (clock64() - t0 > budget) {
                if (status) atomicCAS(status, 0, kStatusRingTimeout);
                return false;
            }
        }
    }
}
// 1-D bulk copy global → shared memory of this CTA, completion counted in bytes on `bar`.
// src and dst 16-byte aligned, bytes a multiple of 16; the source is this GPU's own memory.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}
