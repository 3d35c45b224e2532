// pair_wait.cuh — bounded poll of one (value, epoch) pair in global memory.
// Include inside namespace yule { namespace { … } }.
#pragma once

// Returns the value once the pair carries `epoch`.  Bounded, and bounded once per failure: the first wait that
// runs out of `budget` cycles writes the status word; every wait that starts or polls after that returns at once
// with whatever the pair holds (the host reads the status word and discards the step).
__device__ __forceinline__ float pair_wait(const uint2 *p, uint32_t epoch, int *status, long long budget) {
    long long t0 = 0;
    for (uint32_t it = 0;; it++) {
        uint2 q;
        asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(q.x), "=r"(q.y) : "l"(p) : "memory");
        if (q.y == epoch) return __uint_as_float(q.x);
        if (it == 0) t0 = clock64();
        if (it != 0 && (it & 63u) != 63u) continue;
        if (*reinterpret_cast<volatile int *>(status) != 0) return __uint_as_float(q.x);
        if (clock64() - t0 >= budget) {
            atomicCAS(status, 0, kStatusPeerTimeout);
            return __uint_as_float(q.x);
        }
    }
}

// The same in two steps, for several pairs at once: issue every load (pair_peek), then settle each
// (pair_settle polls only the ones that had not arrived).
__device__ __forceinline__ uint2 pair_peek(const uint2 *p) {
    uint2 q;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(q.x), "=r"(q.y) : "l"(p) : "memory");
    return q;
}
__device__ __forceinline__ float pair_settle(uint2 q, const uint2 *p, uint32_t epoch, int *status, long long budget) {
    return q.y == epoch ? __uint_as_float(q.x) : pair_wait(p, epoch, status, budget);
}
