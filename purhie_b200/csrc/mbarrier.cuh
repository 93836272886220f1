// mbarrier and bulk-copy wrappers with bounded waits.  A wait that does not complete within WAIT_LIMIT_NS sets
// an error word and returns false; nothing here spins without a bound.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace ph_mbar {

constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;   // 2 s

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ bool try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// One look at the barrier that never suspends the thread.
__device__ __forceinline__ bool test_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_timer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool wait(uint64_t* bar, uint32_t parity, int* error_flag, int code) {
    if (try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_timer();
    for (uint32_t i = 0;; ++i) {
        if (try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && global_timer() - t0 > WAIT_LIMIT_NS) {
            atomicExch(error_flag, code);
            return false;
        }
    }
}

// size bytes (a multiple of 16) from global to shared memory, both 16-byte aligned; completion is counted on bar.
__device__ __forceinline__ void bulk_copy(void* dst, const void* src, uint32_t size, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_addr(dst)), "l"(src), "r"(size), "r"(smem_addr(bar)) : "memory");
}

}  // namespace ph_mbar
