// Device-side helpers for the asynchronous machinery the Blackwell kernels
// share: mbarriers, bulk (TMA) copies, bounded waits. Every wait here is
// bounded: a barrier that never completes sets an error word the host reads
// at its next synchronisation instead of hanging the GPU.
#pragma once

#include <cstdint>

namespace gq {

// Error words written to the context's status word (first failure wins).
enum : uint32_t {
    kStatusOk = 0,
    kStatusFullWaitTimedOut = 1,   // a consumer gave up waiting for a bulk copy
    kStatusEmptyWaitTimedOut = 2,  // a producer gave up waiting for a free stage
    kStatusMmaWaitTimedOut = 3,    // a wait on tensor-core completion gave up
    kStatusPeerWaitTimedOut = 16,  // + r: a gather gave up waiting for rank r's block of y
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
// Makes barrier initialisation visible to the async proxy (bulk copies, tcgen05).
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}

// Waits for the barrier's phase `parity`, at most ~2 s. On giving up it records
// `code` in *status (if still clear) and in *failed (shared memory: the other
// warps of the CTA stop waiting too) and returns false.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* failed, uint32_t* status,
                                          uint32_t code) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (*failed) return false;
        if (clock64() - start > 4000000000ll) {
            *failed = code;
            atomicCAS(status, 0u, code);
            return false;
        }
    }
}

// 1-D bulk copy global -> shared, completion counted in bytes on `bar`. Both
// addresses 16-byte aligned, `bytes` a multiple of 16.
__device__ __forceinline__ void bulk_load(void* dst_smem, const void* src_global, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst_smem)),
                 "l"(src_global), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void named_barrier_sync(uint32_t id, uint32_t threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

}  // namespace gq
