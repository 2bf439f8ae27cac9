// mbarrier and bulk-copy (`cp.async.bulk`) primitives for sm_100a, shared by the
// kernels that stage dense rows in shared memory with the asynchronous copy
// unit instead of with register loads.
//
// A bulk copy moves one contiguous span (a dense row is one: k_loc * 4 bytes,
// 16-byte aligned, a multiple of 16 bytes) between global and shared memory
// without passing through registers; loads complete on an mbarrier
// (complete_tx::bytes), stores in bulk groups of the issuing thread.  The source
// of a load may be another GPU's memory (a peer mapping); no copy here uses
// cluster multicast, and every copy targets the shared memory of the issuing
// CTA.  Every wait is bounded.
#pragma once
#include "sp3_cuda.cuh"

namespace sp3 {

constexpr unsigned ASYNC_WAIT_TRIES = 1u << 22;

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
// Makes freshly initialised barriers visible to the asynchronous copy unit; follow with a block barrier.
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false after ASYNC_WAIT_TRIES unsuccessful probes.
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity) {
    for (unsigned i = 0; i < ASYNC_WAIT_TRIES; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// Bounded by time: false when `limit_ns` has passed without the phase completing.
__device__ __forceinline__ bool mbar_wait_ns(unsigned bar, unsigned parity, unsigned long long limit_ns) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = globaltimer_ns();
    for (;;) {
        for (int i = 0; i < 256; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (globaltimer_ns() - t0 > limit_ns) return false;
    }
}

// global -> shared memory of this CTA, `bytes` a multiple of 16, both addresses 16-byte aligned.
__device__ __forceinline__ void bulk_load(unsigned dst_smem, const void* src, unsigned bytes, unsigned bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(dst_smem), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// shared memory of this CTA -> global, in the issuing thread's current bulk group.
__device__ __forceinline__ void bulk_store(void* dst, unsigned src_smem, unsigned bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                 :: "l"(dst), "r"(src_smem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Until at most N of this thread's bulk groups still read their shared-memory source.
template <int N> __device__ __forceinline__ void bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// Until at most N of this thread's bulk groups are incomplete (their global writes done).
template <int N> __device__ __forceinline__ void bulk_wait() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// Orders accesses of the asynchronous copy unit against ordinary loads and stores of this thread.
__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async;" ::: "memory"); }

}  // namespace sp3
