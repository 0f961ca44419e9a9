// Shared-memory barriers with transaction counts and bulk asynchronous copies (global -> shared), the
// plumbing of the producer / consumer pipelines of the matrix-vector and the streaming attention kernels.
// Every wait is bounded in time (%globaltimer): a waiter that has run out records a code in the caller's
// status word and returns, so a kernel always terminates, and it terminates within a known time.
#pragma once

#include "common.cuh"

namespace wgb {

// Default limit of a wait inside one thread block; launches that know the configured limits pass their own.
constexpr unsigned long long ASYNC_WAIT_NS = 4000000000ull;

__device__ __forceinline__ unsigned long long global_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
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
// The same with a suspend-time hint: a thread whose phase has not completed may be parked by the hardware for up
// to about `hint_ns` before the instruction returns false, instead of coming back at once to poll again (polls
// of parked warps take issue slots from the warps that have work).
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t hint_ns)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}
// Bounded wait; after `limit_ns` records `code` in *err (unless an earlier code is there) and returns false.
// The clock is only looked at after a few hundred unsuccessful polls: reading %globaltimer takes far longer
// than a poll, and nearly every wait of a healthy kernel ends within the first handful.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t *err, uint32_t code,
                                          unsigned long long limit_ns = ASYNC_WAIT_NS)
{
#pragma unroll 1
    for (int i = 0; i < 512; i++)
        if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    do {
#pragma unroll 1
        for (int i = 0; i < 256; i++)
            if (mbar_try_wait(bar, parity)) return true;
    } while (global_ns() - t0 < limit_ns);
    if (err) atomicCAS(err, 0u, code);
    return false;
}
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

}  // namespace wgb
