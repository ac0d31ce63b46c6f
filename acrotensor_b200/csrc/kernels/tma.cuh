// Thin wrappers over the sm_100a asynchronous bulk-copy (TMA) and mbarrier instructions
// used to stream contiguous operand spans between global and shared memory.
//
// Rules kept by every caller: both addresses 16-byte aligned and the size a multiple of
// 16 bytes; copies are CTA-local and unicast (no cluster multicast anywhere); every wait
// is bounded and reports through a flag instead of spinning forever.
#ifndef ACRO_B200_KERNELS_TMA_CUH
#define ACRO_B200_KERNELS_TMA_CUH

#include <cstdint>
#include <cuda_runtime.h>

namespace acro_b200_detail
{

__device__ __forceinline__ uint32_t smem_addr(const void *p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t arrivals)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals) : "memory");
}

// Makes mbarrier initialisation visible to the asynchronous proxy.
__device__ __forceinline__ void fence_mbar_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Orders this thread's generic-proxy shared-memory accesses before later async-proxy ones.
__device__ __forceinline__ void fence_proxy_async()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// One arrival that also announces `bytes` of asynchronous copies still to complete.
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return done != 0;
}

// Bounded wait for the phase with the given parity.  Returns false when the limit ran out: about a second
// (2e9 cycles of the SM's own counter, which is cheap to read; a try_wait blocks for a hardware-defined
// interval of its own, so a count of tries alone bounds nothing that can be relied on), or max_tries,
// whichever comes first.  The counter is read only after a first try has failed and then every sixteenth try.
constexpr long long kMbarWaitLimitCycles = 2000000000ll;

__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, uint32_t max_tries = 1u << 22)
{
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    for (uint32_t i = 0; i < max_tries; ++i)
    {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 15u) == 15u && clock64() - start > kMbarWaitLimitCycles) return false;
    }
    return false;
}

// The same wait bounded by the number of tries alone.  Kept for the one kernel whose register allocation
// (and with it 13 % of its speed) changed when the clock came into its waits.
__device__ __forceinline__ bool mbar_wait_counted(uint64_t *bar, uint32_t parity, uint32_t max_tries = 1u << 22)
{
    for (uint32_t i = 0; i < max_tries; ++i)
    {
        if (mbar_try_wait(bar, parity)) return true;
    }
    return false;
}

// global -> shared, completion counted in bytes on `bar`.
__device__ __forceinline__ void bulk_load(void *smem_dst, const void *gmem_src, uint32_t bytes, uint64_t *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_addr(smem_dst)),
                 "l"(gmem_src), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}

// shared -> global, tracked by the issuing thread's bulk async-group.
__device__ __forceinline__ void bulk_store(void *gmem_dst, const void *smem_src, uint32_t bytes)
{
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst), "r"(smem_addr(smem_src)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }

// Waits until at most N of this thread's bulk groups still READ their shared-memory source.
template <int N>
__device__ __forceinline__ void bulk_wait_read()
{
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// Waits until at most N of this thread's bulk groups are still in flight at all.
template <int N>
__device__ __forceinline__ void bulk_wait_all()
{
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

}

#endif
