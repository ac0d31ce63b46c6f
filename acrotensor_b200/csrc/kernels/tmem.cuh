// Tensor memory (TMEM, 256 KB per SM on sm_100a) used as a software-managed operand store.
//
// TMEM is the on-chip memory the fifth-generation tensor cores accumulate into.  Those tensor cores
// have no fp64 kind, but the memory itself can be allocated, written and read from registers
// (tcgen05.alloc / st / ld), through a path of its own that does not go through the shared-memory
// pipe.  The fp64 kernels here use it to park operand fragments that are the same for every tile of
// a launch and too large for the register file.
//
// Geometry: 128 lanes x 512 columns of 32 bits.  Warp w of a CTA reaches lanes 32*(w%4) .. +31 only;
// with the 32x32b shape, lane i of the warp reads or writes N consecutive columns of TMEM lane
// 32*(w%4) + i.  An address is (lane << 16) | column.
//
// Rules kept by every user: one warp allocates (a power of two >= 32 columns) and the same warp frees
// before the CTA ends, on every path; a kernel that allocates runs one CTA per SM, so the allocation
// cannot wait for columns held by a CTA that is waiting for this one.
#ifndef ACRO_B200_KERNELS_TMEM_CUH
#define ACRO_B200_KERNELS_TMEM_CUH

#include <cstdint>
#include "tma.cuh"

namespace acro_b200_detail
{

// Executed by all 32 lanes of ONE warp.  The allocation's base address is written to *slot (shared memory).
__device__ __forceinline__ void tmem_alloc(uint32_t *slot, uint32_t columns)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(slot)), "r"(columns) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

// Executed by all 32 lanes of the warp that allocated.
__device__ __forceinline__ void tmem_free(uint32_t base, uint32_t columns)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
}

// Order TMEM accesses with a following / preceding thread synchronisation (barrier).
__device__ __forceinline__ void tmem_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_wait_loads() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_stores() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Two doubles (four columns) of this lane.
__device__ __forceinline__ void tmem_store_2(uint32_t addr, double a, double b)
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(__double2loint(a)), "r"(__double2hiint(a)),
                 "r"(__double2loint(b)), "r"(__double2hiint(b))
                 : "memory");
}

// Four doubles (eight columns) of this lane; complete after tmem_wait_loads().
__device__ __forceinline__ void tmem_load_4(uint32_t addr, uint32_t (&r)[8])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(addr)
                 : "memory");
}

// Two doubles (four columns) of this lane; complete after tmem_wait_loads().
__device__ __forceinline__ void tmem_load_2(uint32_t addr, uint32_t (&r)[4])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}

__device__ __forceinline__ double tmem_double(uint32_t lo, uint32_t hi) { return __hiloint2double(static_cast<int>(hi), static_cast<int>(lo)); }

// CTA-local named barrier over `threads` threads (a multiple of 32); id 1..15 (0 is __syncthreads).
__device__ __forceinline__ void named_barrier(int id, int threads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory"); }
// One-way use of a named barrier: `threads` counts the arriving and the waiting threads together; the arriving
// threads do not block.
__device__ __forceinline__ void named_barrier_arrive(int id, int threads) { asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(threads) : "memory"); }

}

#endif
