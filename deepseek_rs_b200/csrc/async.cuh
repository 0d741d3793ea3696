// mbarrier + bulk asynchronous copy (TMA, untiled form) helpers for sm_100a. Every wait is bounded.
#pragma once

#include <stdint.h>

namespace dsmoe {

// Device-side error codes written to the handle's status word (first error wins).
constexpr int DEV_ERR_MBAR_TIMEOUT = 1;
constexpr int DEV_ERR_INDEX_RANGE = 2;  // checked build only: an expert index outside [.., n_expert) was replaced by 0

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

// Makes mbarrier initialisation and earlier generic-proxy shared-memory accesses visible to the async proxy.
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

// Untiled bulk copy global -> shared, completion counted in bytes on the mbarrier. Source and destination must be
// 16-byte aligned and the size a multiple of 16. Never multicast.
__device__ __forceinline__ void bulk_g2s(void *dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// One arrival on the mbarrier (release semantics at CTA scope).
__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Named barrier `id` over the first `nthreads` arrivals (a multiple of 32), returning the AND of every participant's
// predicate. All participating warps must call it the same number of times.
__device__ __forceinline__ bool named_barrier_and(uint32_t id, uint32_t nthreads, bool pred)
{
    uint32_t r;
    asm volatile(
        "{\n"
        ".reg .pred p, q;\n"
        "setp.ne.b32 q, %3, 0;\n"
        "bar.red.and.pred p, %1, %2, q;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(r)
        : "r"(id), "r"(nthreads), "r"((uint32_t)pred)
        : "memory");
    return r != 0;
}

// Named barrier `id` over `nthreads` threads (a multiple of 32), no reduction.
__device__ __forceinline__ void named_barrier_sync(uint32_t id, uint32_t nthreads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// Programmatic dependent launch. A kernel launched with the programmatic-serialisation attribute may start while the
// kernel before it in the stream is still running; pdl_wait() blocks until that kernel (and, transitively, everything
// before it, as every kernel of a chain waits) has completed and its writes are visible. Before the wait a kernel may
// only do work that touches no global data of its predecessors (shared-memory tables, barrier set-up).
// pdl_launch_dependents() lets the next kernel's CTAs be scheduled early. Both do nothing in a plain launch.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
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

// The status block every bounded-wait kernel receives: four ints in device memory.
//   [0] first device-side error code (0 = none); kernels only ever change it from 0
//   [1] wait limit in units of 1024 SM clocks; 0 = the default of about two seconds
//   [2] test hook: non-zero makes down_m8_tma_kernel leave one of its copies out, so that a wait runs out
//   [3] unused
constexpr int STATUS_WORDS = 4;
constexpr long long DEFAULT_WAIT_CLOCKS = 4000000000LL;

// Waits for the given phase with a time limit (status[1], default about two seconds of SM clocks). On expiry records
// DEV_ERR_MBAR_TIMEOUT in status[0] (if it was still 0) and returns false; the caller stops using the buffer.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity, int *status)
{
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    long long limit = DEFAULT_WAIT_CLOCKS;
    if (status) {
        const int kclk = *reinterpret_cast<volatile int *>(status + 1);
        if (kclk > 0) limit = (long long)kclk << 10;
    }
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - t0 > limit) {
            if (status) atomicCAS(status, 0, DEV_ERR_MBAR_TIMEOUT);
            return false;
        }
    }
    return true;
}

}  // namespace dsmoe
