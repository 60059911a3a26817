// mbarrier and bulk-copy wrappers shared by the kernels that stage data with the copy engine.
#pragma once

#include "qf_common.cuh"

namespace qf {

#ifdef __CUDACC__

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
template <int OFF>
__device__ __forceinline__ void mbar_arrive_at(uint32_t bar) {  // barrier at a constant offset from `bar`
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0+%1];" ::"r"(bar), "n"(OFF) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}

// Orders this thread's earlier shared-memory accesses made with ordinary loads and stores (generic proxy) before
// later accesses of the copy engine and the tensor cores (async proxy) to the same memory. Needed on both sides of a
// staging buffer: after writing data that the async proxy will read, and after reading data that it will overwrite.
__device__ __forceinline__ void fence_proxy_async_shared() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Bounded wait. Returns false on expiry or when another role aborted.
// A waiting warp backs off with nanosleep so that its polling does not take issue slots from the warps
// that convert; the sleep is short next to the time a pipeline step takes.
// The limit is longer than two exchange waits: with programmatic dependent launch a kernel starts while the
// previous kernel of the stream may still sit in a (legitimate, bounded) wait for a late peer GPU, and the
// early starter's own barriers cannot complete before that kernel has finished.
constexpr long long kWaitCycles = 2 * kExchangeWaitCycles + 1000000000LL;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    int it = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        __nanosleep(it < 8 ? 20 : 60);
        if ((++it & 63) == 0) {
            if (*abort_flag) return false;
            if (clock64() - t0 > kWaitCycles) {
                *abort_flag = 1;
                return false;
            }
        }
    }
}

// Untiled bulk copy global -> shared (16-byte aligned, size a multiple of 16), completion on an mbarrier.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

#endif  // __CUDACC__

}  // namespace qf
