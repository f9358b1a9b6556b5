// mbarrier and bulk-copy (TMA, untiled form) helpers with bounded waits.
//
// Every wait gives up after kWaitCycles, records a code in a caller-supplied error word and lets
// the caller carry on (with wrong numbers) instead of spinning forever; after the first time-out
// in a block all later waits of that block give up almost immediately.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace fk {

constexpr long long kWaitCycles = 2000000000LL;     // about one second of SM clocks
constexpr long long kWaitCyclesAfterAbort = 20000LL;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Non-blocking form: try_wait may suspend the thread for a hardware-chosen time when the phase is not complete,
// which a warp whose lanes watch different barriers pays on every poll; test_wait only looks.
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Returns false on time-out (and raises *abort_flag, a shared-memory word of the block).
// Waiting threads back off with nanosleep: a tight poll of a shared-memory barrier by whole warps
// competes with the shared-memory loads and shuffles of the warps that have work.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long limit = *abort_flag ? kWaitCyclesAfterAbort : kWaitCycles;
    const long long t0 = clock64();
    unsigned ns = 32;
    while (!mbar_try_wait(bar, parity)) {
        __nanosleep(ns);
        if (ns < 256) ns += ns;
        if (clock64() - t0 > limit) {
            *abort_flag = 1;
            return false;
        }
    }
    return true;
}

// Contiguous global -> shared copy of `bytes` (multiple of 16, both addresses 16-byte aligned);
// completion is signalled on `bar` as transaction bytes.
__device__ __forceinline__ void bulk_load(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// The same copy with an L2 eviction hint: the weight streams are read once per call and should not push what is read
// repeatedly (activation rows, pass lists, exchange words) out of L2.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void bulk_load_hint(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
                 : "memory");
}

// Named barrier for a subset of the block's warps.  bar.sync is an aligned instruction: every lane of a
// warp has to execute it together, and a warp counts as arrived as soon as it is executed at all.  Code
// that reaches the barrier after a divergent region (one lane polling a flag, say) must therefore
// reconverge first, or the barrier opens while that lane is still waiting.
__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    __syncwarp();
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ uint4 lds128(const void* smem_ptr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(smem_u32(smem_ptr)));
    return v;
}

}  // namespace fk
