// Device helpers shared by the single-launch decode kernels (decode1.cu: one token; decode_few.cu: two to four).
#pragma once

#include "common.cuh"
#include "tma.cuh"

namespace fk {

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ unsigned ld_relaxed_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long ld_relaxed_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// tight wait on a latency-critical barrier (no back-off)
__device__ __forceinline__ bool mbar_wait_spin(uint64_t* bar, uint32_t parity, long long limit, volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) limit = min(limit, kWaitCyclesAfterAbort);
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - t0 > limit) { *abort_flag = 1; return false; }
    }
    return true;
}

__device__ __forceinline__ uint32_t d1_lds32(const void* smem_ptr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(smem_ptr)));
    return v;
}
__device__ __forceinline__ void d1_ldmatrix_x4(uint32_t (&r)[4], uint32_t smem_addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr));
}
__device__ __forceinline__ void d1_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// mbarrier arrive that cannot be scheduled before `dep` has been computed
__device__ __forceinline__ void d1_release(uint64_t* bar, float dep) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)), "f"(dep) : "memory");
}

__device__ __forceinline__ void d1_release_u(uint64_t* bar, uint32_t dep) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)), "r"(dep) : "memory");
}

// One [16 rows x 64 columns] box (128-byte swizzle, 2 KB, base 1 KB aligned) against 64 values of the token in
// column 0 of B: four k-steps of ldmatrix.x4 + MMA.  bfrag[kk] holds {b0, b1} of k-step kk (zero outside lanes 0..3).
// ldmatrix row address of a lane: matrices 0..3 = (rows 0-7, k 0-7), (rows 8-15, k 0-7), (rows 0-7, k 8-15),
// (rows 8-15, k 8-15); the 16-byte chunk c of row r sits at chunk c ^ (r & 7).
__device__ __forceinline__ void box_load(uint32_t (&a)[4][4], uint32_t box_addr, int lane) {
    const int row = (lane & 7) + ((lane >> 3) & 1) * 8;
    const uint32_t rbase = box_addr + row * 128;
    const int sel = lane >> 4, sw = row & 7;
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) d1_ldmatrix_x4(a[kk], rbase + (((2 * kk + sel) ^ sw) << 4));
}
// The shared-memory and MMA instructions are volatile asm statements and keep their program order, so callers write the
// loads of a box (or of several) out before the MMAs: a load that waits for the MMA before it made every k-step cost
// a full load latency.

}  // namespace fk
