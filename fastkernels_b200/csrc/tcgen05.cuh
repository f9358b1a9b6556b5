// Thin wrappers over the Blackwell tensor-core (tcgen05) and tiled TMA instructions used by the
// grouped GEMM: tensor-memory allocation, UMMA descriptors, MMA issue/commit, accumulator loads.
// sm_100a only.  No cluster-wide forms are used: every copy lands in the issuing block's own
// shared memory and every barrier is block-local.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "tma.cuh"

namespace fk {

// ---- tiled TMA load of a [rows x 64 columns] bf16 box (128-byte swizzle) --------------------------
__device__ __forceinline__ void tma_load_2d(void* dst_smem, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst_smem)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst_smem, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(dst_smem)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
        : "memory");
}
// The same copies with an L2 eviction hint (l2_evict_first_policy(): weights are read once per call).
__device__ __forceinline__ void tma_load_2d_hint(void* dst_smem, const CUtensorMap* map, int x, int y, uint64_t* bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
        ::"r"(smem_u32(dst_smem)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d_hint(void* dst_smem, const CUtensorMap* map, int x, int y, int z, uint64_t* bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5}], [%2], %6;"
        ::"r"(smem_u32(dst_smem)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---- tensor memory --------------------------------------------------------------------------------
// Whole-warp calls (.sync.aligned).  `cols` is a power of two >= 32.
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---- descriptors ----------------------------------------------------------------------------------
// Shared-memory operand, K-major, 128-byte swizzle: rows of 64 bf16 (128 B), 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t umma_smem_desc(const void* smem_ptr) {
    const uint64_t addr = (uint64_t)(smem_u32(smem_ptr) >> 4) & 0x3fffull;
    uint64_t d = addr;                      // start address            bits [0,14)
    d |= (uint64_t)1 << 16;                 // leading byte offset (unused for swizzled K-major) [16,30)
    d |= (uint64_t)(1024 >> 4) << 32;       // stride byte offset = 1024 B [32,46)
    d |= (uint64_t)1 << 46;                 // descriptor version of this architecture [46,48)
    d |= (uint64_t)2 << 61;                 // layout: 128-byte swizzle [61,64)
    return d;
}
// Instruction descriptor: bf16 x bf16 -> fp32, both operands K-major, M = 128, N = n (multiple of 16).
__device__ __forceinline__ uint32_t umma_idesc_bf16(uint32_t n) {
    return (1u << 4)                        // D format fp32
           | (1u << 7)                      // A format bf16
           | (1u << 10)                     // B format bf16
           | ((n >> 3) << 17)               // N >> 3
           | ((128u >> 4) << 24);           // M >> 4
}

// D[tmem] (+)= A[smem] * B[smem]^T, issued by one thread
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// mbarrier arrive when all MMAs issued so far by this thread have completed
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// 16 consecutive fp32 columns of this thread's accumulator lane
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Cached tensor map of a row-major bf16 matrix [rows, cols] with boxes of [box_rows, 64 columns] and
// 128-byte swizzle (tc_gemm.cu).  False when the driver's encoder is not available.
bool weight_tensor_map(const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, CUtensorMap* out);
bool column_pair_map(const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, CUtensorMap* out);
bool gate_up_pair_map(const void* base, uint64_t experts, uint64_t half_rows, uint64_t cols, uint32_t box_rows, CUtensorMap* out);

}  // namespace fk
