// Shared device helpers and the workspace layout of libfkmoe.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fkmoe.h"

namespace fk {

constexpr int kWarp = 32;
constexpr unsigned kFull = 0xffffffffu;
constexpr int kMaxTokenTiles = 4096;   // ticket slots in the workspace

// ---------------------------------------------------------------------------------------------
// Workspace layout.  All offsets are multiples of 256 bytes.
// ---------------------------------------------------------------------------------------------
struct Workspace {
    size_t tickets;      // u32 [kMaxTokenTiles]   router "last block" tickets (self-resetting)
    size_t counters;     // u32 [64]               misc. counters / barrier words (self-resetting)
    size_t meta;         // i32 [16]               [0]=U distinct experts hit, [1]=GEMV pass count, [2]=error word
    size_t tagged;       // u64 [FK_MAX_EXPERTS + (FK_MAX_TOP_K + 1) * FK_MAX_INTERMEDIATE + 8]   single-token kernel:
                         //     (launch tag << 32 | payload) words: the logits, then the SwiGLU activations, then the gate
    size_t ids32;        // i32 [R]
    size_t counts;       // i32 [E]
    size_t offsets;      // i32 [E+1]
    size_t touched;      // i32 [E+1]   ascending list of experts with count>0
    size_t order;        // i32 [R]     packed row -> route (token*k+slot)
    size_t inv;          // i32 [R]     route -> packed row
    size_t passes;       // int4 [R+T+1]  GEMV pass list: (expert or -1 for shared, first packed row, rows<=4, first token)
    size_t shared_gate;  // f32 [T]
    size_t act;          // f32 [(R+T), I]  SwiGLU activations per packed row (+ shared rows)
    size_t y;            // f32 [(R+T), H]  un-weighted expert outputs per packed row
    size_t xg;           // bf16 [Rpad+T16, H] gathered rows for the tensor-core path
    size_t actb;         // bf16 [Rpad+T16, I]
    size_t total;
};

__host__ __device__ inline size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

// Rows of the padded (16-row tiles) packed layout: every expert group rounded up to 16.
__host__ __device__ inline size_t padded_rows(size_t routes, size_t experts) {
    size_t worst = routes + 15 * (routes < experts ? routes : experts);
    return (worst + 15) / 16 * 16;
}

__host__ inline Workspace workspace_layout(const fk_moe_dims& d) {
    Workspace w{};
    size_t T = d.tokens, H = d.hidden, E = d.experts, I = d.intermediate, k = d.top_k;
    size_t R = T * k;
    size_t rows = R + T;
    size_t rpad = padded_rows(R, E) + (T + 15) / 16 * 16;
    size_t o = 0;
    auto take = [&](size_t bytes) { size_t at = o; o = align256(o + bytes); return at; };
    w.tickets = take(sizeof(uint32_t) * kMaxTokenTiles);
    w.counters = take(sizeof(uint32_t) * 64);
    w.meta = take(sizeof(int32_t) * 16);
    w.tagged = take(sizeof(uint64_t) * (FK_MAX_EXPERTS + (FK_MAX_TOP_K + 1) * FK_MAX_INTERMEDIATE + 8));
    w.ids32 = take(sizeof(int32_t) * R);
    w.counts = take(sizeof(int32_t) * E);
    w.offsets = take(sizeof(int32_t) * (E + 1));
    w.touched = take(sizeof(int32_t) * (E + 1));
    w.order = take(sizeof(int32_t) * R);
    w.inv = take(sizeof(int32_t) * R);
    w.passes = take(sizeof(int32_t) * 4 * (R + T + 1));
    w.shared_gate = take(sizeof(float) * T);
    w.act = take(sizeof(float) * rows * I);
    w.y = take(sizeof(float) * rows * H);
    w.xg = take(sizeof(__nv_bfloat16) * rpad * H);
    w.actb = take(sizeof(__nv_bfloat16) * rpad * I);
    w.total = o;
    return w;
}

// ---------------------------------------------------------------------------------------------
// Typed loads
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_float(__half v) { return __half2float(v); }

// Element `i` of an array whose dtype is only known at run time.
__device__ __forceinline__ float load_any(const void* p, int dtype, size_t i) {
    if (dtype == FK_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
    if (dtype == FK_F16) return __half2float(reinterpret_cast<const __half*>(p)[i]);
    return reinterpret_cast<const float*>(p)[i];
}

// Two bf16 packed in a 32-bit word -> two floats (exact: bf16 is the top half of an fp32).
__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// 16-byte streaming load that does not pollute L1 (weights are read once).
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFull, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(kFull, v, o));
    return v;
}

// Programmatic dependent launch: a kernel launched with launch_pdl() may become resident while the
// kernel before it in the stream is still draining.  It must call pdl_wait() before it touches global
// memory (the wait returns once the previous grid has completed and its writes are visible);
// pdl_trigger() lets the next kernel in the stream start its own prologue early.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.0f + expf(-g)) * u; }
__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

}  // namespace fk

// ---------------------------------------------------------------------------------------------
// Host-side error plumbing
// ---------------------------------------------------------------------------------------------
namespace fk {
void note_cuda_error(cudaError_t e, const char* where);
void note_launch();
// Optional per-stage timing hook: when set, stage_mark(i) records event i on the stream.
struct StageTimer {
    cudaEvent_t ev[12];
    int used;
    cudaStream_t stream;
};
extern thread_local StageTimer* g_stage_timer;
inline void stage_mark() {
    if (g_stage_timer && g_stage_timer->used < 12) {
        cudaEventRecord(g_stage_timer->ev[g_stage_timer->used], g_stage_timer->stream);
        g_stage_timer->used++;
    }
}
}
#define FK_CUDA_OK(expr, where)                          \
    do {                                                 \
        cudaError_t e__ = (expr);                        \
        if (e__ != cudaSuccess) {                        \
            fk::note_cuda_error(e__, where);             \
            return FK_ERR_CUDA;                          \
        }                                                \
    } while (0)
namespace fk {
bool pdl_enabled();
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}
}  // namespace fk

#define FK_LAUNCH_OK(where)                              \
    do {                                                 \
        fk::note_launch();                               \
        FK_CUDA_OK(cudaPeekAtLastError(), where);        \
    } while (0)
