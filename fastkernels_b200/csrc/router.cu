// Router: RMSNorm * (offset + w) -> GEMV over [E,H] -> (+bias) -> softmax -> top-k -> renormalise,
// plus the shared-expert gate sigmoid(g . x).  One launch.
//
// Grid (expert tiles, token tiles).  A block holds its tokens' activations in shared memory as
// fp32, computes one expert row per warp for all of them, and writes the logits.  The last block
// to finish a token tile (a self-resetting ticket in the workspace) runs softmax + top-k for those
// tokens, one warp per token, so no second launch and no spin-wait is needed.
//
// Reference semantics: src/fastkernels/reference/qwen36_real.py:23-28, :333-337; the Triton
// kernels this replaces are src/fastkernels/kernels/triton/qwen36_router.py:113-187.
// Tie rule: equal probabilities go to the LOWER expert index.

#include "common.cuh"
#include "kernels.cuh"
#include "tma.cuh"
#include "topk.cuh"

namespace fk {

constexpr int kRouterWarps = 8;

template <typename WT, int VW>
__device__ __forceinline__ void load_vec(const WT* p, float (&out)[VW]);

template <>
__device__ __forceinline__ void load_vec<float, 1>(const float* p, float (&o)[1]) { o[0] = *p; }
template <>
__device__ __forceinline__ void load_vec<__nv_bfloat16, 1>(const __nv_bfloat16* p, float (&o)[1]) { o[0] = __bfloat162float(*p); }
template <>
__device__ __forceinline__ void load_vec<__half, 1>(const __half* p, float (&o)[1]) { o[0] = __half2float(*p); }
template <>
__device__ __forceinline__ void load_vec<float, 4>(const float* p, float (&o)[4]) {
    float4 v = *reinterpret_cast<const float4*>(p);
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
}
template <>
__device__ __forceinline__ void load_vec<__nv_bfloat16, 8>(const __nv_bfloat16* p, float (&o)[8]) {
    uint4 v = *reinterpret_cast<const uint4*>(p);
    o[0] = bf16lo(v.x); o[1] = bf16hi(v.x); o[2] = bf16lo(v.y); o[3] = bf16hi(v.y);
    o[4] = bf16lo(v.z); o[5] = bf16hi(v.z); o[6] = bf16lo(v.w); o[7] = bf16hi(v.w);
}
template <>
__device__ __forceinline__ void load_vec<__half, 8>(const __half* p, float (&o)[8]) {
    uint4 v = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 f = __half22float2(h[i]);
        o[2 * i] = f.x; o[2 * i + 1] = f.y;
    }
}

template <typename WT, int VW, int TPB>
__global__ void __launch_bounds__(kRouterWarps * 32)
router_kernel(RouterParams p) {
    extern __shared__ float smem[];
    float* xs = smem;                         // [TPB][H]
    float* rstd = smem + (size_t)TPB * p.H;   // [TPB]
    __shared__ int is_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tok0 = blockIdx.y * TPB;
    const int H = p.H, E = p.E;
    pdl_trigger();
    pdl_wait();
    const WT* norm_w = reinterpret_cast<const WT*>(p.norm_weight);
    const WT* router_w = reinterpret_cast<const WT*>(p.router_weight);

    // The weight row of this warp does not depend on the activations: start its loads first.
    // Row E (when present) is the shared-expert gate vector: no norm scaling, sigmoid instead of a logit.
    const bool has_gate = p.shared_gate_weight != nullptr && p.shared_gate_out != nullptr;
    const int e = blockIdx.x * kRouterWarps + warp;
    const bool is_gate = has_gate && e == E;
    const bool active = e < E || is_gate;
    const WT* wrow = is_gate ? reinterpret_cast<const WT*>(p.shared_gate_weight) : router_w + (size_t)(active ? e : 0) * H;
    constexpr int PF = 4;                       // chunks of the row in flight per lane
    float wpre[PF][VW];
#pragma unroll
    for (int j = 0; j < PF; ++j) {
        const int h = (lane + j * 32) * VW;
        if (active && h < H) load_vec<WT, VW>(wrow + h, wpre[j]);
        else {
#pragma unroll
            for (int i = 0; i < VW; ++i) wpre[j][i] = 0.f;
        }
    }

    // activations -> shared memory as fp32 (vectorised when the layout allows), norm gains next to them
    float* gain = rstd + TPB;                   // [H]  (norm_offset + norm_weight)
    const bool vec_x = (VW > 1) && (H % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.hidden) & 15) == 0) && p.hidden_dtype != FK_F32;
    if (vec_x) {
        const int chunks = H / 8;
        for (int i = tid; i < TPB * chunks; i += blockDim.x) {
            const int t = i / chunks, c = i - t * chunks;
            const int token = tok0 + t;
            float v[8];
            if (token < p.T) {
                uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned short*>(p.hidden) + (size_t)token * H + c * 8);
                if (p.hidden_dtype == FK_BF16) {
                    v[0] = bf16lo(raw.x); v[1] = bf16hi(raw.x); v[2] = bf16lo(raw.y); v[3] = bf16hi(raw.y);
                    v[4] = bf16lo(raw.z); v[5] = bf16hi(raw.z); v[6] = bf16lo(raw.w); v[7] = bf16hi(raw.w);
                } else {
                    const __half2* hh = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
                    for (int q = 0; q < 4; ++q) { float2 f = __half22float2(hh[q]); v[2 * q] = f.x; v[2 * q + 1] = f.y; }
                }
            } else {
#pragma unroll
                for (int q = 0; q < 8; ++q) v[q] = 0.f;
            }
            float4* dst = reinterpret_cast<float4*>(xs + (size_t)t * H + c * 8);
            dst[0] = make_float4(v[0], v[1], v[2], v[3]);
            dst[1] = make_float4(v[4], v[5], v[6], v[7]);
        }
    } else {
        for (int i = tid; i < TPB * H; i += blockDim.x) {
            int t = i / H, h = i - t * H;
            int token = tok0 + t;
            xs[i] = token < p.T ? load_any(p.hidden, p.hidden_dtype, (size_t)token * H + h) : 0.f;
        }
    }
    for (int h = tid * VW; h < H; h += blockDim.x * VW) {
        float nw[VW];
        load_vec<WT, VW>(norm_w + h, nw);
#pragma unroll
        for (int i = 0; i < VW; ++i) gain[h + i] = p.norm_offset + nw[i];
    }
    __syncthreads();
    // mean square per token
    for (int t = warp; t < TPB; t += kRouterWarps) {
        float ss = 0.f;
#pragma unroll 8
        for (int h = lane; h < H; h += 32) ss += xs[t * H + h] * xs[t * H + h];
        ss = warp_sum(ss);
        if (lane == 0) rstd[t] = rsqrtf(ss / (float)H + p.eps);
    }
    __syncthreads();

    if (active) {
        float acc[TPB];
#pragma unroll
        for (int t = 0; t < TPB; ++t) acc[t] = 0.f;
        for (int h0 = lane * VW; h0 < H; h0 += PF * 32 * VW) {
            float wnext[PF][VW];
#pragma unroll
            for (int j = 0; j < PF; ++j) {          // next group of chunks in flight while this one is used
                const int h = h0 + (PF + j) * 32 * VW;
                if (h < H) load_vec<WT, VW>(wrow + h, wnext[j]);
                else {
#pragma unroll
                    for (int i = 0; i < VW; ++i) wnext[j][i] = 0.f;
                }
            }
#pragma unroll
            for (int j = 0; j < PF; ++j) {
                const int h = h0 + j * 32 * VW;
                if (h < H) {
                    float w[VW];
#pragma unroll
                    for (int i = 0; i < VW; ++i) w[i] = is_gate ? wpre[j][i] : wpre[j][i] * gain[h + i];
#pragma unroll
                    for (int t = 0; t < TPB; ++t) {
#pragma unroll
                        for (int i = 0; i < VW; ++i) acc[t] = fmaf(w[i], xs[t * H + h + i], acc[t]);
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < PF; ++j) {
#pragma unroll
                for (int i = 0; i < VW; ++i) wpre[j][i] = wnext[j][i];
            }
        }
#pragma unroll
        for (int t = 0; t < TPB; ++t) {
            float v = warp_sum(acc[t]);
            if (lane == 0 && tok0 + t < p.T) {
                if (is_gate) {
                    p.shared_gate_out[tok0 + t] = sigmoidf_(v);
                } else {
                    float logit = v * rstd[t];
                    if (p.router_bias) logit += p.router_bias[e];
                    p.logits[(size_t)(tok0 + t) * E + e] = logit;
                }
            }
        }
    }

    // ticket: the last expert-tile block of this token tile selects the top-k
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        unsigned t = atomicAdd(p.tickets + blockIdx.y, 1u);
        is_last = (t == gridDim.x - 1);
        if (is_last) p.tickets[blockIdx.y] = 0u;    // re-arm for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (int t = warp; t < TPB; t += kRouterWarps) {
        int token = tok0 + t;
        if (token >= p.T) continue;
        const float* row = p.logits + (size_t)token * E;
        long long* ids = p.topk_ids + (size_t)token * p.top_k;
        int* ids32 = p.ids32 ? p.ids32 + (size_t)token * p.top_k : nullptr;
        float* wts = p.topk_weights + (size_t)token * p.top_k;
        if (E <= 256) topk_warp<8>(row, E, p.top_k, ids, ids32, wts);
        else topk_warp<32>(row, E, p.top_k, ids, ids32, wts);
    }
}

// bf16 fast path: every warp's weight row is bulk-copied (TMA, untiled form) into shared memory at
// kernel start, all rows in flight together, and the dot products are short rolled loops over 16-byte
// shared-memory vectors.  A kernel this short is bound by instruction fetch and load latency, so the
// code is kept small on purpose.  H must be a multiple of 256.
// XB: the activations are bf16 and stay bf16 in shared memory (half the space, so a block can hold 32
// tokens and amortise each weight row over all of them); otherwise they are widened to fp32.
template <int TPB, bool XB>
__global__ void __launch_bounds__(kRouterWarps * 32) router_fast_kernel(RouterParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int H = p.H, E = p.E;
    __nv_bfloat16* wrows = reinterpret_cast<__nv_bfloat16*>(smem_raw);                 // [8][H]
    constexpr int XE = XB ? 2 : 4;                                                    // bytes per stored activation
    unsigned char* xs_raw = smem_raw + (size_t)kRouterWarps * H * 2;                  // [TPB][H] bf16 or fp32
    float* xs = reinterpret_cast<float*>(xs_raw);
    float* gain = reinterpret_cast<float*>(xs_raw + (size_t)TPB * H * XE);            // [H]
    float* rstd = gain + H;                                                           // [TPB]
    uint64_t* bars = reinterpret_cast<uint64_t*>(rstd + TPB + (TPB & 1));             // [8]
    __shared__ int is_last;
    __shared__ int abort_flag;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tok0 = blockIdx.y * TPB;
    pdl_trigger();
    pdl_wait();
    const bool has_gate = p.shared_gate_weight != nullptr && p.shared_gate_out != nullptr;
    const int e = blockIdx.x * kRouterWarps + warp;
    const bool is_gate = has_gate && e == E;
    const bool active = e < E || is_gate;
    if (tid == 0) abort_flag = 0;
    // Each warp's barrier covers its weight row and, when the activations stay bf16, the rows of the
    // tokens whose mean square the warp takes: all copies of the block are in flight at once.
    if (lane == 0) {
        mbar_init(&bars[warp], 1);
        mbar_init_fence();
        uint32_t bytes = active ? (uint32_t)H * 2 : 0u;
        if (XB)
            for (int t = warp; t < TPB; t += kRouterWarps)
                if (tok0 + t < p.T) bytes += (uint32_t)H * 2;
        mbar_expect_tx(&bars[warp], bytes);
        if (active) {
            const __nv_bfloat16* wrow = is_gate ? reinterpret_cast<const __nv_bfloat16*>(p.shared_gate_weight)
                                                : reinterpret_cast<const __nv_bfloat16*>(p.router_weight) + (size_t)e * H;
            bulk_load(wrows + (size_t)warp * H, wrow, (uint32_t)H * 2, &bars[warp]);
        }
        if (XB)
            for (int t = warp; t < TPB; t += kRouterWarps)
                if (tok0 + t < p.T)
                    bulk_load(xs_raw + (size_t)t * H * 2, reinterpret_cast<const __nv_bfloat16*>(p.hidden) + (size_t)(tok0 + t) * H,
                              (uint32_t)H * 2, &bars[warp]);
    }
    // activations -> fp32 in shared memory; norm gains next to them
    const int chunks = H / 8;
    for (int i = tid; i < (XB ? 0 : TPB * chunks); i += blockDim.x) {
        const int t = i / chunks, c = i - t * chunks;
        const int token = tok0 + t;
        float v[8];
        if (token < p.T) {
            if (p.hidden_dtype == FK_BF16) {
                const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.hidden) + (size_t)token * H + c * 8);
                v[0] = bf16lo(raw.x); v[1] = bf16hi(raw.x); v[2] = bf16lo(raw.y); v[3] = bf16hi(raw.y);
                v[4] = bf16lo(raw.z); v[5] = bf16hi(raw.z); v[6] = bf16lo(raw.w); v[7] = bf16hi(raw.w);
            } else {
#pragma unroll
                for (int q = 0; q < 8; ++q) v[q] = load_any(p.hidden, p.hidden_dtype, (size_t)token * H + c * 8 + q);
            }
        } else {
#pragma unroll
            for (int q = 0; q < 8; ++q) v[q] = 0.f;
        }
        float4* dst = reinterpret_cast<float4*>(xs + (size_t)t * H + c * 8);
        dst[0] = make_float4(v[0], v[1], v[2], v[3]);
        dst[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
    for (int c = tid; c < chunks; c += blockDim.x) {
        const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.norm_weight) + c * 8);
        const float o = p.norm_offset;
        float4* dst = reinterpret_cast<float4*>(gain + c * 8);
        dst[0] = make_float4(o + bf16lo(raw.x), o + bf16hi(raw.x), o + bf16lo(raw.y), o + bf16hi(raw.y));
        dst[1] = make_float4(o + bf16lo(raw.z), o + bf16hi(raw.z), o + bf16lo(raw.w), o + bf16hi(raw.w));
    }
    __syncthreads();
    if (XB) mbar_wait(&bars[warp], 0, &abort_flag);     // this warp's rows (and its weight row) have landed
    for (int t = warp; t < TPB; t += kRouterWarps) {
        float ss = 0.f;
        if (XB) {
#pragma unroll 2
            for (int h = lane * 8; h < H; h += 256) {
                const uint4 v = *reinterpret_cast<const uint4*>(xs_raw + ((size_t)t * H + h) * 2);
                float f;
                f = bf16lo(v.x); ss = fmaf(f, f, ss); f = bf16hi(v.x); ss = fmaf(f, f, ss);
                f = bf16lo(v.y); ss = fmaf(f, f, ss); f = bf16hi(v.y); ss = fmaf(f, f, ss);
                f = bf16lo(v.z); ss = fmaf(f, f, ss); f = bf16hi(v.z); ss = fmaf(f, f, ss);
                f = bf16lo(v.w); ss = fmaf(f, f, ss); f = bf16hi(v.w); ss = fmaf(f, f, ss);
            }
        } else {
#pragma unroll 4
            for (int h = lane * 4; h < H; h += 128) {
                const float4 v = *reinterpret_cast<const float4*>(xs + (size_t)t * H + h);
                ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
            }
        }
        ss = warp_sum(ss);
        if (lane == 0) rstd[t] = rsqrtf(ss / (float)H + p.eps);
    }
    __syncthreads();

    if (active) {
        if (!XB) mbar_wait(&bars[warp], 0, &abort_flag);
        float acc[TPB];
#pragma unroll
        for (int t = 0; t < TPB; ++t) acc[t] = 0.f;
        const unsigned char* wrow = reinterpret_cast<const unsigned char*>(wrows + (size_t)warp * H);
#pragma unroll 1
        for (int c = lane * 8; c < H; c += 256) {
            const uint4 w = lds128(wrow + (size_t)c * 2);
            float wf[8];
            wf[0] = bf16lo(w.x); wf[1] = bf16hi(w.x); wf[2] = bf16lo(w.y); wf[3] = bf16hi(w.y);
            wf[4] = bf16lo(w.z); wf[5] = bf16hi(w.z); wf[6] = bf16lo(w.w); wf[7] = bf16hi(w.w);
            if (!is_gate) {
                const float4 g0 = *reinterpret_cast<const float4*>(gain + c), g1 = *reinterpret_cast<const float4*>(gain + c + 4);
                wf[0] *= g0.x; wf[1] *= g0.y; wf[2] *= g0.z; wf[3] *= g0.w;
                wf[4] *= g1.x; wf[5] *= g1.y; wf[6] *= g1.z; wf[7] *= g1.w;
            }
#pragma unroll
            for (int t = 0; t < TPB; ++t) {
                float4 x0, x1;
                if (XB) {
                    const uint4 xv = *reinterpret_cast<const uint4*>(xs_raw + ((size_t)t * H + c) * 2);
                    x0 = make_float4(bf16lo(xv.x), bf16hi(xv.x), bf16lo(xv.y), bf16hi(xv.y));
                    x1 = make_float4(bf16lo(xv.z), bf16hi(xv.z), bf16lo(xv.w), bf16hi(xv.w));
                } else {
                    x0 = *reinterpret_cast<const float4*>(xs + (size_t)t * H + c);
                    x1 = *reinterpret_cast<const float4*>(xs + (size_t)t * H + c + 4);
                }
                float a = acc[t];
                a = fmaf(wf[0], x0.x, a); a = fmaf(wf[1], x0.y, a); a = fmaf(wf[2], x0.z, a); a = fmaf(wf[3], x0.w, a);
                a = fmaf(wf[4], x1.x, a); a = fmaf(wf[5], x1.y, a); a = fmaf(wf[6], x1.z, a); a = fmaf(wf[7], x1.w, a);
                acc[t] = a;
            }
        }
#pragma unroll
        for (int t = 0; t < TPB; ++t) {
            const float v = warp_sum(acc[t]);
            if (lane == 0 && tok0 + t < p.T) {
                if (is_gate) {
                    p.shared_gate_out[tok0 + t] = sigmoidf_(v);
                } else {
                    float logit = v * rstd[t];
                    if (p.router_bias) logit += p.router_bias[e];
                    p.logits[(size_t)(tok0 + t) * E + e] = logit;
                }
            }
        }
    }

    // ticket: the last expert-tile block of this token tile selects the top-k
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        unsigned t = atomicAdd(p.tickets + blockIdx.y, 1u);
        is_last = (t == gridDim.x - 1);
        if (is_last) p.tickets[blockIdx.y] = 0u;    // re-arm for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (int t = warp; t < TPB; t += kRouterWarps) {
        const int token = tok0 + t;
        if (token >= p.T) continue;
        const float* row = p.logits + (size_t)token * E;
        long long* ids = p.topk_ids + (size_t)token * p.top_k;
        int* ids32 = p.ids32 ? p.ids32 + (size_t)token * p.top_k : nullptr;
        float* wts = p.topk_weights + (size_t)token * p.top_k;
        if (E <= 256) topk_warp<8>(row, E, p.top_k, ids, ids32, wts);
        else topk_warp<32>(row, E, p.top_k, ids, ids32, wts);
    }
}

template <int TPB, bool XB>
static int launch_router_fast(const RouterParams& p, cudaStream_t stream) {
    const int gate = (p.shared_gate_weight && p.shared_gate_out) ? 1 : 0;
    dim3 grid((p.E + gate + kRouterWarps - 1) / kRouterWarps, (p.T + TPB - 1) / TPB);
    const size_t smem = (size_t)kRouterWarps * p.H * 2 + (size_t)TPB * p.H * (XB ? 2 : 4) + sizeof(float) * ((size_t)p.H + TPB + 2) + 8 * sizeof(uint64_t) + 16;
    auto kern = router_fast_kernel<TPB, XB>;
    FK_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "router attr");
    FK_CUDA_OK(launch_pdl(kern, grid, dim3(kRouterWarps * 32), smem, stream, p), "router launch");
    FK_LAUNCH_OK("router launch");
    return FK_OK;
}

template <typename WT, int VW>
static int launch_router_t(const RouterParams& p, cudaStream_t stream) {
    dim3 block(kRouterWarps * 32);
    if (p.T <= 64) {
        constexpr int TPB = 4;
        size_t smem = sizeof(float) * ((size_t)TPB * p.H + TPB + p.H);
        dim3 grid((p.E + (p.shared_gate_weight && p.shared_gate_out ? 1 : 0) + kRouterWarps - 1) / kRouterWarps, (p.T + TPB - 1) / TPB);
        auto kern = router_kernel<WT, VW, TPB>;
        FK_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "router attr");
        FK_CUDA_OK(launch_pdl(kern, grid, block, smem, stream, p), "router launch");
    } else {
        constexpr int TPB = 8;
        size_t smem = sizeof(float) * ((size_t)TPB * p.H + TPB + p.H);
        dim3 grid((p.E + (p.shared_gate_weight && p.shared_gate_out ? 1 : 0) + kRouterWarps - 1) / kRouterWarps, (p.T + TPB - 1) / TPB);
        auto kern = router_kernel<WT, VW, TPB>;
        FK_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "router attr");
        FK_CUDA_OK(launch_pdl(kern, grid, block, smem, stream, p), "router launch");
    }
    FK_LAUNCH_OK("router launch");
    return FK_OK;
}

int launch_router(const RouterParams& p, int weight_dtype, cudaStream_t stream) {
    if (p.T <= 0) return FK_OK;
    if ((p.T + 3) / 4 > kMaxTokenTiles) return FK_ERR_ARG;
    const bool aligned = ((reinterpret_cast<uintptr_t>(p.router_weight) | reinterpret_cast<uintptr_t>(p.norm_weight)) & 15) == 0;
    switch (weight_dtype) {
        case FK_F32:
            return (aligned && p.H % 4 == 0) ? launch_router_t<float, 4>(p, stream) : launch_router_t<float, 1>(p, stream);
        case FK_BF16:
            if (aligned && p.H % 256 == 0 && p.H <= 4096 && ((reinterpret_cast<uintptr_t>(p.hidden) | reinterpret_cast<uintptr_t>(p.shared_gate_weight)) & 15) == 0)
            {
                // 32 bf16 tokens per block from 32 tokens up; small batches keep 4-token blocks for parallelism
                // tokens per block grow with the batch so that the grid stays near two blocks per SM
                if (p.hidden_dtype == FK_BF16) {
                    if (p.T <= 32) return launch_router_fast<4, true>(p, stream);
                    if (p.T <= 64) return launch_router_fast<8, true>(p, stream);
                    if (p.T <= 128) return launch_router_fast<16, true>(p, stream);
                    return launch_router_fast<32, true>(p, stream);
                }
                return p.T <= 64 ? launch_router_fast<4, false>(p, stream) : launch_router_fast<8, false>(p, stream);
            }
            return (aligned && p.H % 8 == 0) ? launch_router_t<__nv_bfloat16, 8>(p, stream)
                                             : launch_router_t<__nv_bfloat16, 1>(p, stream);
        case FK_F16:
            return (aligned && p.H % 8 == 0) ? launch_router_t<__half, 8>(p, stream) : launch_router_t<__half, 1>(p, stream);
        default:
            return FK_ERR_UNSUPPORTED;
    }
}

}  // namespace fk

// ---------------------------------------------------------------------------------------------
// Router without caller-provided scratch (fk_moe_router_noalloc)
// ---------------------------------------------------------------------------------------------
// The router's only scratch is its "last block" tickets.  Here they live in a fixed array inside the
// library image instead of the caller's workspace, so a caller that cannot allocate device memory
// (and therefore has no workspace to hand over) can still route tokens.
namespace fk {

constexpr int kNoAllocTicketSlots = 1024;      // 4 KB per device; one slot per token tile
static __device__ __align__(256) unsigned g_noalloc_tickets[kNoAllocTicketSlots];

// Device address of the array for the current device.  In host code the symbol's name is only a
// handle; the address a kernel can use has to be asked for, once per device, with that device current.
static int noalloc_tickets(unsigned** out) {
    static unsigned* cached[64] = {nullptr};
    int dev = 0;
    FK_CUDA_OK(cudaGetDevice(&dev), "noalloc get device");
    if (dev < 0 || dev >= 64) return FK_ERR_UNSUPPORTED;
    if (cached[dev] == nullptr) {
        unsigned* ptr = nullptr;
        FK_CUDA_OK(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_tickets), "noalloc symbol address");
        if (ptr == nullptr) return FK_ERR_CUDA;
        cached[dev] = ptr;
    }
    *out = cached[dev];
    return FK_OK;
}

int launch_router_noalloc(RouterParams p, int weight_dtype, cudaStream_t stream) {
    const int tpb = 4;                                       // fewest tokens per block launch_router may pick
    if ((p.T + tpb - 1) / tpb > kNoAllocTicketSlots) return FK_ERR_ARG;
    unsigned* tickets = nullptr;
    int st = noalloc_tickets(&tickets);
    if (st != FK_OK) return st;
    // every call shares the array and finds what the previous call left: start from zero
    FK_CUDA_OK(cudaMemsetAsync(tickets, 0, sizeof(unsigned) * kNoAllocTicketSlots, stream), "noalloc ticket clear");
    p.tickets = tickets;
    return launch_router(p, weight_dtype, stream);
}

}  // namespace fk
