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

#include <atomic>

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
        long long* ids2 = p.ids_mirror ? p.ids_mirror + (size_t)token * p.top_k : nullptr;
        float* wts2 = p.weights_mirror ? p.weights_mirror + (size_t)token * p.top_k : nullptr;
        if (E <= 256) topk_warp<8>(row, E, p.top_k, ids, ids32, wts, wts2, ids2);
        else topk_warp<32>(row, E, p.top_k, ids, ids32, wts, wts2, ids2);
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
    unsigned char* nwraw = reinterpret_cast<unsigned char*>(bars + kRouterWarps);     // [H] bf16 norm weights as stored
    __shared__ int is_last;
    __shared__ int abort_flag;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tok0 = blockIdx.y * TPB;
    pdl_trigger();
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
        if (warp == 0) bytes += (uint32_t)H * 2;     // the norm weights ride on warp 0's barrier
        if (XB)
            for (int t = warp; t < TPB; t += kRouterWarps)
                if (tok0 + t < p.T) bytes += (uint32_t)H * 2;
        mbar_expect_tx(&bars[warp], bytes);
        if (active) {
            // weights are constants: their copy starts while the kernel before this one is still draining
            const __nv_bfloat16* wrow = is_gate ? reinterpret_cast<const __nv_bfloat16*>(p.shared_gate_weight)
                                                : reinterpret_cast<const __nv_bfloat16*>(p.router_weight) + (size_t)e * H;
            bulk_load(wrows + (size_t)warp * H, wrow, (uint32_t)H * 2, &bars[warp]);
        }
        // one copy per block: per-thread loads of the same 4 KB from hundreds of blocks queue up on a few L2 lines
        if (warp == 0) bulk_load(nwraw, p.norm_weight, (uint32_t)H * 2, &bars[0]);
        pdl_wait();           // the activations (and the tickets) may come from the kernel before
        if (XB)
            for (int t = warp; t < TPB; t += kRouterWarps)
                if (tok0 + t < p.T)
                    bulk_load(xs_raw + (size_t)t * H * 2, reinterpret_cast<const __nv_bfloat16*>(p.hidden) + (size_t)(tok0 + t) * H,
                              (uint32_t)H * 2, &bars[warp]);
    }
    pdl_wait();
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
    __syncthreads();
    mbar_wait(&bars[0], 0, &abort_flag);                // norm weights (and warp 0's rows)
    for (int c = tid; c < chunks; c += blockDim.x) {
        const uint4 raw = lds128(nwraw + (size_t)c * 16);
        const float o = p.norm_offset;
        float4* dst = reinterpret_cast<float4*>(gain + c * 8);
        dst[0] = make_float4(o + bf16lo(raw.x), o + bf16hi(raw.x), o + bf16lo(raw.y), o + bf16hi(raw.y));
        dst[1] = make_float4(o + bf16lo(raw.z), o + bf16hi(raw.z), o + bf16lo(raw.w), o + bf16hi(raw.w));
    }
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
        long long* ids2 = p.ids_mirror ? p.ids_mirror + (size_t)token * p.top_k : nullptr;
        float* wts2 = p.weights_mirror ? p.weights_mirror + (size_t)token * p.top_k : nullptr;
        if (E <= 256) topk_warp<8>(row, E, p.top_k, ids, ids32, wts, wts2, ids2);
        else topk_warp<32>(row, E, p.top_k, ids, ids32, wts, wts2, ids2);
    }
}

// dynamic shared memory of router_fast_kernel<TPB, XB> at hidden size H
static size_t router_fast_smem(int tpb, bool xb, int H) {
    return (size_t)kRouterWarps * H * 2 + (size_t)tpb * H * (xb ? 2 : 4) + sizeof(float) * ((size_t)H + tpb + 2) + 8 * sizeof(uint64_t) + (size_t)H * 2 + 16;
}
constexpr size_t kMaxBlockSmem = 227 * 1024;       // opt-in limit of one block on sm_100

template <int TPB, bool XB>
static int launch_router_fast(const RouterParams& p, cudaStream_t stream) {
    const int gate = (p.shared_gate_weight && p.shared_gate_out) ? 1 : 0;
    dim3 grid((p.E + gate + kRouterWarps - 1) / kRouterWarps, (p.T + TPB - 1) / TPB);
    const size_t smem = router_fast_smem(TPB, XB, p.H);
    auto kern = router_fast_kernel<TPB, XB>;
    FK_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "router attr");
    FK_CUDA_OK(launch_pdl(kern, grid, dim3(kRouterWarps * 32), smem, stream, p), "router launch");
    FK_LAUNCH_OK("router launch");
    return FK_OK;
}

// ---------------------------------------------------------------------------------------------
// Tensor-core router for larger batches (bf16 activations and weights, H <= 2048, H % 256 == 0)
// ---------------------------------------------------------------------------------------------
// From a few dozen tokens on the CUDA-core router is bound by instruction issue (one FMA and one
// unpack per product).  Here a block owns 16 tokens x 32 experts; its 8 warps split K, each running
// m16n8k16 MMAs with the tokens as M and the experts as N, and the K-slices meet in shared memory.
// The A operand is x * (offset + norm_weight), an fp32 value, split into three bf16 terms (8 + 8 + 8
// mantissa bits: the split is exact), so the products are exact and only the fp32 accumulation
// rounds, as in the CUDA-core kernels.  The shared gate g . x uses the raw bf16 activations (one MMA).
// Rows sit 16 bytes further apart in shared memory than in HBM, so fragment loads hit 32 banks.
constexpr int kRmTokens = 16;
constexpr int kRmExperts = 32;
constexpr int kRmWarps = 16;               // K slices per block

__device__ __forceinline__ uint32_t rm_lds32(const unsigned char* ptr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(ptr)));
    return v;
}
__device__ __forceinline__ void rm_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// (x, y) -> three packed bf16 pairs whose sum is (x, y) exactly
__device__ __forceinline__ void rm_split3(float x, float y, uint32_t& h, uint32_t& m, uint32_t& l) {
    __nv_bfloat162 a = __floats2bfloat162_rn(x, y);
    float2 af = __bfloat1622float2(a);
    const float rx = x - af.x, ry = y - af.y;
    __nv_bfloat162 b = __floats2bfloat162_rn(rx, ry);
    float2 bf = __bfloat1622float2(b);
    __nv_bfloat162 c = __floats2bfloat162_rn(rx - bf.x, ry - bf.y);
    h = *reinterpret_cast<uint32_t*>(&a);
    m = *reinterpret_cast<uint32_t*>(&b);
    l = *reinterpret_cast<uint32_t*>(&c);
}

__global__ void __launch_bounds__(kRmWarps * 32, 1) router_mma_kernel(RouterParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int H = p.H, E = p.E;
    const int RS = H * 2 + 16;                                                        // padded row stride in bytes
    unsigned char* xs = smem_raw;                                                     // [16][RS]  activations
    unsigned char* ws = xs + (size_t)kRmTokens * RS;                                  // [33][RS]  expert rows (+ gate row)
    float* gain = reinterpret_cast<float*>(ws + (size_t)(kRmExperts + 1) * RS);       // [H]
    float* rstd = gain + H;                                                           // [16]
    uint64_t* bar = reinterpret_cast<uint64_t*>(rstd + kRmTokens);
    unsigned char* nwraw = reinterpret_cast<unsigned char*>(bar + 2);                 // [H] bf16 norm weights as stored
    float* partial = reinterpret_cast<float*>(ws);                                    // [kRmWarps][16][33], after the MMAs
    __shared__ int is_last;
    __shared__ int abort_flag;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tok0 = blockIdx.y * kRmTokens, e0 = blockIdx.x * kRmExperts;
    const int ntok = min(kRmTokens, p.T - tok0), nexp = min(kRmExperts, E - e0);
    const bool with_gate = blockIdx.x == 0 && p.shared_gate_weight != nullptr && p.shared_gate_out != nullptr;
    pdl_trigger();
    if (tid == 0) {
        abort_flag = 0;
        mbar_init(bar, 1);
        mbar_init_fence();
        mbar_expect_tx(bar, (uint32_t)((ntok + nexp + (with_gate ? 1 : 0) + 1) * H * 2));
    }
    __syncthreads();
    // weights are constants: their copies start while the kernel before this one is still draining
    if (warp == 1) {
        if (lane < nexp)
            bulk_load(ws + (size_t)lane * RS, reinterpret_cast<const __nv_bfloat16*>(p.router_weight) + (size_t)(e0 + lane) * H,
                      (uint32_t)H * 2, bar);
        if (lane == 0 && with_gate) bulk_load(ws + (size_t)kRmExperts * RS, p.shared_gate_weight, (uint32_t)H * 2, bar);
        if (lane == 1) bulk_load(nwraw, p.norm_weight, (uint32_t)H * 2, bar);
    }
    pdl_wait();
    if (warp == 0 && lane < ntok)
        bulk_load(xs + (size_t)lane * RS, reinterpret_cast<const __nv_bfloat16*>(p.hidden) + (size_t)(tok0 + lane) * H,
                  (uint32_t)H * 2, bar);
    mbar_wait(bar, 0, &abort_flag);
    for (int c = tid; c < H / 8; c += blockDim.x) {
        const uint4 raw = lds128(nwraw + (size_t)c * 16);
        const float o = p.norm_offset;
        float4* dst = reinterpret_cast<float4*>(gain + c * 8);
        dst[0] = make_float4(o + bf16lo(raw.x), o + bf16hi(raw.x), o + bf16lo(raw.y), o + bf16hi(raw.y));
        dst[1] = make_float4(o + bf16lo(raw.z), o + bf16hi(raw.z), o + bf16lo(raw.w), o + bf16hi(raw.w));
    }
    __syncthreads();

    // mean squares: two tokens per warp
    for (int t = warp; t < kRmTokens; t += kRmWarps) {
        float ss = 0.f;
        if (t < ntok) {
            for (int h = lane * 8; h < H; h += 256) {
                const uint4 v = lds128(xs + (size_t)t * RS + (size_t)h * 2);
                float f;
                f = bf16lo(v.x); ss = fmaf(f, f, ss); f = bf16hi(v.x); ss = fmaf(f, f, ss);
                f = bf16lo(v.y); ss = fmaf(f, f, ss); f = bf16hi(v.y); ss = fmaf(f, f, ss);
                f = bf16lo(v.z); ss = fmaf(f, f, ss); f = bf16hi(v.z); ss = fmaf(f, f, ss);
                f = bf16lo(v.w); ss = fmaf(f, f, ss); f = bf16hi(v.w); ss = fmaf(f, f, ss);
            }
        }
        ss = warp_sum(ss);
        if (lane == 0) rstd[t] = rsqrtf(ss / (float)H + p.eps);
    }

    // this warp's K slice: H/kRmWarps columns, 16 per MMA
    const int gid = lane >> 2, tig = lane & 3;
    const int ksteps = H / (16 * kRmWarps);
    float acc[4][4], gacc[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        gacc[j] = 0.f;
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[j][q] = 0.f;
    }
    {
        const int kbase = warp * (H / kRmWarps) + 2 * tig;
        const unsigned char* xa = xs + (size_t)gid * RS + (size_t)kbase * 2;
        const unsigned char* xb = xa + (size_t)8 * RS;
        const unsigned char* wb = ws + (size_t)gid * RS + (size_t)kbase * 2;
        const float* gp = gain + kbase;
#pragma unroll 2
        for (int ks = 0; ks < ksteps; ++ks) {
            const uint32_t x00 = rm_lds32(xa + ks * 32), x01 = rm_lds32(xa + ks * 32 + 16);   // row gid:     k, k + 8
            const uint32_t x10 = rm_lds32(xb + ks * 32), x11 = rm_lds32(xb + ks * 32 + 16);   // row gid + 8
            const float2 g0 = *reinterpret_cast<const float2*>(gp + ks * 16);
            const float2 g1 = *reinterpret_cast<const float2*>(gp + ks * 16 + 8);
            uint32_t ah[4], am[4], al[4];
            rm_split3(bf16lo(x00) * g0.x, bf16hi(x00) * g0.y, ah[0], am[0], al[0]);
            rm_split3(bf16lo(x10) * g0.x, bf16hi(x10) * g0.y, ah[1], am[1], al[1]);
            rm_split3(bf16lo(x01) * g1.x, bf16hi(x01) * g1.y, ah[2], am[2], al[2]);
            rm_split3(bf16lo(x11) * g1.x, bf16hi(x11) * g1.y, ah[3], am[3], al[3]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const unsigned char* wr = wb + (size_t)j * 8 * RS + ks * 32;
                const uint32_t b0 = rm_lds32(wr), b1 = rm_lds32(wr + 16);
                rm_mma(acc[j], ah[0], ah[1], ah[2], ah[3], b0, b1);
                rm_mma(acc[j], am[0], am[1], am[2], am[3], b0, b1);
                rm_mma(acc[j], al[0], al[1], al[2], al[3], b0, b1);
            }
            if (with_gate) {
                // N column 0 is the gate row; the other seven columns read rows that do not exist: keep them zero
                const unsigned char* wr = ws + (size_t)kRmExperts * RS + (size_t)kbase * 2 + ks * 32;
                const uint32_t b0 = gid == 0 ? rm_lds32(wr) : 0u, b1 = gid == 0 ? rm_lds32(wr + 16) : 0u;
                rm_mma(gacc, x00, x10, x01, x11, b0, b1);
            }
        }
    }
    __syncthreads();                       // every warp is done with the weight rows: their space takes the partial sums
    {
        float* pw = partial + (size_t)warp * kRmTokens * 33;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            pw[gid * 33 + j * 8 + 2 * tig] = acc[j][0];
            pw[gid * 33 + j * 8 + 2 * tig + 1] = acc[j][1];
            pw[(gid + 8) * 33 + j * 8 + 2 * tig] = acc[j][2];
            pw[(gid + 8) * 33 + j * 8 + 2 * tig + 1] = acc[j][3];
        }
        if (with_gate && tig == 0) {
            pw[gid * 33 + 32] = gacc[0];
            pw[(gid + 8) * 33 + 32] = gacc[2];
        }
    }
    __syncthreads();
    for (int idx = tid; idx < kRmTokens * kRmExperts; idx += blockDim.x) {
        const int t = idx >> 5, e = idx & 31;
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < kRmWarps; ++w) sum += partial[(size_t)(w * kRmTokens + t) * 33 + e];
        if (t < ntok && e < nexp) {
            float logit = sum * rstd[t];
            if (p.router_bias) logit += p.router_bias[e0 + e];
            p.logits[(size_t)(tok0 + t) * E + e0 + e] = logit;
        }
    }
    if (with_gate && tid < ntok) {
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < kRmWarps; ++w) sum += partial[(size_t)(w * kRmTokens + tid) * 33 + 32];
        p.shared_gate_out[tok0 + tid] = sigmoidf_(sum);
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
    for (int t = warp; t < ntok; t += kRmWarps) {
        const int token = tok0 + t;
        const float* row = p.logits + (size_t)token * E;
        long long* ids = p.topk_ids + (size_t)token * p.top_k;
        int* ids32 = p.ids32 ? p.ids32 + (size_t)token * p.top_k : nullptr;
        float* wts = p.topk_weights + (size_t)token * p.top_k;
        long long* ids2 = p.ids_mirror ? p.ids_mirror + (size_t)token * p.top_k : nullptr;
        float* wts2 = p.weights_mirror ? p.weights_mirror + (size_t)token * p.top_k : nullptr;
        if (E <= 256) topk_warp<8>(row, E, p.top_k, ids, ids32, wts, wts2, ids2);
        else topk_warp<32>(row, E, p.top_k, ids, ids32, wts, wts2, ids2);
    }
}

static int launch_router_mma(const RouterParams& p, cudaStream_t stream) {
    dim3 grid((p.E + kRmExperts - 1) / kRmExperts, (p.T + kRmTokens - 1) / kRmTokens);
    const size_t rs = (size_t)p.H * 2 + 16;
    const size_t smem = (kRmTokens + kRmExperts + 1) * rs + sizeof(float) * ((size_t)p.H + kRmTokens) + 16 + (size_t)p.H * 2;
    FK_CUDA_OK(cudaFuncSetAttribute(router_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "router attr");
    FK_CUDA_OK(launch_pdl(router_mma_kernel, grid, dim3(kRmWarps * 32), smem, stream, p), "router launch");
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
                    // from 64 tokens the tensor-core router wins (measured: equal at 64, 19 vs 27 us at 128, 19 vs 51 at 256)
                    if (p.T >= 64 && p.H <= 2048 && p.H % (16 * kRmWarps) == 0 &&
                        (size_t)(kRmWarps * kRmTokens * 33) * sizeof(float) <= (size_t)33 * (p.H * 2 + 16))
                        return launch_router_mma(p, stream);
                    // more tokens per block amortise a weight row over more tokens, as far as the block's shared memory
                    // allows (32 tokens of 4096 columns do not fit: 16 are taken there)
                    if (p.T <= 32) return launch_router_fast<4, true>(p, stream);
                    if (p.T <= 64) return launch_router_fast<8, true>(p, stream);
                    if (p.T <= 128 || router_fast_smem(32, true, p.H) > kMaxBlockSmem) return launch_router_fast<16, true>(p, stream);
                    return launch_router_fast<32, true>(p, stream);
                }
                if (p.T > 64 && router_fast_smem(8, false, p.H) <= kMaxBlockSmem) return launch_router_fast<8, false>(p, stream);
                return launch_router_fast<4, false>(p, stream);
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
    // one slot per device ordinal; host threads that make the first call on a device together all store the same value
    static std::atomic<unsigned*> cached[64];
    int dev = 0;
    FK_CUDA_OK(cudaGetDevice(&dev), "noalloc get device");
    if (dev < 0 || dev >= 64) return FK_ERR_UNSUPPORTED;
    unsigned* ptr = cached[dev].load(std::memory_order_acquire);
    if (ptr == nullptr) {
        FK_CUDA_OK(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_tickets), "noalloc symbol address");
        if (ptr == nullptr) return FK_ERR_CUDA;
        cached[dev].store(ptr, std::memory_order_release);
    }
    *out = ptr;
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
