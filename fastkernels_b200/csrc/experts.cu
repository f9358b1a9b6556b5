// Expert MLPs grouped by expert: gate_up GEMV + SwiGLU -> act, down GEMV -> y, ordered combine.
//
// The generic kernels here take any dtype and any H / I (one warp per output element, scalar loads); the bf16 fast
// paths are the streaming GEMV (gemv_tma.cu), the tensor-core grouped GEMM (tc_gemm.cu) and the single-token kernel.
// The combine kernel sums a token's k routed rows in slot order (the reference's in-order slot
// loop, src/fastkernels/kernels/triton/qwen36_expert.py:778-795), adds the gated shared expert
// and optionally the residual, so results do not depend on scheduling.
//
// Reference math: src/fastkernels/reference/qwen36_real.py:339-353.

#include "common.cuh"
#include "kernels.cuh"

namespace fk {

// ---------------------------------------------------------------------------------------------
// Generic kernels
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ int row_expert_of(const ExpertParams& p, int pos) {
    // binary search: largest e with offsets[e] <= pos
    int lo = 0, hi = p.E;
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (p.offsets[mid] <= pos) lo = mid; else hi = mid;
    }
    return lo;
}

template <typename WT>
__global__ void gate_up_generic_kernel(ExpertParams p) {
    const int lane = threadIdx.x & 31;
    const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    const int routed_rows = p.offsets[p.E];
    const int shared_rows = p.shared_gate_up ? p.shared_n : 0;
    const long long total = (long long)(p.routes + shared_rows) * p.I;
    for (long long w = warp; w < total; w += nwarps) {
        int pos = (int)(w / p.I), i = (int)(w - (long long)pos * p.I);
        const WT* wbase;
        int token;
        if (pos >= p.routes) {
            token = p.shared_tok0 + pos - p.routes;
            wbase = reinterpret_cast<const WT*>(p.shared_gate_up);
        } else {
            if (pos >= routed_rows) continue;
            int e = row_expert_of(p, pos);
            token = p.order[pos] / p.top_k;
            wbase = reinterpret_cast<const WT*>(p.gate_up) + (size_t)e * 2 * p.I * p.H;
        }
        const WT* grow = wbase + (size_t)i * p.H;
        const WT* urow = wbase + (size_t)(p.I + i) * p.H;
        float g = 0.f, u = 0.f;
        for (int h = lane; h < p.H; h += 32) {
            float x = load_any(p.hidden, p.hidden_dtype, (size_t)token * p.H + h);
            g = fmaf(to_float(grow[h]), x, g);
            u = fmaf(to_float(urow[h]), x, u);
        }
        g = warp_sum(g);
        u = warp_sum(u);
        if (lane == 0) p.act[(size_t)pos * p.I + i] = silu_mul(g, u);
    }
}

template <typename WT>
__global__ void down_generic_kernel(ExpertParams p) {
    const int lane = threadIdx.x & 31;
    const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    const int routed_rows = p.offsets[p.E];
    const int shared_rows = p.shared_down ? p.shared_n : 0;
    const long long total = (long long)(p.routes + shared_rows) * p.H;
    for (long long w = warp; w < total; w += nwarps) {
        int pos = (int)(w / p.H), h = (int)(w - (long long)pos * p.H);
        const WT* wrow;
        if (pos >= p.routes) {
            wrow = reinterpret_cast<const WT*>(p.shared_down) + (size_t)h * p.I;
        } else {
            if (pos >= routed_rows) continue;
            int e = row_expert_of(p, pos);
            wrow = reinterpret_cast<const WT*>(p.down) + ((size_t)e * p.H + h) * p.I;
        }
        const float* a = p.act + (size_t)pos * p.I;
        float s = 0.f;
        for (int i = lane; i < p.I; i += 32) s = fmaf(to_float(wrow[i]), a[i], s);
        s = warp_sum(s);
        if (lane == 0) p.y[(size_t)pos * p.H + h] = s;
    }
}

int launch_experts_generic(const ExpertParams& p, int weight_dtype, cudaStream_t stream) {
    if (p.T <= 0) return FK_OK;
    const int shared_rows = p.shared_gate_up ? p.shared_n : 0;
    long long gu_warps = (long long)(p.routes + shared_rows) * p.I;
    long long dn_warps = (long long)(p.routes + shared_rows) * p.H;
    auto blocks = [](long long warps) { long long b = (warps + 7) / 8; return (int)(b > 148 * 16 ? 148 * 16 : (b < 1 ? 1 : b)); };
    switch (weight_dtype) {
        case FK_F32:
            gate_up_generic_kernel<float><<<blocks(gu_warps), 256, 0, stream>>>(p);
            FK_LAUNCH_OK("generic gate_up launch");
            stage_mark();
            down_generic_kernel<float><<<blocks(dn_warps), 256, 0, stream>>>(p);
            break;
        case FK_BF16:
            gate_up_generic_kernel<__nv_bfloat16><<<blocks(gu_warps), 256, 0, stream>>>(p);
            FK_LAUNCH_OK("generic gate_up launch");
            stage_mark();
            down_generic_kernel<__nv_bfloat16><<<blocks(dn_warps), 256, 0, stream>>>(p);
            break;
        case FK_F16:
            gate_up_generic_kernel<__half><<<blocks(gu_warps), 256, 0, stream>>>(p);
            FK_LAUNCH_OK("generic gate_up launch");
            stage_mark();
            down_generic_kernel<__half><<<blocks(dn_warps), 256, 0, stream>>>(p);
            break;
        default:
            return FK_ERR_UNSUPPORTED;
    }
    FK_LAUNCH_OK("generic down launch");
    stage_mark();
    return FK_OK;
}

// ---------------------------------------------------------------------------------------------
// Ordered combine
// ---------------------------------------------------------------------------------------------
// One thread per token and four output columns: the positions and weights of all slots are fetched first, then
// all rows, so the kernel is two dependent memory round trips deep whatever top_k is.  Slots are summed in order.
__global__ void __launch_bounds__(256) combine_kernel(ExpertParams p) {
    pdl_trigger();
    pdl_wait();
    const int H4 = p.H >> 2;
    const long long total = (long long)p.T * H4;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / H4), h = (int)(i - (long long)t * H4) * 4;
        int pos[FK_MAX_TOP_K];
        float w[FK_MAX_TOP_K];
#pragma unroll
        for (int s = 0; s < FK_MAX_TOP_K; ++s) {
            pos[s] = s < p.top_k ? p.inv[t * p.top_k + s] : -1;
            w[s] = s < p.top_k ? p.topk_weights[t * p.top_k + s] : 0.f;
        }
        const bool shared = p.shared_down && t >= p.shared_tok0 && t < p.shared_tok0 + p.shared_n;
        float4 v[FK_MAX_TOP_K], sh = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int s = 0; s < FK_MAX_TOP_K; ++s)
            v[s] = pos[s] >= 0 ? *reinterpret_cast<const float4*>(p.y + (size_t)pos[s] * p.H + h) : make_float4(0.f, 0.f, 0.f, 0.f);
        float gate = 1.f;
        if (shared) {
            sh = *reinterpret_cast<const float4*>(p.y + (size_t)(p.routes + t - p.shared_tok0) * p.H + h);
            if (p.shared_gate) gate = p.shared_gate[t];
        }
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int s = 0; s < FK_MAX_TOP_K; ++s) {
            if (pos[s] >= 0) {
                acc.x = fmaf(w[s], v[s].x, acc.x); acc.y = fmaf(w[s], v[s].y, acc.y);
                acc.z = fmaf(w[s], v[s].z, acc.z); acc.w = fmaf(w[s], v[s].w, acc.w);
            }
        }
        if (shared) {
            if (p.shared_gate) { acc.x += gate * sh.x; acc.y += gate * sh.y; acc.z += gate * sh.z; acc.w += gate * sh.w; }
            else { acc.x += sh.x; acc.y += sh.y; acc.z += sh.z; acc.w += sh.w; }
        }
        *reinterpret_cast<float4*>(p.out + (size_t)t * p.H + h) = acc;
        if (p.layer_hidden) {
            const size_t o = (size_t)t * p.H + h;
            float4 r;
            r.x = load_any(p.hidden, p.hidden_dtype, o) + acc.x; r.y = load_any(p.hidden, p.hidden_dtype, o + 1) + acc.y;
            r.z = load_any(p.hidden, p.hidden_dtype, o + 2) + acc.z; r.w = load_any(p.hidden, p.hidden_dtype, o + 3) + acc.w;
            *reinterpret_cast<float4*>(p.layer_hidden + o) = r;
        }
    }
}

// any H, any alignment
__global__ void combine_scalar_kernel(ExpertParams p) {
    pdl_trigger();
    pdl_wait();
    const long long total = (long long)p.T * p.H;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        int t = (int)(i / p.H), h = (int)(i - (long long)t * p.H);
        float acc = 0.f;
        for (int s = 0; s < p.top_k; ++s) {
            int pos = p.inv[t * p.top_k + s];
            if (pos >= 0) acc = fmaf(p.topk_weights[t * p.top_k + s], p.y[(size_t)pos * p.H + h], acc);
        }
        if (p.shared_down && t >= p.shared_tok0 && t < p.shared_tok0 + p.shared_n) {
            float sh = p.y[(size_t)(p.routes + t - p.shared_tok0) * p.H + h];
            acc += p.shared_gate ? p.shared_gate[t] * sh : sh;
        }
        p.out[i] = acc;
        if (p.layer_hidden) p.layer_hidden[i] = load_any(p.hidden, p.hidden_dtype, (size_t)i) + acc;
    }
}

int launch_combine(const ExpertParams& p, cudaStream_t stream) {
    if (p.T <= 0) return FK_OK;
    const bool vec = p.H % 4 == 0 && p.top_k <= FK_MAX_TOP_K &&
                     ((reinterpret_cast<uintptr_t>(p.out) | reinterpret_cast<uintptr_t>(p.y) | reinterpret_cast<uintptr_t>(p.layer_hidden)) & 15) == 0;
    long long total = (long long)p.T * (vec ? p.H / 4 : p.H);
    int blocks = (int)((total + 255) / 256);
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (vec) FK_CUDA_OK(launch_pdl(combine_kernel, dim3(blocks), dim3(256), 0, stream, p), "combine launch");
    else FK_CUDA_OK(launch_pdl(combine_scalar_kernel, dim3(blocks), dim3(256), 0, stream, p), "combine launch");
    FK_LAUNCH_OK("combine launch");
    return FK_OK;
}

// ---------------------------------------------------------------------------------------------
// Stand-alone fused SwiGLU: out[n,c] = silu(gu[n,c]) * gu[n,I+c]
// (src/fastkernels/kernels/triton/moe.py:33-45: fp32 math, result stored in the input dtype)
// ---------------------------------------------------------------------------------------------
template <typename TT>
__device__ __forceinline__ TT from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }

template <typename TT>
__global__ void swiglu_kernel(const TT* __restrict__ gu, TT* __restrict__ out, long long rows, int I) {
    const long long total = rows * I;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        long long n = i / I;
        int c = (int)(i - n * I);
        float g = to_float(gu[n * 2 * I + c]), u = to_float(gu[n * 2 * I + I + c]);
        out[i] = from_float<TT>(silu_mul(g, u));
    }
}

int launch_swiglu(const void* gate_up, void* out, int dtype, long long rows, int I, cudaStream_t stream) {
    if (rows < 0 || I < 0) return FK_ERR_ARG;
    long long total = rows * I;
    if (total == 0) return FK_OK;
    long long b = (total + 255) / 256;
    int blocks = (int)(b > 148 * 16 ? 148 * 16 : b);
    switch (dtype) {
        case FK_F32: swiglu_kernel<float><<<blocks, 256, 0, stream>>>((const float*)gate_up, (float*)out, rows, I); break;
        case FK_BF16: swiglu_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, rows, I); break;
        case FK_F16: swiglu_kernel<__half><<<blocks, 256, 0, stream>>>((const __half*)gate_up, (__half*)out, rows, I); break;
        default: return FK_ERR_UNSUPPORTED;
    }
    FK_LAUNCH_OK("swiglu launch");
    return FK_OK;
}

}  // namespace fk
