// Expert MLPs grouped by expert: gate_up GEMV + SwiGLU -> act, down GEMV -> y, ordered combine.
//
// Two families:
//  * generic kernels: one warp per output element, scalar loads, any dtype and any H / I;
//  * bf16 weight-streaming GEMV kernels: every lane owns 8 consecutive columns (one 16-byte
//    load per weight row), the K dimension is split across lanes and warps, activations of up
//    to 4 tokens of the expert stay in registers, and partial sums are folded with a
//    transposing warp-shuffle reduction (one shuffle per value instead of five).
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
// bf16 weight-streaming GEMV
// ---------------------------------------------------------------------------------------------
constexpr int kGemvThreads = 256;
constexpr int kGemvWarps = 8;

template <int V> struct Log2 { static constexpr int value = 1 + Log2<V / 2>::value; };
template <> struct Log2<1> { static constexpr int value = 0; };

// After the call, v[0] of lane L holds the warp-wide sum of the value with index L >> (5 - log2 V).
template <int V>
__device__ __forceinline__ void warp_transpose_reduce(float (&v)[V], int lane) {
    constexpr int L = Log2<V>::value;
#pragma unroll
    for (int s = 0; s < L; ++s) {
        const int half = V >> (s + 1);
        const int off = 16 >> s;
        const bool upper = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < half; ++i) {
            float send = upper ? v[i] : v[i + half];
            float keep = upper ? v[i + half] : v[i];
            v[i] = keep + __shfl_xor_sync(kFull, send, off);
        }
    }
#pragma unroll
    for (int off = 16 >> L; off > 0; off >>= 1) v[0] += __shfl_xor_sync(kFull, v[0], off);
}

__device__ __forceinline__ void unpack8(const uint4& w, float (&f)[8]) {
    f[0] = bf16lo(w.x); f[1] = bf16hi(w.x); f[2] = bf16lo(w.y); f[3] = bf16hi(w.y);
    f[4] = bf16lo(w.z); f[5] = bf16hi(w.z); f[6] = bf16lo(w.w); f[7] = bf16hi(w.w);
}

// 8 consecutive elements starting at `elem` (a multiple of 8) of an array of run-time dtype.
__device__ __forceinline__ void load8_any(const void* base, int dtype, size_t elem, float (&o)[8]) {
    if (dtype == FK_BF16) {
        uint4 v = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(base) + elem);
        unpack8(v, o);
    } else if (dtype == FK_F16) {
        uint4 v = *reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(base) + elem);
        const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 f = __half22float2(h[i]);
            o[2 * i] = f.x; o[2 * i + 1] = f.y;
        }
    } else {
        const float4* q = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + elem);
        float4 a = q[0], b = q[1];
        o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
    }
}

// Tile geometry shared by host and device.
__host__ __device__ constexpr int gemv_tile_pairs(int kch) { return (8 / kch) * 4 > 16 ? (8 / kch) * 4 : 16; }
constexpr int kDownTileRows = 64;

// One pass of the gate_up tile for NT tokens: streams 2*TP rows of K = KCH*256 columns.
template <int NT, int KCH>
__device__ __forceinline__ void gate_up_pass(const ExpertParams& p, const __nv_bfloat16* __restrict__ W, int tile,
                                             int row_pos, int tok_first, int nvalid, bool shared,
                                             float (*partial)[kGemvWarps][32], int& buf) {
    constexpr int RG = kGemvWarps / KCH;
    constexpr int RS = NT == 1 ? 8 : 4;         // weight rows in flight per lane
    constexpr int PP = RS / 2;                  // gate/up pairs per step per row group
    constexpr int V = RS * NT;
    constexpr int SH = 5 - Log2<V>::value;
    constexpr int TP = gemv_tile_pairs(KCH);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int kw = warp % KCH, rg = warp / KCH;
    const int K = KCH * 256;
    const int col0 = kw * 256 + lane * 8;

    float x[NT][8];
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        if (t < nvalid) {
            int token = shared ? (tok_first + t) : (p.order[row_pos + t] / p.top_k);
            load8_any(p.hidden, p.hidden_dtype, (size_t)token * K + col0, x[t]);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) x[t][i] = 0.f;
        }
    }
    constexpr int STEPS = TP / (PP * RG);
#pragma unroll 1
    for (int step = 0; step < STEPS; ++step) {
        const int pair0 = tile * TP + (step * RG + rg) * PP;
        uint4 w[RS];
#pragma unroll
        for (int q = 0; q < PP; ++q) {
            w[q] = ld_stream16(W + (size_t)(pair0 + q) * K + col0);
            w[PP + q] = ld_stream16(W + (size_t)(p.I + pair0 + q) * K + col0);
        }
        float acc[V];
#pragma unroll
        for (int r = 0; r < RS; ++r) {
            float wf[8];
            unpack8(w[r], wf);
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                float a = 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i) a = fmaf(wf[i], x[t][i], a);
                acc[r * NT + t] = a;
            }
        }
        warp_transpose_reduce<V>(acc, lane);
        if ((lane & ((1 << SH) - 1)) == 0) partial[buf][warp][lane >> SH] = acc[0];
        __syncthreads();
        if (tid < RG * PP * NT) {
            const int rg2 = tid / (PP * NT), rem = tid - rg2 * (PP * NT);
            const int q = rem / NT, t = rem - q * NT;
            float g = 0.f, u = 0.f;
#pragma unroll
            for (int k2 = 0; k2 < KCH; ++k2) {
                g += partial[buf][rg2 * KCH + k2][q * NT + t];
                u += partial[buf][rg2 * KCH + k2][(PP + q) * NT + t];
            }
            if (t < nvalid) {
                const int col = tile * TP + (step * RG + rg2) * PP + q;
                p.act[(size_t)(row_pos + t) * p.I + col] = silu_mul(g, u);
            }
        }
        buf ^= 1;
    }
}

template <int KCH>
__global__ void __launch_bounds__(kGemvThreads) gate_up_gemv_kernel(ExpertParams p) {
    __shared__ float partial[2][kGemvWarps][32];
    constexpr int TP = gemv_tile_pairs(KCH);
    const int U = p.meta[0];
    const int has_shared = p.shared_gate_up != nullptr ? 1 : 0;
    const int tiles = p.I / TP;
    const int items = (U + has_shared) * tiles;
    const __nv_bfloat16* gate_up = reinterpret_cast<const __nv_bfloat16*>(p.gate_up);
    int buf = 0;
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
        const int u = item / tiles, tile = item - u * tiles;
        const bool shared = (u == U);
        const __nv_bfloat16* W;
        int n, row_base;
        if (shared) {
            W = reinterpret_cast<const __nv_bfloat16*>(p.shared_gate_up);
            n = p.T;
            row_base = p.routes;
        } else {
            const int e = p.touched[u];
            W = gate_up + (size_t)e * 2 * p.I * p.H;
            row_base = p.offsets[e];
            n = p.counts[e];
        }
        int done = 0;
        while (done < n) {
            const int rem = n - done;
            if (rem == 1) { gate_up_pass<1, KCH>(p, W, tile, row_base + done, done, 1, shared, partial, buf); done += 1; }
            else if (rem == 2) { gate_up_pass<2, KCH>(p, W, tile, row_base + done, done, 2, shared, partial, buf); done += 2; }
            else { const int nv = rem < 4 ? rem : 4; gate_up_pass<4, KCH>(p, W, tile, row_base + done, done, nv, shared, partial, buf); done += nv; }
        }
    }
}

// One pass of a down tile (kDownTileRows output rows) for NT tokens; K = I = KCH*256.
template <int NT, int KCH>
__device__ __forceinline__ void down_pass(const ExpertParams& p, const __nv_bfloat16* __restrict__ W, int tile,
                                          int row_pos, int nvalid, float (*partial)[kGemvWarps][32], int& buf) {
    constexpr int RG = kGemvWarps / KCH;
    constexpr int RS = NT == 1 ? 8 : 4;
    constexpr int V = RS * NT;
    constexpr int SH = 5 - Log2<V>::value;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int kw = warp % KCH, rg = warp / KCH;
    const int K = KCH * 256;
    const int col0 = kw * 256 + lane * 8;

    float x[NT][8];
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        if (t < nvalid) {
            const float4* a = reinterpret_cast<const float4*>(p.act + (size_t)(row_pos + t) * K + col0);
            float4 lo = a[0], hi = a[1];
            x[t][0] = lo.x; x[t][1] = lo.y; x[t][2] = lo.z; x[t][3] = lo.w;
            x[t][4] = hi.x; x[t][5] = hi.y; x[t][6] = hi.z; x[t][7] = hi.w;
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) x[t][i] = 0.f;
        }
    }
    constexpr int STEPS = kDownTileRows / (RS * RG);
#pragma unroll 1
    for (int step = 0; step < STEPS; ++step) {
        const int h0 = tile * kDownTileRows + (step * RG + rg) * RS;
        uint4 w[RS];
#pragma unroll
        for (int r = 0; r < RS; ++r) w[r] = ld_stream16(W + (size_t)(h0 + r) * K + col0);
        float acc[V];
#pragma unroll
        for (int r = 0; r < RS; ++r) {
            float wf[8];
            unpack8(w[r], wf);
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                float a = 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i) a = fmaf(wf[i], x[t][i], a);
                acc[r * NT + t] = a;
            }
        }
        warp_transpose_reduce<V>(acc, lane);
        if ((lane & ((1 << SH) - 1)) == 0) partial[buf][warp][lane >> SH] = acc[0];
        __syncthreads();
        if (tid < RG * RS * NT) {
            const int rg2 = tid / (RS * NT), rem = tid - rg2 * (RS * NT);
            const int r = rem / NT, t = rem - r * NT;
            float s = 0.f;
#pragma unroll
            for (int k2 = 0; k2 < KCH; ++k2) s += partial[buf][rg2 * KCH + k2][r * NT + t];
            if (t < nvalid) {
                const int h = tile * kDownTileRows + (step * RG + rg2) * RS + r;
                p.y[(size_t)(row_pos + t) * p.H + h] = s;
            }
        }
        buf ^= 1;
    }
}

template <int KCH>
__global__ void __launch_bounds__(kGemvThreads) down_gemv_kernel(ExpertParams p) {
    __shared__ float partial[2][kGemvWarps][32];
    const int U = p.meta[0];
    const int has_shared = p.shared_down != nullptr ? 1 : 0;
    const int tiles = p.H / kDownTileRows;
    const int items = (U + has_shared) * tiles;
    const __nv_bfloat16* down = reinterpret_cast<const __nv_bfloat16*>(p.down);
    int buf = 0;
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
        const int u = item / tiles, tile = item - u * tiles;
        const __nv_bfloat16* W;
        int n, row_base;
        if (u == U) {
            W = reinterpret_cast<const __nv_bfloat16*>(p.shared_down);
            n = p.T;
            row_base = p.routes;
        } else {
            const int e = p.touched[u];
            W = down + (size_t)e * p.H * p.I;
            row_base = p.offsets[e];
            n = p.counts[e];
        }
        int done = 0;
        while (done < n) {
            const int rem = n - done;
            if (rem == 1) { down_pass<1, KCH>(p, W, tile, row_base + done, 1, partial, buf); done += 1; }
            else if (rem == 2) { down_pass<2, KCH>(p, W, tile, row_base + done, 2, partial, buf); done += 2; }
            else { const int nv = rem < 4 ? rem : 4; down_pass<4, KCH>(p, W, tile, row_base + done, nv, partial, buf); done += nv; }
        }
    }
}

static bool kch_ok(int k) { return k == 256 || k == 512 || k == 1024 || k == 2048; }

bool gemv_path_supported(const ExpertParams& p, int weight_dtype) {
    if (weight_dtype != FK_BF16) return false;
    if (!kch_ok(p.H) || !kch_ok(p.I)) return false;
    if (p.I % gemv_tile_pairs(p.H / 256) != 0 || p.H % kDownTileRows != 0) return false;
    uintptr_t bits = reinterpret_cast<uintptr_t>(p.hidden) | reinterpret_cast<uintptr_t>(p.gate_up) |
                     reinterpret_cast<uintptr_t>(p.down) | reinterpret_cast<uintptr_t>(p.shared_gate_up) |
                     reinterpret_cast<uintptr_t>(p.shared_down);
    return (bits & 15) == 0;
}

int launch_experts_gemv(const ExpertParams& p, cudaStream_t stream) {
    if (p.T <= 0) return FK_OK;
    const int grid = 148 * 2;
    switch (p.H / 256) {
        case 1: gate_up_gemv_kernel<1><<<grid, kGemvThreads, 0, stream>>>(p); break;
        case 2: gate_up_gemv_kernel<2><<<grid, kGemvThreads, 0, stream>>>(p); break;
        case 4: gate_up_gemv_kernel<4><<<grid, kGemvThreads, 0, stream>>>(p); break;
        case 8: gate_up_gemv_kernel<8><<<grid, kGemvThreads, 0, stream>>>(p); break;
        default: return FK_ERR_UNSUPPORTED;
    }
    FK_LAUNCH_OK("gate_up gemv launch");
    stage_mark();   // end of gate_up
    switch (p.I / 256) {
        case 1: down_gemv_kernel<1><<<grid, kGemvThreads, 0, stream>>>(p); break;
        case 2: down_gemv_kernel<2><<<grid, kGemvThreads, 0, stream>>>(p); break;
        case 4: down_gemv_kernel<4><<<grid, kGemvThreads, 0, stream>>>(p); break;
        case 8: down_gemv_kernel<8><<<grid, kGemvThreads, 0, stream>>>(p); break;
        default: return FK_ERR_UNSUPPORTED;
    }
    FK_LAUNCH_OK("down gemv launch");
    stage_mark();   // end of down
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
