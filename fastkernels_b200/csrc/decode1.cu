// Whole MoE layer for ONE token in one cooperative launch (bf16 weights).
//
// One block per SM.  The layer has three dependent phases; the blocks meet at two grid-wide
// barriers (bounded spins on counters in the workspace, co-residency guaranteed by the cooperative
// launch):
//   A  router rows -> logits, shared-expert gate_up pairs -> shared activations, gate dot   (static)
//   -- barrier 1 --  every block runs softmax + top-k (by rank) on the 256 logits itself
//   B  the 8 selected experts' gate_up pairs -> activations; shared-expert down rows
//   -- barrier 2 --
//   C  the 8 selected experts' down rows for this block's slice of the output, summed in slot order
//      with the routing weights, plus the gated shared expert (and the residual)
// Work is split evenly by bytes: every block streams the same share of every matrix.
//
// A producer warp issues bulk copies (one weight row or gate/up pair per 8 KB stage) into a
// 16-stage shared-memory ring and runs ahead across the barriers: phase C addresses depend only on
// the expert ids, so those rows are already in flight while the blocks wait at barrier 2.  Eight
// consumer warps take the stages round-robin; a stage is handled by one warp (16-byte shared loads,
// the token's activations in registers, shuffle reduction), so consumers never synchronise with
// each other inside a phase.  Code that runs once per launch (router rows, top-k, down rows) is
// written as short rolled loops: at this size the kernel is bound by instruction fetch and memory
// latency, not by issue rate.
//
// Reference math: src/fastkernels/reference/qwen36_real.py:329-354.

#include <cooperative_groups.h>

#include "common.cuh"
#include "kernels.cuh"
#include "tma.cuh"
#include "topk.cuh"

namespace fk {

constexpr int kD1Stages = 16;
constexpr int kD1StageBytes = 8192;
constexpr int kD1Consumers = 8;                  // warps
// Stage `it` lives in slot it % kD1Stages and is consumed by warp it % kD1Consumers.  The slot count must be a
// multiple of the warp count: then a slot always belongs to the same warp, which meets its laps in order.  With
// any other ratio another warp can reach lap k of a slot while lap k-1 is still in flight (bulk copies complete
// out of order, e.g. after a TLB miss), and a one-bit phase parity cannot tell "lap k landed" from "lap k-1 has
// not landed yet": the warp would read the slot early and release it twice.
static_assert(kD1Stages % kD1Consumers == 0, "every ring slot must belong to one consumer warp");
constexpr int kD1Threads = (kD1Consumers + 1) * 32;
constexpr int kD1MaxRows = 64;                   // output rows per block (H / #blocks rounded up)

struct D1Smem {
    unsigned char stage[kD1Stages][kD1StageBytes];
    uint64_t full[kD1Stages];
    uint64_t empty[kD1Stages];
    uint64_t ids_ready;
    uint64_t xready;                              // the token's activations and the norm weights are in shared memory
    uint64_t staged_a;                            // logits and shared activations of all blocks are in shared memory
    uint64_t staged_b;                            // routed activations of all blocks are in shared memory
    int4 desc[kD1Stages];                         // what each stage holds (written by the producer)
    float dpart[FK_MAX_TOP_K][kD1MaxRows];       // un-weighted down outputs per slot
    float ysh[kD1MaxRows];                       // shared-expert down outputs
    float weights[FK_MAX_TOP_K];                 // selected probabilities, descending
    float wnorm[FK_MAX_TOP_K];                   // renormalised routing weights
    float red[2 * kD1Consumers];                 // block reductions of the softmax
    int ids[FK_MAX_TOP_K];
    int abort_flag;
};

enum D1Kind { kRouterRow = 0, kGateRow = 1, kSharedPair = 2, kRoutedPair = 3, kSharedDown = 4, kRoutedDown = 5, kNone = 6 };

struct D1Plan {
    // static split of the work of block b among G blocks
    int nA_router, nA_gate, nA_pair, nB_pair, nB_down, nC;   // stages per kind
    int pair0, q0, h0, nh;                                    // first shared pair, first routed pair, output slice
    int rows_per_stage;                                       // down rows per stage (8 KB / row bytes)
};

struct D1Stage {
    int kind, a, b, c;   // see decode_stage
};

__device__ __forceinline__ D1Plan make_plan(const DecodeParams& p, int b, int G) {
    D1Plan pl;
    pl.nA_router = (p.E - b + G - 1) / G;
    if (b >= p.E) pl.nA_router = 0;
    pl.nA_gate = (p.shared_gate != nullptr && b == G - 1) ? 1 : 0;
    const int has_shared = p.shared_gate_up != nullptr;
    const unsigned ub = (unsigned)b, uG = (unsigned)G;
    pl.pair0 = (int)(ub * (unsigned)p.I / uG);
    const int pair1 = (int)((ub + 1u) * (unsigned)p.I / uG);
    pl.nA_pair = has_shared ? pair1 - pl.pair0 : 0;
    pl.q0 = (int)(ub * (unsigned)(p.top_k * p.I) / uG);
    const int q1 = (int)((ub + 1u) * (unsigned)(p.top_k * p.I) / uG);
    pl.nB_pair = q1 - pl.q0;
    pl.h0 = (int)(ub * (unsigned)p.H / uG);
    pl.nh = (int)((ub + 1u) * (unsigned)p.H / uG) - pl.h0;
    pl.rows_per_stage = min(8, kD1StageBytes / (p.I * 2));
    const int down_stages = (pl.nh + pl.rows_per_stage - 1) / pl.rows_per_stage;
    pl.nB_down = has_shared ? down_stages : 0;
    pl.nC = down_stages * p.top_k;
    return pl;
}

// Stage number `it` of a block -> what it holds.
//   kRouterRow : a = expert row            kGateRow : -
//   kSharedPair: a = pair index            kRoutedPair: a = slot, b = pair index
//   kSharedDown: a = first local row, b = rows      kRoutedDown: a = slot, b = first local row, c = rows
__device__ __forceinline__ D1Stage decode_stage(const D1Plan& pl, const DecodeParams& p, int it, int blk, int G) {
    D1Stage s{kNone, 0, 0, 0};
    if (it < pl.nA_router) { s.kind = kRouterRow; s.a = blk + it * G; return s; }
    it -= pl.nA_router;
    if (it < pl.nA_gate) { s.kind = kGateRow; return s; }
    it -= pl.nA_gate;
    if (it < pl.nA_pair) { s.kind = kSharedPair; s.a = pl.pair0 + it; return s; }
    it -= pl.nA_pair;
    if (it < pl.nB_pair) { const int q = pl.q0 + it; s.kind = kRoutedPair; s.a = q / p.I; s.b = q - s.a * p.I; return s; }
    it -= pl.nB_pair;
    if (it < pl.nB_down) {
        s.kind = kSharedDown; s.a = it * pl.rows_per_stage; s.b = min(pl.rows_per_stage, pl.nh - s.a); return s;
    }
    it -= pl.nB_down;
    if (it < pl.nC) {
        const int per_slot = pl.nC / p.top_k;
        s.kind = kRoutedDown; s.a = it / per_slot;
        s.b = (it - s.a * per_slot) * pl.rows_per_stage; s.c = min(pl.rows_per_stage, pl.nh - s.b); return s;
    }
    return s;
}

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// optional trace: p.trace[block][slot] = nanosecond timestamp of a phase boundary (16 words per block;
// words 8 and 9 hold the SM cycle counter at start and exit)
#define D1_TRACE(slot) do { if (p.trace) p.trace[(size_t)blk * 16 + (slot)] = global_ns(); } while (0)

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Orders this thread's earlier generic-proxy accesses (and what it has acquired from other threads) before its
// later bulk copies, which read and write memory through the async proxy.
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Bounded spin until *word >= target; false on time-out.
__device__ __forceinline__ bool spin_until(const unsigned* word, unsigned target, volatile int* abort_flag) {
    if (ld_acquire_u32(word) >= target) return true;
    const long long limit = *abort_flag ? kWaitCyclesAfterAbort : kWaitCycles;
    const long long t0 = clock64();
    while (ld_acquire_u32(word) < target) {
        if (clock64() - t0 > limit) { *abort_flag = 1; return false; }
    }
    return true;
}

// gate and up row of one pair against the token's activations held in registers (hot loop, unrolled)
__device__ __forceinline__ void pair_dot(const unsigned char* grow, const unsigned char* urow, const float (&x)[8][8],
                                         int lane, int nch, float& g, float& u) {
    float g0 = 0.f, g1 = 0.f, u0 = 0.f, u1 = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        if (j < nch) {
            const uint4 a = lds128(grow + (size_t)(j * 256 + lane * 8) * 2);
            const uint4 b = lds128(urow + (size_t)(j * 256 + lane * 8) * 2);
            g0 = fmaf(bf16lo(a.x), x[j][0], g0); g1 = fmaf(bf16hi(a.x), x[j][1], g1);
            g0 = fmaf(bf16lo(a.y), x[j][2], g0); g1 = fmaf(bf16hi(a.y), x[j][3], g1);
            g0 = fmaf(bf16lo(a.z), x[j][4], g0); g1 = fmaf(bf16hi(a.z), x[j][5], g1);
            g0 = fmaf(bf16lo(a.w), x[j][6], g0); g1 = fmaf(bf16hi(a.w), x[j][7], g1);
            u0 = fmaf(bf16lo(b.x), x[j][0], u0); u1 = fmaf(bf16hi(b.x), x[j][1], u1);
            u0 = fmaf(bf16lo(b.y), x[j][2], u0); u1 = fmaf(bf16hi(b.y), x[j][3], u1);
            u0 = fmaf(bf16lo(b.z), x[j][4], u0); u1 = fmaf(bf16hi(b.z), x[j][5], u1);
            u0 = fmaf(bf16lo(b.w), x[j][6], u0); u1 = fmaf(bf16hi(b.w), x[j][7], u1);
        }
    }
    g = warp_sum(g0 + g1);
    u = warp_sum(u0 + u1);
}

// one bf16 row of nch*256 columns against a vector in shared memory (rolled on purpose: this code
// runs a handful of times per launch, and a short loop costs far fewer instruction fetches)
__device__ __forceinline__ float row_dot_smem(const unsigned char* row, const float* vec, int lane, int nch) {
    float a0 = 0.f, a1 = 0.f;
#pragma unroll 2
    for (int j = 0; j < nch; ++j) {
        const int c = j * 256 + lane * 8;
        const uint4 w = lds128(row + (size_t)c * 2);
        const float4 v0 = *reinterpret_cast<const float4*>(vec + c);
        const float4 v1 = *reinterpret_cast<const float4*>(vec + c + 4);
        a0 = fmaf(bf16lo(w.x), v0.x, a0); a1 = fmaf(bf16hi(w.x), v0.y, a1);
        a0 = fmaf(bf16lo(w.y), v0.z, a0); a1 = fmaf(bf16hi(w.y), v0.w, a1);
        a0 = fmaf(bf16lo(w.z), v1.x, a0); a1 = fmaf(bf16hi(w.z), v1.y, a1);
        a0 = fmaf(bf16lo(w.w), v1.z, a0); a1 = fmaf(bf16hi(w.w), v1.w, a1);
    }
    return warp_sum(a0 + a1);
}

// up to 8 rows of nch*256 columns (row stride = row_bytes) against one vector in shared memory, all
// rows at once: 8 independent sums per lane, folded with a transposing shuffle reduction.
// Returns in every lane the sum of the row (lane >> 2), i.e. lanes 4r..4r+3 hold row r.
__device__ __forceinline__ float rows8_dot_smem(const unsigned char* base, int row_bytes, int nrows, const float* vec,
                                                int lane, int nch) {
    float acc[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) acc[r] = 0.f;
#pragma unroll 1
    for (int j = 0; j < nch; ++j) {
        const int c = j * 256 + lane * 8;
        const float4 v0 = *reinterpret_cast<const float4*>(vec + c);
        const float4 v1 = *reinterpret_cast<const float4*>(vec + c + 4);
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            if (r < nrows) {
                const uint4 w = lds128(base + (size_t)r * row_bytes + (size_t)c * 2);
                float a = acc[r];
                a = fmaf(bf16lo(w.x), v0.x, a); a = fmaf(bf16hi(w.x), v0.y, a);
                a = fmaf(bf16lo(w.y), v0.z, a); a = fmaf(bf16hi(w.y), v0.w, a);
                a = fmaf(bf16lo(w.z), v1.x, a); a = fmaf(bf16hi(w.z), v1.y, a);
                a = fmaf(bf16lo(w.w), v1.z, a); a = fmaf(bf16hi(w.w), v1.w, a);
                acc[r] = a;
            }
        }
    }
    // transposing reduction: 4 + 2 + 1 exchanges, then two plain steps
#pragma unroll
    for (int st = 0; st < 3; ++st) {
        const int half = 4 >> st, off = 16 >> st;
        const bool upper = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (i < half) {
                const float send = upper ? acc[i] : acc[i + half];
                const float keep = upper ? acc[i + half] : acc[i];
                acc[i] = keep + __shfl_xor_sync(kFull, send, off);
            }
        }
    }
    acc[0] += __shfl_xor_sync(kFull, acc[0], 2);
    acc[0] += __shfl_xor_sync(kFull, acc[0], 1);
    return acc[0];
}

// k rounds of warp arg-max over probabilities in shared memory (ties to the lower index); lane r
// writes the r-th winner.  Non-negative floats order like their bit patterns: key = bits + 1, 0 = taken.
template <int EPL>
__device__ __forceinline__ void select_warp(const float* probs, int E, int top_k, int* ids, float* vals, int lane) {
    unsigned key[EPL];
#pragma unroll
    for (int j = 0; j < EPL; ++j) key[j] = (j * 32 + lane < E) ? __float_as_uint(probs[j * 32 + lane]) + 1u : 0u;
#pragma unroll 1
    for (int r = 0; r < top_k; ++r) {
        unsigned best = 0u;
#pragma unroll
        for (int j = 0; j < EPL; ++j) best = max(best, key[j]);
        const unsigned m = __reduce_max_sync(kFull, best);
        unsigned cand = 0x7fffffffu;
#pragma unroll
        for (int j = EPL - 1; j >= 0; --j) cand = (key[j] == m) ? (unsigned)(j * 32 + lane) : cand;
        const unsigned bi = __reduce_min_sync(kFull, cand);
#pragma unroll
        for (int j = 0; j < EPL; ++j) key[j] = ((unsigned)(j * 32 + lane) == bi) ? 0u : key[j];
        if (lane == r) { ids[r] = (int)bi; vals[r] = __uint_as_float(m - 1u); }
    }
}

// Block-wide softmax over the logits in `probs` (shared memory), then top-k by one warp (threads = cthreads
// consumer threads, E <= 1024).
// Every thread owns the experts e = ctid, ctid + cthreads, ... for the softmax.
// Writes ids/weights to shared memory (and to global memory from block 0).
__device__ __forceinline__ void block_topk(const DecodeParams& p, D1Smem& s, float* probs, int ctid, int cthreads, bool write_global) {
    const int E = p.E, lane = ctid & 31, w = ctid >> 5;
    float m = -INFINITY;
    for (int e = ctid; e < E; e += cthreads) {
        const float l = probs[e];                 // the logits were bulk-copied here
        m = fmaxf(m, l);
    }
    m = warp_max(m);
    if (lane == 0) s.red[w] = m;
    named_bar_sync(1, cthreads);
    m = s.red[0];
    for (int i = 1; i < kD1Consumers; ++i) m = fmaxf(m, s.red[i]);
    float sum = 0.f;
    for (int e = ctid; e < E; e += cthreads) {
        const float ex = expf(probs[e] - m);
        probs[e] = ex;
        sum += ex;
    }
    sum = warp_sum(sum);
    if (lane == 0) s.red[kD1Consumers + w] = sum;
    named_bar_sync(1, cthreads);
    sum = 0.f;
    for (int i = 0; i < kD1Consumers; ++i) sum += s.red[kD1Consumers + i];
    for (int e = ctid; e < E; e += cthreads) probs[e] = probs[e] / sum;
    named_bar_sync(1, cthreads);
    // selection by one warp: k rounds of two hardware warp reductions over keys held 8 (or 32) per lane
    if (w == 0) {
        if (E <= 256) select_warp<8>(probs, E, p.top_k, s.ids, s.weights, lane);
        else select_warp<32>(probs, E, p.top_k, s.ids, s.weights, lane);
    }
    named_bar_sync(1, cthreads);
    if (ctid < p.top_k) {
        float total = 0.f;
        for (int r = 0; r < p.top_k; ++r) total += s.weights[r];
        const float wgt = s.weights[ctid] / total;
        if (write_global) {
            p.topk_ids[ctid] = s.ids[ctid];
            p.topk_weights[ctid] = wgt;
            if (p.ids_mirror) p.ids_mirror[ctid] = s.ids[ctid];
            if (p.weights_mirror) p.weights_mirror[ctid] = wgt;
        }
        s.wnorm[ctid] = wgt;
    }
    named_bar_sync(1, cthreads);
}

__global__ void __launch_bounds__(kD1Threads, 1) decode1_kernel(DecodeParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    D1Smem& s = *reinterpret_cast<D1Smem*>(smem_raw);
    float* ract_s = reinterpret_cast<float*>(smem_raw + sizeof(D1Smem));          // [top_k][I]; softmax scratch before
    float* sact_s = ract_s + (size_t)FK_MAX_TOP_K * p.I;                          // [I]
    float* xg_s = sact_s + p.I;                                                   // [H]  x * (offset + norm_weight)
    unsigned char* xraw_s = reinterpret_cast<unsigned char*>(xg_s + p.H);         // [H] activations as stored (<= 4 bytes each)
    unsigned char* nw_s = xraw_s + (size_t)p.H * 4;                               // [H] bf16 norm weights
    unsigned char* uraw_s = nw_s + (size_t)p.H * 2;                               // [H] fp32 previous update (stack mode)
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = gridDim.x, blk = blockIdx.x;
    const int H = p.H, I = p.I;
    const int nchH = H / 256, nchI = I / 256;
    if (tid == 0) { D1_TRACE(0); if (p.trace) p.trace[(size_t)blk * 16 + 8] = (unsigned long long)clock64(); }

    // The producer warp prepares the ring itself (one slot per lane) and starts phase A before the block
    // meets: the first copies are then in flight while the consumers still wait for their activations.
    if (warp == kD1Consumers) {
        if (lane < kD1Stages) {
            mbar_init(&s.full[lane], 1);
            mbar_init(&s.empty[lane], 1);
        }
        if (lane == 0) {
            mbar_init(&s.ids_ready, 1);
            mbar_init(&s.xready, 1);
            mbar_init(&s.staged_a, 1);
            mbar_init(&s.staged_b, 1);
            s.abort_flag = 0;
        }
        mbar_init_fence();
        __syncwarp();
        // One copy of the token and of the norm weights per block.  (Plain loads by every consumer warp of
        // every block all hit the same few L2 lines and took 4 us to come back.)
        if (lane == 0) {
            if (p.resid_in) {
                const uint32_t rb = (uint32_t)H * 4u;
                mbar_expect_tx(&s.xready, rb + (p.update_in ? rb : 0u) + (uint32_t)H * 2u);
                bulk_load(xraw_s, p.resid_in, rb, &s.xready);
                if (p.update_in) bulk_load(uraw_s, p.update_in, rb, &s.xready);
            } else {
                const uint32_t xb = (uint32_t)H * (p.hidden_dtype == FK_F32 ? 4u : 2u);
                mbar_expect_tx(&s.xready, xb + (uint32_t)H * 2u);
                bulk_load(xraw_s, p.hidden, xb, &s.xready);
            }
            bulk_load(nw_s, p.norm_weight, (uint32_t)H * 2u, &s.xready);
        }
    }

    const D1Plan pl = make_plan(p, blk, G);
    const int nA = pl.nA_router + pl.nA_gate + pl.nA_pair;
    const int nB = pl.nB_pair + pl.nB_down;
    const int total = nA + nB + pl.nC;
    const __nv_bfloat16* router_w = reinterpret_cast<const __nv_bfloat16*>(p.router_weight);
    const __nv_bfloat16* gate_up = reinterpret_cast<const __nv_bfloat16*>(p.gate_up);
    const __nv_bfloat16* down = reinterpret_cast<const __nv_bfloat16*>(p.down);
    const __nv_bfloat16* sgu = reinterpret_cast<const __nv_bfloat16*>(p.shared_gate_up);
    const __nv_bfloat16* sdn = reinterpret_cast<const __nv_bfloat16*>(p.shared_down);

    if (warp == kD1Consumers) {
        // ------------------------------------------------------------------ producer warp
        // Lane l owns ring slot l: the lanes decode and issue up to kD1Stages stages side by side, so the
        // issue rate does not depend on one thread's instruction latency.
        auto issue = [&](int it, bool wait) {
            const D1Stage st = decode_stage(pl, p, it, blk, G);
            const int slot = it % kD1Stages;
            const uint32_t par = (it / kD1Stages) & 1u;
            const __nv_bfloat16 *src0 = nullptr, *src1 = nullptr;
            uint32_t bytes0 = 0, bytes1 = 0;
            switch (st.kind) {
                case kRouterRow: src0 = router_w + (size_t)st.a * H; bytes0 = H * 2; break;
                case kGateRow: src0 = reinterpret_cast<const __nv_bfloat16*>(p.shared_gate); bytes0 = H * 2; break;
                case kSharedPair:
                    src0 = sgu + (size_t)st.a * H; src1 = sgu + (size_t)(I + st.a) * H; bytes0 = bytes1 = H * 2; break;
                case kRoutedPair: {
                    const __nv_bfloat16* w = gate_up + (size_t)s.ids[st.a] * 2 * I * H;
                    src0 = w + (size_t)st.b * H; src1 = w + (size_t)(I + st.b) * H; bytes0 = bytes1 = H * 2; break;
                }
                case kSharedDown: src0 = sdn + (size_t)(pl.h0 + st.a) * I; bytes0 = st.b * I * 2; break;
                case kRoutedDown:
                    src0 = down + ((size_t)s.ids[st.a] * H + pl.h0 + st.b) * I; bytes0 = st.c * I * 2; break;
                default: break;
            }
            if (wait) mbar_wait(&s.empty[slot], par ^ 1u, &s.abort_flag);
            s.desc[slot] = make_int4(st.kind, st.a, st.b, st.c);
            mbar_expect_tx(&s.full[slot], bytes0 + bytes1);
            bulk_load(s.stage[slot], src0, bytes0, &s.full[slot]);
            if (bytes1) bulk_load(s.stage[slot] + bytes0, src1, bytes1, &s.full[slot]);
        };
        for (int base = 0; base < nA; base += kD1Stages) {            // phase A: static addresses
            const int it = base + lane;
            if (lane < kD1Stages && it < nA) issue(it, true);
        }
        __syncwarp();
        __syncthreads();                                               // the consumers may use the barriers from here on
        if (lane == 0) D1_TRACE(2);
        mbar_wait(&s.ids_ready, 0, &s.abort_flag);                     // the consumers select the experts
        if (lane == 0) D1_TRACE(4);
        // phases B and C: addresses depend on the ids only, so C is issued as soon as ring slots free up
        for (int base = (nA / kD1Stages) * kD1Stages; base < total; base += kD1Stages) {
            const int it = base + lane;
            if (lane < kD1Stages && it >= nA && it < total) issue(it, true);
        }
    } else {
        // ------------------------------------------------------------------ consumer warps
        __syncthreads();                                               // ring barriers initialised by the producer warp
        const int cthreads = kD1Consumers * 32;
        mbar_wait(&s.xready, 0, &s.abort_flag);
        // the token's activations, 8 consecutive columns of every 256-column chunk per lane
        float x[8][8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (j < nchH) {
                const size_t el = (size_t)j * 256 + lane * 8;
                if (p.resid_in) {
                    const uint4 a = lds128(xraw_s + el * 4), b = lds128(xraw_s + el * 4 + 16);
                    x[j][0] = __uint_as_float(a.x); x[j][1] = __uint_as_float(a.y); x[j][2] = __uint_as_float(a.z); x[j][3] = __uint_as_float(a.w);
                    x[j][4] = __uint_as_float(b.x); x[j][5] = __uint_as_float(b.y); x[j][6] = __uint_as_float(b.z); x[j][7] = __uint_as_float(b.w);
                    if (p.update_in) {
                        const uint4 c = lds128(uraw_s + el * 4), d = lds128(uraw_s + el * 4 + 16);
                        x[j][0] += __uint_as_float(c.x); x[j][1] += __uint_as_float(c.y); x[j][2] += __uint_as_float(c.z); x[j][3] += __uint_as_float(c.w);
                        x[j][4] += __uint_as_float(d.x); x[j][5] += __uint_as_float(d.y); x[j][6] += __uint_as_float(d.z); x[j][7] += __uint_as_float(d.w);
                    }
                } else if (p.hidden_dtype == FK_BF16) {
                    const uint4 v = lds128(xraw_s + el * 2);
                    x[j][0] = bf16lo(v.x); x[j][1] = bf16hi(v.x); x[j][2] = bf16lo(v.y); x[j][3] = bf16hi(v.y);
                    x[j][4] = bf16lo(v.z); x[j][5] = bf16hi(v.z); x[j][6] = bf16lo(v.w); x[j][7] = bf16hi(v.w);
                } else if (p.hidden_dtype == FK_F32) {
                    const uint4 a = lds128(xraw_s + el * 4), b = lds128(xraw_s + el * 4 + 16);
                    x[j][0] = __uint_as_float(a.x); x[j][1] = __uint_as_float(a.y); x[j][2] = __uint_as_float(a.z); x[j][3] = __uint_as_float(a.w);
                    x[j][4] = __uint_as_float(b.x); x[j][5] = __uint_as_float(b.y); x[j][6] = __uint_as_float(b.z); x[j][7] = __uint_as_float(b.w);
                } else {
                    const uint4 v = lds128(xraw_s + el * 2);
                    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 f = __half22float2(h[i]);
                        x[j][2 * i] = f.x; x[j][2 * i + 1] = f.y;
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) x[j][i] = 0.f;
            }
        }

        if (p.resid_in) {
            // layer-stack mode: x holds the new residual stream.  This block stores its slice of it, then the token
            // is its unit-gain RMS norm rounded to the activation dtype, exactly what a separate norm kernel would
            // have handed over.
            if (warp == 1) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int col = j * 256 + lane * 8 + i;
                        if (j < nchH && col >= pl.h0 && col < pl.h0 + pl.nh) p.resid_out[col] = x[j][i];
                    }
                }
            }
            float so = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
#pragma unroll
                for (int i = 0; i < 8; ++i) so = fmaf(x[j][i], x[j][i], so);
            }
            const float inv = rsqrtf(warp_sum(so) / (float)H + p.resid_eps);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float v = x[j][i] * inv;
                    x[j][i] = p.hidden_dtype == FK_BF16 ? __bfloat162float(__float2bfloat16_rn(v))
                            : (p.hidden_dtype == FK_F16 ? __half2float(__float2half_rn(v)) : v);
                }
            }
        }
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
#pragma unroll
            for (int i = 0; i < 8; ++i) ss = fmaf(x[j][i], x[j][i], ss);
        }
        const float rstd = rsqrtf(warp_sum(ss) / (float)H + p.eps);
        if (tid == 0) D1_TRACE(10);
        // warp 0 publishes x * gain for the router rows (rows are spread over the warps)
        if (warp == 0) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (j < nchH) {
                    const int c = j * 256 + lane * 8;
                    const uint4 g = lds128(nw_s + (size_t)c * 2);
                    const float o = p.norm_offset;
                    float4 lo = make_float4(x[j][0] * (o + bf16lo(g.x)), x[j][1] * (o + bf16hi(g.x)),
                                            x[j][2] * (o + bf16lo(g.y)), x[j][3] * (o + bf16hi(g.y)));
                    float4 hi = make_float4(x[j][4] * (o + bf16lo(g.z)), x[j][5] * (o + bf16hi(g.z)),
                                            x[j][6] * (o + bf16lo(g.w)), x[j][7] * (o + bf16hi(g.w)));
                    *reinterpret_cast<float4*>(xg_s + c) = lo;
                    *reinterpret_cast<float4*>(xg_s + c + 4) = hi;
                }
            }
        }
        named_bar_sync(1, cthreads);

        int phase = 0;
        for (int it = warp;;) {
            const int limit = phase == 0 ? nA : (phase == 1 ? nA + nB : total);
            if (it >= limit) {
                // phase boundary: every consumer warp passes here exactly once per phase
                if (phase == 0) {
                    // publish phase A (logits, shared activations, gate); when every block has, select the experts
                    if (tid == 0) D1_TRACE(13);
                    __threadfence();
                    if (tid == 0) D1_TRACE(14);
                    named_bar_sync(1, cthreads);
                    if (tid == 0) {
                        atomicAdd(p.bar + 0, 1u);
                        D1_TRACE(1);
                        spin_until(p.bar + 0, (unsigned)G, &s.abort_flag);
                        D1_TRACE(3);
                        // What the other blocks published is fetched by ONE bulk copy per block.  (Plain loads by
                        // every thread of every block pile thousands of requests onto a handful of L2 lines.)
                        fence_proxy_async();
                        const uint32_t sb = p.shared_gate_up ? (uint32_t)I * 4u : 0u;
                        mbar_expect_tx(&s.staged_a, (uint32_t)p.E * 4u + sb);
                        bulk_load(ract_s, p.logits, (uint32_t)p.E * 4u, &s.staged_a);
                        if (sb) bulk_load(sact_s, p.sact, sb, &s.staged_a);
                    }
                    if (!p.shared_gate_up && tid < I / 4) reinterpret_cast<float4*>(sact_s)[tid] = make_float4(0.f, 0.f, 0.f, 0.f);
                    named_bar_sync(1, cthreads);
                    mbar_wait(&s.staged_a, 0, &s.abort_flag);
                    block_topk(p, s, ract_s, tid, cthreads, blk == 0);
                    if (tid == 0) mbar_arrive(&s.ids_ready);
                    fence_proxy_async();              // the softmax scratch is overwritten by a bulk copy later
                    named_bar_sync(1, cthreads);
                } else if (phase == 1) {
                    // publish the routed activations, wait for every block's, stage them in shared memory
                    __threadfence();
                    named_bar_sync(1, cthreads);
                    if (tid == 0) {
                        atomicAdd(p.bar + 1, 1u);
                        D1_TRACE(5);
                        spin_until(p.bar + 1, (unsigned)G, &s.abort_flag);
                        D1_TRACE(6);
                        fence_proxy_async();
                        const uint32_t rb = (uint32_t)(p.top_k * I) * 4u;
                        mbar_expect_tx(&s.staged_b, rb);
                        bulk_load(ract_s, p.ract, rb, &s.staged_b);
                    }
                    named_bar_sync(1, cthreads);
                    mbar_wait(&s.staged_b, 0, &s.abort_flag);
                } else {
                    break;
                }
                ++phase;
                continue;
            }
            const int slot = it % kD1Stages;
            const uint32_t par = (it / kD1Stages) & 1u;
            mbar_wait(&s.full[slot], par, &s.abort_flag);
            if (tid == 0 && it == 0) D1_TRACE(11);
            const int4 st = s.desc[slot];                  // kind, a, b, c (see decode_stage)
            const unsigned char* base = s.stage[slot];
            float dep = 0.f;
            if (st.x == kSharedPair || st.x == kRoutedPair || st.x == kGateRow) {
                float g, u;
                pair_dot(base, base + (size_t)H * 2, x, lane, nchH, g, u);   // the gate row has no partner: u is unused
                dep = g + u;
                if (lane == 0) {
                    if (st.x == kGateRow) *p.sgate = sigmoidf_(g);
                    else if (st.x == kSharedPair) p.sact[st.y] = silu_mul(g, u);
                    else p.ract[(size_t)st.y * I + st.z] = silu_mul(g, u);
                }
            } else if (st.x == kRouterRow) {
                const float acc = row_dot_smem(base, xg_s, lane, nchH);
                dep = acc;
                if (lane == 0) {
                    float logit = acc * rstd;
                    if (p.router_bias) logit += p.router_bias[st.y];
                    p.logits[st.y] = logit;
                }
            } else {
                const bool routed = st.x == kRoutedDown;
                const float* vec = routed ? ract_s + (size_t)st.y * I : sact_s;
                const int row0 = routed ? st.z : st.y, nrows = routed ? st.w : st.z;
                // rows_per_stage <= 8 is checked on the host
                const float d = rows8_dot_smem(base, I * 2, nrows, vec, lane, nchI);
                dep = d;
                const int r = lane >> 2;
                if ((lane & 3) == 0 && r < nrows) {
                    if (routed) s.dpart[st.y][row0 + r] = d;
                    else s.ysh[row0 + r] = d;
                }
            }
            if (lane == 0) {
                // the data dependence keeps the release behind the last use of the stage
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&s.empty[slot])), "f"(dep) : "memory");
            }
            if (tid == 0 && it == 0) D1_TRACE(12);
            it += kD1Consumers;
        }

        named_bar_sync(1, cthreads);
        if (tid == 0) D1_TRACE(15);
        if (tid < pl.nh) {
            float acc = 0.f;
            for (int sl = 0; sl < p.top_k; ++sl) acc = fmaf(s.wnorm[sl], s.dpart[sl][tid], acc);
            if (p.shared_gate_up) {
                const float sh = s.ysh[tid];
                acc += p.shared_gate ? __ldcg(p.sgate) * sh : sh;
            }
            p.out[pl.h0 + tid] = acc;
            if (p.layer_hidden && !p.resid_in) p.layer_hidden[pl.h0 + tid] = load_any(p.hidden, p.hidden_dtype, (size_t)(pl.h0 + tid)) + acc;
        }
    }

    // leave: the last block to depart re-arms the barrier words for the next launch
    __syncthreads();
    if (tid == 0) {
        D1_TRACE(7);
        if (p.trace) p.trace[(size_t)blk * 16 + 9] = (unsigned long long)clock64();
        if (s.abort_flag && p.error_word) atomicExch(p.error_word, 2);
        __threadfence();
        const unsigned old = atomicAdd(p.bar + 2, 1u);
        if (old == (unsigned)G - 1) {
            p.bar[0] = 0u; p.bar[1] = 0u; p.bar[2] = 0u;
            __threadfence();
        }
    }
}

bool decode1_supported(const DecodeParams& p, int weight_dtype) {
    if (weight_dtype != FK_BF16) return false;
    if (p.H % 256 != 0 || p.H > 2048 || p.I % 256 != 0 || p.I > 512) return false;
    if (p.top_k < 1 || p.E < p.top_k) return false;
    const int G = sm_count();
    if ((p.H + G - 1) / G + 1 > kD1MaxRows) return false;
    uintptr_t bits = reinterpret_cast<uintptr_t>(p.hidden) | reinterpret_cast<uintptr_t>(p.norm_weight) |
                     reinterpret_cast<uintptr_t>(p.router_weight) | reinterpret_cast<uintptr_t>(p.gate_up) |
                     reinterpret_cast<uintptr_t>(p.down) | reinterpret_cast<uintptr_t>(p.shared_gate_up) |
                     reinterpret_cast<uintptr_t>(p.shared_down) | reinterpret_cast<uintptr_t>(p.shared_gate) |
                     reinterpret_cast<uintptr_t>(p.logits);
    if (p.E % 4 != 0) return false;            // the logits travel as one bulk copy
    bits |= reinterpret_cast<uintptr_t>(p.resid_in) | reinterpret_cast<uintptr_t>(p.update_in) | reinterpret_cast<uintptr_t>(p.resid_out);
    return (bits & 15) == 0;
}

int launch_decode1(const DecodeParams& p, cudaStream_t stream) {
    const int smem = (int)(sizeof(D1Smem) + sizeof(float) * ((size_t)(FK_MAX_TOP_K + 1) * p.I + p.H) + (size_t)p.H * 10 + 128);
    FK_CUDA_OK(cudaFuncSetAttribute(decode1_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "decode1 attr");
    DecodeParams copy = p;
    void* args[] = {&copy};
    FK_CUDA_OK(cudaLaunchCooperativeKernel((const void*)decode1_kernel, dim3(sm_count()), dim3(kD1Threads), args, smem, stream),
               "decode1 launch");
    note_launch();
    return FK_OK;
}

}  // namespace fk
