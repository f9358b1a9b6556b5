// Whole MoE layer for TWO TO FOUR tokens in one launch (bf16 weights and activations, H = 2048, I = 512), one block
// per SM.  Same construction as the single-token kernel (decode1.cu): weights stream through a 16-stage ring of
// 128-byte-swizzled TMA boxes and are multiplied with mma.sync (16 weight rows = M); the two grid-wide dependences of
// the layer (logits, activations) are exchanged as tagged 64-bit words instead of barriers; every wait is bounded.
// What is different with several tokens:
//
//   * the tokens are the N columns of the MMA (token t = column t), so a weight tile is read once for all tokens that
//     use it;
//   * experts chosen by more than one token are streamed once: after the select warps (one per token) have their
//     top-k, one of them builds the list of DISTINCT experts of the batch (warp match), with for every token the
//     routing slot and weight it gives that expert.  Every block derives the same list, so the work split needs no
//     communication: distinct expert u contributes 32 gate_up atoms (16 gate/up pairs each) dealt evenly over all
//     blocks, and one [16 x 512] down tile to every block that owns 16 output rows;
//   * activations travel as plain bf16 (what the grouped-GEMM path of larger batches does too) and are fetched with
//     bulk copies once a counter says that every block has published; the down products are weighted and summed
//     per token in registers, expert by expert in list order, so the result does not depend on scheduling;
//   * the experts are worked off in two halves with a counter each, so that the exchange of the first half's
//     activations runs under the second half's gate_up stream and the exchange of the second half's under the
//     first half's down tiles: neither exchange (a fence, a count, a 16 KB copy: 3 us) shows in the run time.
//
// The staged path (router, permutation, gate_up, down, combine: five launches) needs 49 us for four tokens, of which
// the 171 MB of weights account for 26 us at the copy bandwidth; the rest is the latency of five dependent launches.
//
// Reference math: src/fastkernels/reference/qwen36_real.py:329-354.

#include <cuda.h>

#include "common.cuh"
#include "decode_common.cuh"
#include "kernels.cuh"
#include "tcgen05.cuh"
#include "topk.cuh"

namespace fk {

constexpr int kFH = 2048, kFI = 512;             // the shape this kernel is built for
constexpr int kFMaxT = 4;                        // tokens per launch
constexpr int kFStages = 16;
constexpr int kFStageBytes = 8192;
constexpr int kFConsumers = 8;                   // warps
static_assert(kFStages % kFConsumers == 0, "every ring slot must belong to one consumer warp");
static_assert(kFH == kFConsumers * 256 && kFI == kFConsumers * 64, "one K-slice per consumer warp");
constexpr int kFThreads = (kFConsumers + 1 + kFMaxT) * 32;   // consumers + producer warp + one select warp per token
constexpr int kFTile = 16;                       // MMA M: gate (or up) rows per stage, output rows per block
constexpr int kFMaxRouterRows = 3;               // router rows of a block, the shared-expert gate vector included
static_assert((kFMaxRouterRows + 1) * kFMaxT == 16, "the router reduction below is written for 16 values per lane");
constexpr int kFMaxAtoms = 6;                    // gate_up atoms per block and half (the shared expert's one included)
constexpr int kFUnits = kFMaxT * FK_MAX_TOP_K;   // (token, routing slot) pairs = the most distinct experts
constexpr int kFActRows = kFUnits + kFMaxT;      // activation rows of I values: (token, slot), then the shared expert per token
constexpr int kFAtomsPerExpert = kFI / kFTile;   // 32
constexpr int kFWordsPerRow = kFI / 2;           // 32-bit words (two bf16) per activation row in global memory

struct FSmem {
    unsigned char stage[kFStages][kFStageBytes];                  // 1 KB aligned: the swizzle is a function of the address
    unsigned char sdown[kFConsumers][2048];                       // the shared expert's down tile, one [16 x 64] box per warp
    union {
        struct {
            unsigned char rrow[kFMaxRouterRows][kFH * 2];         // router rows as stored
            unsigned char xraw[kFMaxT][kFH * 2];                  // the tokens as stored (bf16)
            unsigned char nw[kFH * 2];                            // bf16 norm weights
        } in;                                                     // read until the tokens sit in registers (start of gate_up)
        unsigned char act[kFActRows * kFI * 2];                   // bf16 activations of all rows (written in the down phase)
    } u;
    float bpart[2 * kFMaxAtoms][kFConsumers][kFTile][kFMaxT];     // gate_up: K-slice sums per atom (gate, up), row, token; reused by the second half
    float cpart[2][kFConsumers][kFTile][kFMaxT];                  // down: K-slice sums, [0] routed (weighted), [1] shared expert
    float rpart[kFMaxRouterRows + 1][kFMaxT][kFConsumers];        // router rows: K-slice sums; last row: sum of squares
    uint64_t full[kFStages];
    uint64_t empty[kFStages];
    uint64_t xready;                              // tokens, norm weights and the launch tag are in shared memory
    uint64_t rrfull;                              // the router rows have landed
    uint64_t sdfull;                              // sdown has landed
    uint64_t rdone;                               // every warp has written its router K-slice sums
    uint64_t sel_done;                            // every select warp has written its token's ids and weights
    uint64_t plan_ready;                          // the distinct-expert list is complete
    uint64_t actfull[2];                          // the activation rows of a half have landed in shared memory
    uint64_t pubbar[2];                           // the consumers have stored this block's activations of a half
    float wnorm[kFMaxT][FK_MAX_TOP_K];            // renormalised routing weights
    int ids[kFMaxT][FK_MAX_TOP_K];
    int uexp[kFUnits];                            // distinct experts in order of first appearance in (token, slot) order
    float uw[kFUnits][kFMaxT];                    // routing weight token t gives distinct expert u (0: not chosen)
    int urow[kFUnits][kFMaxT];                    // activation row of that choice (rows are numbered expert by expert in list
                                                  // order, so a half's rows are contiguous), or -1
    float gate[kFMaxT];                           // sigmoid gate of the shared expert per token
    int U;                                        // number of distinct experts
    int rows0, rows;                              // activation rows of the first half, of both
    unsigned tag;                                 // this launch's tag for the exchanged words
    unsigned done_target;                         // value of the "activations published" counter once every block has added to it
    int abort_flag;
};

struct FPlan {
    int nrr;            // router rows of this block (gate vector included)
    int gate_row;       // index of the gate vector among them, or -1
    int shared_atom;    // the shared expert's gate_up atom of this block, or -1
    int tile;           // output tile, or -1
};

__device__ __forceinline__ FPlan few_static_plan(const DecodeParams& p, int b, int G) {
    FPlan pl;
    pl.nrr = b < p.E ? (p.E - b + G - 1) / G : 0;
    pl.gate_row = (p.shared_gate != nullptr && b == G - 1) ? pl.nrr : -1;
    if (pl.gate_row >= 0) pl.nrr += 1;
    pl.shared_atom = (p.shared_gate_up != nullptr && b < kFAtomsPerExpert) ? b : -1;
    pl.tile = b < kFH / kFTile ? b : -1;
    return pl;
}
// The distinct experts are worked off in two halves (the first one a multiple of four experts), each with its own
// "published" counter: while the second half's gate_up streams, the first half's activations are already exchanged,
// and while the second half's are exchanged, the first half's down tiles are multiplied.  Within a half the atoms are
// dealt round-robin over all blocks (so that the 32 atoms of one expert are streamed by 32 different SMs); the
// remainders of the two halves go to different blocks, and the blocks that hold a shared-expert atom come last.
struct FDyn {
    int U, U0;              // distinct experts; those of the first half
    int first0, cnt0;       // this block's atoms of the first half: first0 + k * G (k < cnt0) out of U0 * 32
    int first1, cnt1;       // ... of the second half, out of (U - U0) * 32, counted from atom U0 * 32
    int G;
};
// Atoms rb, rb + G, rb + 2 G, ... of `total`: consecutive atoms (the 32 of one expert) go to 32 different blocks.
__device__ __forceinline__ void few_deal(int total, int b, int G, int rot, int& first, int& count) {
    const int rb = (b + G - rot % G) % G;
    first = rb;
    count = rb < total ? (total - rb + G - 1) / G : 0;
}
__device__ __forceinline__ FDyn few_dynamic_plan(int U, int b, int G, bool has_shared) {
    FDyn d;
    d.G = G;
    d.U = min(max(U, 0), kFUnits);
    d.U0 = min(d.U, 4 * ((d.U + 7) / 8));
    const int rot0 = has_shared ? kFAtomsPerExpert : 0;
    few_deal(d.U0 * kFAtomsPerExpert, b, G, rot0, d.first0, d.cnt0);
    few_deal((d.U - d.U0) * kFAtomsPerExpert, b, G, rot0 + (d.U0 * kFAtomsPerExpert) % G, d.first1, d.cnt1);
    return d;
}
// global atom (expert * 32 + atom within the expert) of the block's k-th routed atom
__device__ __forceinline__ int few_atom(const FDyn& d, int k) {
    return k < d.cnt0 ? d.first0 + k * d.G : d.U0 * kFAtomsPerExpert + d.first1 + (k - d.cnt0) * d.G;
}

#define FEW_TRACE(slot) do { if (p.trace) p.trace[(size_t)blockIdx.x * 32 + (slot)] = global_ns(); } while (0)

__device__ __forceinline__ void few_barriers_ready_arrive() { asm volatile("bar.arrive 2, %0;" ::"r"(kFThreads) : "memory"); }
__device__ __forceinline__ void few_barriers_ready_wait() { asm volatile("bar.sync 2, %0;" ::"r"(kFThreads) : "memory"); }

// Select warp of token t: wait until every expert's logit of this token and launch has been published, softmax + top-k
// on the values the lanes already hold (lane L owns experts j*32 + L).
template <int EPL>
__device__ __forceinline__ void few_poll_and_select(const DecodeParams& p, FSmem& s, int t, int lane, bool write_global) {
    const unsigned tag = s.tag;
    const unsigned long long* src = p.tagged + (size_t)t * p.E;
    float v[EPL];
    const long long t0 = clock64();
    bool complete = true;
    for (;;) {
        unsigned long long w[EPL];
#pragma unroll
        for (int j = 0; j < EPL; ++j) {               // all loads in flight together: one round trip per poll
            const int e = j * 32 + lane;
            w[j] = e < p.E ? ld_relaxed_u64(src + e) : 0ull;
        }
        bool ok = true;
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
            const int e = j * 32 + lane;
            ok = ok & (e >= p.E || (unsigned)(w[j] >> 32) == tag);
            v[j] = e < p.E ? __uint_as_float((unsigned)w[j]) : -INFINITY;
        }
        if (__all_sync(kFull, ok)) break;
        if (clock64() - t0 > p.wait_cycles) { complete = false; break; }
        __nanosleep(32);       // polling warps of 148 blocks without a pause keep the publishing stores waiting
    }
    complete = __all_sync(kFull, complete);
    if (!complete && lane == 0) s.abort_flag = 1;
    if (t == 0 && lane == 0) FEW_TRACE(18);
    int my_i;
    float my_w;
    topk_warp_regs<EPL>(v, p.E, p.top_k, lane, my_i, my_w);
    if (lane < p.top_k) {
        s.ids[t][lane] = my_i;
        s.wnorm[t][lane] = my_w;
        if (write_global) {
            const size_t o = (size_t)t * p.top_k + lane;
            p.topk_ids[o] = my_i;
            p.topk_weights[o] = my_w;
            if (p.ids_mirror) p.ids_mirror[o] = my_i;
            if (p.weights_mirror) p.weights_mirror[o] = my_w;
        }
    }
    __syncwarp();
}

// "Token t does not use expert u" everywhere: done by the listing warp while it waits for the logits.
__device__ __forceinline__ void few_clear_plan(FSmem& s, int lane) {
    for (int i = lane; i < kFUnits * kFMaxT; i += 32) {
        (&s.uw[0][0])[i] = 0.f;
        (&s.urow[0][0])[i] = -1;
    }
    __syncwarp();
}

// The distinct experts of the batch, by one warp: lane i stands for (token i / top_k, slot i % top_k).
__device__ __forceinline__ void few_build_plan(const DecodeParams& p, FSmem& s, int lane) {
    const int n = p.T * p.top_k;
    const bool valid = lane < n;
    const int t = valid ? lane / p.top_k : 0, sl = valid ? lane % p.top_k : 0;
    const int id = valid ? s.ids[t][sl] : -1 - lane;                 // padding lanes match nobody
    const unsigned same = __match_any_sync(kFull, id);
    const bool leader = valid && (__ffs(same) - 1 == lane);
    const unsigned leaders = __ballot_sync(kFull, leader);
    const int u_of_leader = __popc(leaders & ((1u << lane) - 1u));
    const int u = __shfl_sync(kFull, u_of_leader, __ffs(same) - 1);   // the list position of this lane's expert
    if (leader) s.uexp[u] = id;
    // activation rows, expert by expert in list order, tokens ascending within an expert
    const int members = __popc(same);
    int base = leader ? members : 0;                                  // exclusive prefix sum over the leaders, in lane order
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int v = __shfl_up_sync(kFull, base, off);
        if (lane >= off) base += v;
    }
    base -= leader ? members : 0;
    const int row = __shfl_sync(kFull, base, __ffs(same) - 1) + __popc(same & ((1u << lane) - 1u));
    if (valid) {
        s.uw[u][t] = s.wnorm[t][sl];                                  // a token chooses an expert at most once
        s.urow[u][t] = row;
    }
    const int U = __popc(leaders);
    const int U0 = min(U, 4 * ((U + 7) / 8));
    const unsigned in_first = __ballot_sync(kFull, valid && u < U0);
    if (lane == 0) { s.U = U; s.rows0 = __popc(in_first); s.rows = n; }
    __syncwarp();
}

__global__ void __launch_bounds__(kFThreads, 1)
decode_few_kernel(const __grid_constant__ CUtensorMap gu_map, const __grid_constant__ CUtensorMap sgu_map,
                  const __grid_constant__ CUtensorMap dn_map, const __grid_constant__ CUtensorMap sdn_map, DecodeParams p) {
    extern __shared__ unsigned char smem_raw[];
    FSmem& s = *reinterpret_cast<FSmem*>(smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = gridDim.x, blk = blockIdx.x;
    constexpr int H = kFH, I = kFI;
    const int T = p.T;
    pdl_trigger();            // the next kernel in the stream may start its own constant loads as SMs free up
    if (tid == 0) FEW_TRACE(0);

    const FPlan pl = few_static_plan(p, blk, G);
    const bool has_shared = p.shared_gate_up != nullptr;
    unsigned long long* const gatew = p.actw + (size_t)kFActRows * kFWordsPerRow;     // one tagged word per token

    if (warp == kFConsumers) {
        // ------------------------------------------------------------------ producer warp
        if (lane < kFStages) {
            mbar_init(&s.full[lane], 1);
            mbar_init(&s.empty[lane], 1);
        }
        if (lane == 0) {
            mbar_init(&s.xready, 2);              // the copies' transaction count + the tag
            mbar_init(&s.rrfull, 1);
            mbar_init(&s.sdfull, 1);
            mbar_init(&s.rdone, kFConsumers);
            mbar_init(&s.sel_done, (uint32_t)T);
            mbar_init(&s.plan_ready, 1);
            mbar_init(&s.actfull[0], 1);
            mbar_init(&s.actfull[1], 1);
            mbar_init(&s.pubbar[0], 1);
            mbar_init(&s.pubbar[1], 1);
            s.abort_flag = 0;
            prefetch_tensormap(&gu_map);
            prefetch_tensormap(&dn_map);
        }
        mbar_init_fence();
        __syncwarp();
        few_barriers_ready_arrive();              // does not wait
        // routing-independent copies that do not go through the ring: the block's router rows ...
        if (lane == 0) mbar_expect_tx(&s.rrfull, (uint32_t)(pl.nrr * H * 2));
        __syncwarp();
        if (lane < pl.nrr) {
            const void* src = lane == pl.gate_row ? p.shared_gate
                                                  : (const void*)(reinterpret_cast<const __nv_bfloat16*>(p.router_weight) + (size_t)(blk + lane * G) * H);
            bulk_load(s.u.in.rrow[lane], src, (uint32_t)H * 2, &s.rrfull);
        }
        // ... and the shared expert's down tile of the block's output rows
        if (has_shared && pl.tile >= 0) {
            if (lane == 16) mbar_expect_tx(&s.sdfull, kFConsumers * 2048);
            __syncwarp();
            if (lane >= 16 && lane < 16 + kFConsumers)
                tma_load_2d(s.sdown[lane - 16], &sdn_map, (lane - 16) * 64, pl.tile * kFTile, &s.sdfull);
        }
        // Lane l owns ring slot l.  Stage n of consumer warp w is number it = 8 n + w of the block's queue: first the
        // gate_up stages (two per atom: the shared expert's atom, if the block has one, is known from the start), then
        // the down stages (four distinct experts each) of a block that owns output rows.
        const uint64_t wpolicy = l2_evict_first_policy();      // expert weights are read once per call: first out of L2
        const int nstatic = pl.shared_atom >= 0 ? 2 * kFConsumers : 0;
        int total = nstatic, nB = nstatic / kFConsumers;
        FDyn dyn{};
        bool token_issued = false, planned = false;
#pragma unroll 1
        for (int base = 0; base < total || !planned; base += kFStages) {
#pragma unroll 1
            for (int half = 0; half < 2; ++half) {
                const int it = base + lane;
                if (half == 1) {
                    if (!token_issued) {
                        token_issued = true;
                        pdl_wait();                               // the tokens (and the tag word) may come from the kernel before
                        if (lane == 0) FEW_TRACE(20);
                        if (lane == 0) {
                            mbar_expect_tx(&s.xready, (uint32_t)(T + 1) * (uint32_t)H * 2u);
                            for (int t = 0; t < T; ++t)
                                bulk_load(s.u.in.xraw[t], reinterpret_cast<const unsigned char*>(p.hidden) + (size_t)t * H * 2, (uint32_t)H * 2u, &s.xready);
                            bulk_load(s.u.in.nw, p.norm_weight, (uint32_t)H * 2u, &s.xready);
                            s.tag = ld_relaxed_u32(p.bar + 3) + 1u;
                            // word 1 counts the finished launches of this kernel on this workspace, words 0 and 2 the
                            // blocks that have published the activations of the first / second half of the experts
                            // (never reset: G more per launch)
                            s.done_target = (ld_relaxed_u32(p.bar + 1) + 1u) * (unsigned)G;
                            mbar_arrive(&s.xready);
                        }
                        __syncwarp();
                    }
                    if (!planned) {
                        planned = true;
                        if (lane == 0) {
                            const long long t0 = clock64();
                            while (!mbar_try_wait(&s.plan_ready, 0)) {
                                __nanosleep(32);
                                if (clock64() - t0 > kWaitCycles) { s.abort_flag = 1; break; }
                            }
                            FEW_TRACE(4);
                        }
                        __syncwarp();
                        dyn = few_dynamic_plan(*reinterpret_cast<volatile int*>(&s.U), blk, G, has_shared);
                        nB = nstatic / kFConsumers + 2 * (dyn.cnt0 + dyn.cnt1);
                        const int nC = pl.tile >= 0 ? (dyn.U + 3) / 4 : 0;
                        total = (nB + nC) * kFConsumers;
                    }
                }
                bool pending = lane < kFStages && it < total && ((it < nstatic) == (half == 0));
                const int n = it >> 3, w = it & 7;                // stage n of warp w
                const int slot = it % kFStages;
                const uint32_t par = (it / kFStages) & 1u;
                const long long t0 = clock64();
                while (__any_sync(kFull, pending)) {
                    bool go = false;
                    if (pending) {
                        go = mbar_test_wait(&s.empty[slot], par ^ 1u);         // passes at once on a slot's first lap
                        if (!go && clock64() - t0 > kWaitCycles) { s.abort_flag = 1; go = true; }
                    }
                    if (go) {
                        pending = false;
                        unsigned char* dst = s.stage[slot];
                        if (n < nB) {
                            // half n & 1 of an atom: columns [256 w + 128 (n & 1), + 128) of its 16 gate rows and of
                            // their up rows, as two copies of [2 halves x 16 rows x 64 columns] (4 KB each)
                            const CUtensorMap* map;
                            int y, z;
                            if (it < nstatic) {
                                map = &sgu_map;
                                y = pl.shared_atom * kFTile;
                                z = 0;
                            } else {
                                const int a = few_atom(dyn, (n - nstatic / kFConsumers) >> 1);
                                map = &gu_map;
                                y = (a % kFAtomsPerExpert) * kFTile;
                                z = 2 * s.uexp[a / kFAtomsPerExpert];
                            }
                            mbar_expect_tx(&s.full[slot], kFStageBytes);
#pragma unroll
                            for (int op = 0; op < 2; ++op)
                                tma_load_3d_hint(dst + op * 4096, map, w * 256 + (n & 1) * 128 + op * 64, y, z, &s.full[slot], wpolicy);
                        } else {
                            // Down tiles of a group of four distinct experts: warps 0-3 take the group's first two
                            // experts, warps 4-7 the other two, each a quarter of the columns (128) of the block's 16
                            // output rows: one copy of 4 KB per expert.  (Copies of 2 KB, four per stage, kept this
                            // warp busier issuing than the memory system delivering.)
                            const int c = n - nB;
                            const int nu = min(2, max(0, dyn.U - c * 4 - 2 * (w >> 2)));
                            mbar_expect_tx(&s.full[slot], (uint32_t)nu * 4096u);       // nothing to fetch: the arrival alone completes the phase
                            for (int q = 0; q < nu; ++q)
                                tma_load_3d_hint(dst + q * 4096, &dn_map, 0, 2 * (w & 3), s.uexp[c * 4 + 2 * (w >> 2) + q] * H + pl.tile * kFTile, &s.full[slot], wpolicy);
                        }
                    }
                    // no pause and no suspending wait here: a lane that sleeps holds up the lanes whose slots are free
                }
            }
        }
        if (lane == 0) FEW_TRACE(14);
    } else if (warp > kFConsumers) {
        // ------------------------------------------------------------------ select warps, one per token
        const int t = warp - kFConsumers - 1;
        few_barriers_ready_wait();
        if (t < T) {
            pdl_wait();
            if (t == 0) few_clear_plan(s, lane);
            mbar_wait_spin(&s.xready, 0, kWaitCycles, &s.abort_flag);      // the tag travels with the tokens
            if (p.E <= 256) few_poll_and_select<8>(p, s, t, lane, blk == 0);
            else few_poll_and_select<32>(p, s, t, lane, blk == 0);
            if (lane == 0) mbar_arrive(&s.sel_done);
            if (t == 0) {
                mbar_wait_spin(&s.sel_done, 0, kWaitCycles, &s.abort_flag);
                few_build_plan(p, s, lane);
                if (lane == 0) { mbar_arrive(&s.plan_ready); FEW_TRACE(19); }
                // afterwards this warp counts the block's two publications (see `publish` below)
                if (lane == 0) {
#pragma unroll 1
                    for (int which = 0; which < 2; ++which) {
                        mbar_wait(&s.pubbar[which], 0, &s.abort_flag);
                        __threadfence();
                        atomicAdd(p.bar + (which ? 2 : 0), 1u);
                    }
                }
            }
            if (t == 1 && pl.tile >= 0) {
                // This warp has nothing else to do: it fetches the activation rows for the block's down phase.  Per
                // half of the experts: watch the counter of the blocks that have published (one thread per block),
                // then one bulk copy of the half's rows (the shared expert's rows travel with the first half) into the
                // space the tokens and router rows no longer need.  (Tagged words, as for the logits, were tried
                // first: 1024 warps polling 9 MB of them took 7 us per round.)
                mbar_wait(&s.plan_ready, 0, &s.abort_flag);
                if (lane == 0) {
                    const unsigned char* src = reinterpret_cast<const unsigned char*>(p.act_rows);
                    const int rows0 = min(max(s.rows0, 0), kFUnits), rows = min(max(s.rows, rows0), kFUnits);
                    const long long t0 = clock64();
#pragma unroll 1
                    for (int half = 0; half < 2; ++half) {
                        const unsigned target = s.done_target;
                        const unsigned* counter = p.bar + (half ? 2 : 0);
                        while ((int)(ld_acquire_u32(counter) - target) < 0) {
                            if (clock64() - t0 > (s.abort_flag ? min(p.wait_cycles, kWaitCyclesAfterAbort) : p.wait_cycles)) { s.abort_flag = 1; break; }
                            __nanosleep(100);
                        }
                        FEW_TRACE(half ? 25 : 22);
                        asm volatile("fence.proxy.async;" ::: "memory");       // the copies read what other blocks' threads stored
                        const int r0 = half ? rows0 : 0, r1 = half ? rows : rows0;
                        const uint32_t routed_bytes = (uint32_t)(r1 - r0) * I * 2u;
                        const uint32_t shared_bytes = (half == 0 && has_shared) ? (uint32_t)T * I * 2u : 0u;
                        mbar_expect_tx(&s.actfull[half], routed_bytes + shared_bytes);      // no bytes: the arrival completes the phase
                        if (routed_bytes) bulk_load(s.u.act + (size_t)r0 * I * 2, src + (size_t)r0 * I * 2, routed_bytes, &s.actfull[half]);
                        if (shared_bytes) bulk_load(s.u.act + (size_t)kFUnits * I * 2, src + (size_t)kFUnits * I * 2, shared_bytes, &s.actfull[half]);
                    }
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ consumer warps
        const int cthreads = kFConsumers * 32;
        const int gid = lane >> 2, tig = lane & 3;
        // the router bias of this block's rows is a constant: fetched before the tokens arrive
        float bias_v = 0.f;
        if (warp == 0 && p.router_bias && lane < pl.nrr * T && lane / T != pl.gate_row) bias_v = __ldg(p.router_bias + blk + (lane / T) * G);
        few_barriers_ready_wait();
        pdl_wait();
        mbar_wait_spin(&s.xready, 0, kWaitCycles, &s.abort_flag);
        if (tid == 0) FEW_TRACE(2);

        // ---- router rows (and the shared-expert gate vector): K-slice sums on the CUDA cores, token by token
        {
            const int c0 = warp * 256 + lane * 8;
            const uint4 g = lds128(s.u.in.nw + (size_t)c0 * 2);
            const float o = p.norm_offset;
            float gw[8];
            gw[0] = o + bf16lo(g.x); gw[1] = o + bf16hi(g.x); gw[2] = o + bf16lo(g.y); gw[3] = o + bf16hi(g.y);
            gw[4] = o + bf16lo(g.z); gw[5] = o + bf16hi(g.z); gw[6] = o + bf16lo(g.w); gw[7] = o + bf16hi(g.w);
            mbar_wait(&s.rrfull, 0, &s.abort_flag);
            float rw[kFMaxRouterRows][8];
#pragma unroll
            for (int r = 0; r < kFMaxRouterRows; ++r) {
                uint4 w = make_uint4(0u, 0u, 0u, 0u);
                if (r < pl.nrr) w = lds128(s.u.in.rrow[r] + (size_t)c0 * 2);
                rw[r][0] = bf16lo(w.x); rw[r][1] = bf16hi(w.x); rw[r][2] = bf16lo(w.y); rw[r][3] = bf16hi(w.y);
                rw[r][4] = bf16lo(w.z); rw[r][5] = bf16hi(w.z); rw[r][6] = bf16lo(w.w); rw[r][7] = bf16hi(w.w);
            }
            // value r * 4 + t: this lane's part of row r against token t; 12 + t: of the token's sum of squares
            float v[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = 0.f;
#pragma unroll
            for (int t = 0; t < kFMaxT; ++t) {
                if (t < T) {
                    const uint4 xw = lds128(s.u.in.xraw[t] + (size_t)c0 * 2);
                    float xv[8];
                    xv[0] = bf16lo(xw.x); xv[1] = bf16hi(xw.x); xv[2] = bf16lo(xw.y); xv[3] = bf16hi(xw.y);
                    xv[4] = bf16lo(xw.z); xv[5] = bf16hi(xw.z); xv[6] = bf16lo(xw.w); xv[7] = bf16hi(xw.w);
                    float ss = 0.f;
#pragma unroll
                    for (int i = 0; i < 8; ++i) ss = fmaf(xv[i], xv[i], ss);
                    v[kFMaxRouterRows * 4 + t] = ss;
#pragma unroll
                    for (int r = 0; r < kFMaxRouterRows; ++r) {
                        const bool gate = r == pl.gate_row;            // the gate vector meets the raw token
                        float a0 = 0.f, a1 = 0.f;
#pragma unroll
                        for (int i = 0; i < 8; i += 2) {
                            a0 = fmaf(rw[r][i], gate ? xv[i] : xv[i] * gw[i], a0);
                            a1 = fmaf(rw[r][i + 1], gate ? xv[i + 1] : xv[i + 1] * gw[i + 1], a1);
                        }
                        v[r * 4 + t] = a0 + a1;
                    }
                }
            }
            // Sixteen sums over the warp in sixteen shuffles instead of eighty: at every level a lane hands over the half of
            // its values that its partner keeps, so that lane l ends up with the total of value l & 15.
#pragma unroll
            for (int half = 8; half >= 1; half >>= 1) {
                const bool up = (lane & half) != 0;
#pragma unroll
                for (int i = 0; i < half; ++i) {
                    const float send = up ? v[i] : v[i + half];
                    const float recv = __shfl_xor_sync(kFull, send, half);
                    v[i] = (up ? v[i + half] : v[i]) + recv;
                }
            }
            const float total = v[0] + __shfl_xor_sync(kFull, v[0], 16);
            if (lane < 16) s.rpart[lane >> 2][lane & 3][warp] = total;
            __syncwarp();
            if (lane == 0) mbar_arrive(&s.rdone);
            if (warp == 0) {
                // the eight K-slices meet here, in warp order; lane = row * T + token
                mbar_wait_spin(&s.rdone, 0, kWaitCycles, &s.abort_flag);
                if (lane < pl.nrr * T) {
                    const int r = lane / T, t = lane - r * T;
                    float acc = 0.f, sq = 0.f;
#pragma unroll
                    for (int w = 0; w < kFConsumers; ++w) { acc += s.rpart[r][t][w]; sq += s.rpart[kFMaxRouterRows][t][w]; }
                    if (r == pl.gate_row) {
                        atomicExch(gatew + t, ((unsigned long long)s.tag << 32) | (unsigned long long)__float_as_uint(sigmoidf_(acc)));
                    } else {
                        const int e = blk + r * G;
                        float logit = acc * rsqrtf(sq / (float)H + p.eps);
                        if (p.router_bias) logit += bias_v;
                        // an atomic is performed at L2 at once; a plain store is seen by the pollers much later
                        atomicExch(p.tagged + (size_t)t * p.E + e, ((unsigned long long)s.tag << 32) | (unsigned long long)__float_as_uint(logit));
                        p.logits[(size_t)t * p.E + e] = logit;
                    }
                }
                if (lane == 0) FEW_TRACE(3);
            }
        }

        // ---- gate_up: token gid is column gid of the MMA's B operand
        uint32_t bx[16][2];
#pragma unroll
        for (int ks = 0; ks < 16; ++ks) {
            const unsigned char* src = s.u.in.xraw[gid & (kFMaxT - 1)] + (size_t)(warp * 256 + ks * 16 + 2 * tig) * 2;
            bx[ks][0] = gid < T ? d1_lds32(src) : 0u;
            bx[ks][1] = gid < T ? d1_lds32(src + 16) : 0u;
        }
        const int sh = pl.shared_atom >= 0 ? 1 : 0;
        const unsigned tag = s.tag;
        FDyn dyn{};                                    // known once the distinct experts are listed
        // The K-slice sums of the block's atoms [j0, j1) meet (they sit in bpart from index 0 on); SwiGLU; the activations
        // go to global memory as plain bf16 pairs; then "this block has published half `which`": a thread of another
        // warp, which has met this block's threads at a barrier, fences (the block's stores are visible before the
        // count) and adds one.  Work item = (atom, pair of rows, token).
        auto publish = [&](int j0, int j1, int which) {
            named_bar_sync(1, cthreads);
            const int items = (j1 - j0) * (kFTile / 2) * T;
            for (int item = tid; item < items; item += cthreads) {
                const int t = item % T, rp = (item / T) % (kFTile / 2), jb = item / (T * (kFTile / 2)), j = j0 + jb;
                int row, atom_in_expert;
                if (j < sh) {
                    row = kFUnits + t;
                    atom_in_expert = pl.shared_atom;
                } else {
                    const int a = few_atom(dyn, j - sh);
                    row = s.urow[a / kFAtomsPerExpert][t];
                    atom_in_expert = a % kFAtomsPerExpert;
                }
                if (row < 0) continue;                                // this token did not choose the expert
                float acts[2];
#pragma unroll
                for (int k2 = 0; k2 < 2; ++k2) {
                    const int r = 2 * rp + k2;
                    float gsum = 0.f, usum = 0.f;
#pragma unroll
                    for (int w = 0; w < kFConsumers; ++w) { gsum += s.bpart[2 * jb][w][r][t]; usum += s.bpart[2 * jb + 1][w][r][t]; }
                    acts[k2] = silu_mul(gsum, usum);
                }
                p.act_rows[(size_t)row * kFWordsPerRow + atom_in_expert * (kFTile / 2) + rp] =
                    (unsigned)__bfloat16_as_ushort(__float2bfloat16_rn(acts[0])) |
                    ((unsigned)__bfloat16_as_ushort(__float2bfloat16_rn(acts[1])) << 16);
            }
            named_bar_sync(1, cthreads);
            // the fence takes a microsecond or two under load: it is left to a warp that has nothing else to do
            if (tid == 0) { mbar_arrive(&s.pubbar[which]); FEW_TRACE(which ? 5 : 21); }
        };
        int n_first = sh, natoms = sh;                 // atoms of the first half (the shared expert's included), of both halves
        bool planned = false, published0 = false;
#pragma unroll 1
        for (int j = 0; ; ++j) {
            if (j >= natoms && !planned) {
                planned = true;
                mbar_wait(&s.plan_ready, 0, &s.abort_flag);
                dyn = few_dynamic_plan(s.U, blk, G, has_shared);
                n_first = sh + dyn.cnt0;
                natoms = n_first + dyn.cnt1;
            }
            if (planned && !published0 && j == n_first) {
                published0 = true;
                publish(0, n_first, 0);
            }
            if (j >= natoms) break;
            const int jb = j < n_first ? j : j - n_first;      // the second half reuses the K-slice sum buffers
            // a stage holds four boxes: gate and up rows over columns [0, 64) of the stage, then over [64, 128)
            float gs[4] = {0.f, 0.f, 0.f, 0.f}, us[4] = {0.f, 0.f, 0.f, 0.f};   // rows gid, gid + 8 x tokens 2 tig, 2 tig + 1
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int it = (2 * j + h) * kFConsumers + warp;
                const int slot = it % kFStages;
                mbar_wait(&s.full[slot], (it / kFStages) & 1u, &s.abort_flag);
                if (tid == 0 && j == 0 && h == 0) FEW_TRACE(11);
                const uint32_t base = smem_u32(s.stage[slot]);
                float c[8][4];                             // gate: c[0..3], up: c[4..7]; two per box: dependent MMAs wait for each other
#pragma unroll
                for (int q = 0; q < 8; ++q) { c[q][0] = c[q][1] = c[q][2] = c[q][3] = 0.f; }
                {
                    uint32_t a[4][4][4];
#pragma unroll
                    for (int sl = 0; sl < 4; ++sl) box_load(a[sl], base + sl * 2048, lane);
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
                        for (int sl = 0; sl < 4; ++sl) {
                            const int ks = h * 8 + (sl >> 1) * 4 + kk;          // k-step within the warp's 256 columns
                            d1_mma(c[(sl & 1) * 4 + (sl >> 1) * 2 + (kk & 1)], a[sl][kk], bx[ks][0], bx[ks][1]);
                        }
                    }
                }
                float dep = 0.f;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float gv = (c[0][i] + c[1][i]) + (c[2][i] + c[3][i]);
                    const float uv = (c[4][i] + c[5][i]) + (c[6][i] + c[7][i]);
                    gs[i] += gv; us[i] += uv;
                    dep += gv + uv;
                }
                if (lane == 0) d1_release(&s.empty[slot], dep);
            }
            if (tig < 2) {
                *reinterpret_cast<float2*>(&s.bpart[2 * jb][warp][gid][2 * tig]) = make_float2(gs[0], gs[1]);
                *reinterpret_cast<float2*>(&s.bpart[2 * jb][warp][gid + 8][2 * tig]) = make_float2(gs[2], gs[3]);
                *reinterpret_cast<float2*>(&s.bpart[2 * jb + 1][warp][gid][2 * tig]) = make_float2(us[0], us[1]);
                *reinterpret_cast<float2*>(&s.bpart[2 * jb + 1][warp][gid + 8][2 * tig]) = make_float2(us[2], us[3]);
            }
        }
        publish(n_first, natoms, 1);

        if (pl.tile >= 0) {
            // ---- down: the block's 16 output rows for every token
            const int U = dyn.U;
            float resid_v = 0.f;
            if (tid < kFTile * T && p.layer_hidden)
                resid_v = load_any(p.hidden, p.hidden_dtype, (size_t)(tid / kFTile) * H + pl.tile * kFTile + (tid % kFTile));
            const bool want_gate = has_shared && p.shared_gate != nullptr;
            if (warp == 0 && lane < T) {
                float gv = 1.f;
                if (want_gate) {
                    unsigned long long gw2 = 0ull;
                    const long long t0 = clock64();
                    for (;;) {
                        gw2 = ld_relaxed_u64(gatew + lane);
                        if ((unsigned)(gw2 >> 32) == tag) break;
                        if (clock64() - t0 > (s.abort_flag ? min(p.wait_cycles, kWaitCyclesAfterAbort) : p.wait_cycles)) { s.abort_flag = 1; break; }
                        __nanosleep(64);
                    }
                    gv = __uint_as_float((unsigned)gw2);
                }
                s.gate[lane] = gv;
            }
            __syncwarp();
            mbar_wait(&s.actfull[0], 0, &s.abort_flag);       // the first half's rows (fetched by a select warp)
            if (tid == 0) FEW_TRACE(12);
            // B fragments of activation row `row` (or zeros when negative) of this lane's token: k-steps from column col0 on
            auto act_frag = [&](int row, int col0, auto& b) {
                const unsigned char* src = s.u.act + ((size_t)max(row, 0) * I + col0 + 2 * tig) * 2;
#pragma unroll
                for (int kk = 0; kk < (int)(sizeof(b) / sizeof(b[0])); ++kk) {
                    b[kk][0] = row >= 0 ? d1_lds32(src + kk * 32) : 0u;
                    b[kk][1] = row >= 0 ? d1_lds32(src + kk * 32 + 16) : 0u;
                }
            };
            float acc[4] = {0.f, 0.f, 0.f, 0.f};          // rows gid, gid + 8 x tokens 2 tig, 2 tig + 1, routing weights applied
            const int nC = (U + 3) / 4;
            const int nB = 2 * natoms;
            const int first_of_second_half = dyn.U0 < U ? dyn.U0 / 4 : nC;        // U0 is a multiple of four when U0 < U
            const int hf = warp >> 2, qd = warp & 3;      // which two experts of a group, which quarter of the columns
#pragma unroll 1
            for (int cst = 0; cst < nC; ++cst) {
                if (cst == first_of_second_half) mbar_wait(&s.actfull[1], 0, &s.abort_flag);
                const int it = (nB + cst) * kFConsumers + warp;
                const int slot = it % kFStages;
                mbar_wait(&s.full[slot], (it / kFStages) & 1u, &s.abort_flag);
                if (tid == 0 && cst == 0) FEW_TRACE(26);
                const uint32_t base = smem_u32(s.stage[slot]);
                const int nu = min(2, max(0, U - cst * 4 - 2 * hf));
                // The stage goes into registers and the slot back to the producer before the arithmetic: a warp has
                // two slots, and a slot held for the whole computation caps its stream at two stages per (refill
                // latency + computation).  A [16 rows x 128 columns] box holds row r as lines 2 r (columns 0-63) and
                // 2 r + 1 (columns 64-127); the 16-byte chunk c of a line sits at chunk c ^ (line & 7).
                uint32_t a[2][8][4];
                {
                    const int row = (lane & 7) + ((lane >> 3) & 1) * 8, sel = lane >> 4;
#pragma unroll
                    for (int q = 0; q < 2; ++q) {
#pragma unroll
                        for (int kk = 0; kk < 8; ++kk) {
                            const int line = row * 2 + (kk >> 2);
                            d1_ldmatrix_x4(a[q][kk], base + q * 4096 + line * 128 + (((2 * (kk & 3) + sel) ^ (line & 7)) << 4));
                        }
                    }
                    uint32_t dep = 0u;
#pragma unroll
                    for (int q = 0; q < 2; ++q) {
#pragma unroll
                        for (int kk = 0; kk < 8; ++kk) dep ^= a[q][kk][0];
                    }
                    if (lane == 0) d1_release_u(&s.empty[slot], dep);
                }
                if (nu > 0) {
                    // both boxes together: all fragment loads first, then four independent MMA chains
                    const int u0 = cst * 4 + 2 * hf, u1 = nu > 1 ? u0 + 1 : -1;
                    uint32_t b0[8][2], b1[8][2];
                    act_frag(gid < T ? s.urow[u0][gid & (kFMaxT - 1)] : -1, qd * 128, b0);
                    act_frag(gid < T && u1 >= 0 ? s.urow[u1][gid & (kFMaxT - 1)] : -1, qd * 128, b1);
                    const int ta = (2 * tig) & (kFMaxT - 1), tb = (2 * tig + 1) & (kFMaxT - 1);
                    const float w0a = tig < 2 ? s.uw[u0][ta] : 0.f, w0b = tig < 2 ? s.uw[u0][tb] : 0.f;
                    const float w1a = (tig < 2 && u1 >= 0) ? s.uw[u1][ta] : 0.f, w1b = (tig < 2 && u1 >= 0) ? s.uw[u1][tb] : 0.f;
                    float c0[2][4], c1[2][4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) { c0[0][i] = c0[1][i] = c1[0][i] = c1[1][i] = 0.f; }
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk) {
                        d1_mma(c0[kk & 1], a[0][kk], b0[kk][0], b0[kk][1]);
                        d1_mma(c1[kk & 1], a[1][kk], b1[kk][0], b1[kk][1]);
                    }
                    // a column whose token did not choose the expert is left out rather than added with weight 0
                    // (0 x a non-finite product would not be 0)
                    acc[0] = w0a != 0.f ? fmaf(w0a, c0[0][0] + c0[1][0], acc[0]) : acc[0];
                    acc[1] = w0b != 0.f ? fmaf(w0b, c0[0][1] + c0[1][1], acc[1]) : acc[1];
                    acc[2] = w0a != 0.f ? fmaf(w0a, c0[0][2] + c0[1][2], acc[2]) : acc[2];
                    acc[3] = w0b != 0.f ? fmaf(w0b, c0[0][3] + c0[1][3], acc[3]) : acc[3];
                    acc[0] = w1a != 0.f ? fmaf(w1a, c1[0][0] + c1[1][0], acc[0]) : acc[0];
                    acc[1] = w1b != 0.f ? fmaf(w1b, c1[0][1] + c1[1][1], acc[1]) : acc[1];
                    acc[2] = w1a != 0.f ? fmaf(w1a, c1[0][2] + c1[1][2], acc[2]) : acc[2];
                    acc[3] = w1b != 0.f ? fmaf(w1b, c1[0][3] + c1[1][3], acc[3]) : acc[3];
                }
                if (tid == 0 && cst == 0) FEW_TRACE(27);
            }
            // the shared expert: one box, every token a column
            float cs[4] = {0.f, 0.f, 0.f, 0.f};
            if (has_shared) {
                mbar_wait(&s.sdfull, 0, &s.abort_flag);
                uint32_t b[4][2], a[4][4];
                act_frag(gid < T ? kFUnits + gid : -1, warp * 64, b);
                box_load(a, smem_u32(s.sdown[warp]), lane);
                float c[2][4];
#pragma unroll
                for (int i = 0; i < 4; ++i) c[0][i] = c[1][i] = 0.f;
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) d1_mma(c[kk & 1], a[kk], b[kk][0], b[kk][1]);
#pragma unroll
                for (int i = 0; i < 4; ++i) cs[i] = c[0][i] + c[1][i];
            }
            if (tig < 2) {
                *reinterpret_cast<float2*>(&s.cpart[0][warp][gid][2 * tig]) = make_float2(acc[0], acc[1]);
                *reinterpret_cast<float2*>(&s.cpart[0][warp][gid + 8][2 * tig]) = make_float2(acc[2], acc[3]);
                *reinterpret_cast<float2*>(&s.cpart[1][warp][gid][2 * tig]) = make_float2(cs[0], cs[1]);
                *reinterpret_cast<float2*>(&s.cpart[1][warp][gid + 8][2 * tig]) = make_float2(cs[2], cs[3]);
            }
            named_bar_sync(1, cthreads);
            if (tid == 0) FEW_TRACE(13);
            if (tid < kFTile * T) {
                // thread (token, row): the eight K-slices in warp order, then the gated shared expert
                const int t = tid / kFTile, row = tid % kFTile;
                float routed = 0.f, shared = 0.f;
#pragma unroll
                for (int w = 0; w < kFConsumers; ++w) { routed += s.cpart[0][w][row][t]; shared += s.cpart[1][w][row][t]; }
                const float outv = has_shared ? fmaf(s.gate[t], shared, routed) : routed;
                const size_t o = (size_t)t * H + pl.tile * kFTile + row;
                p.out[o] = outv;
                if (p.layer_hidden) p.layer_hidden[o] = resid_v + outv;
            }
            if (tid == 0) FEW_TRACE(15);
        }
    }

    __syncthreads();
    if (tid == 0) {
        FEW_TRACE(7);
        if (s.abort_flag && p.error_word) atomicExch(p.error_word, 2);
        // Block 0 owns an output tile, so it has seen every block's activations, and a block publishes those after it
        // has read the launch tag: all blocks have read it by now, and block 0 advances it for the next launch.
        if (blk == 0) { p.bar[3] = s.tag; p.bar[1] = p.bar[1] + 1u; }
    }
}

static size_t decode_few_smem_bytes() { return sizeof(FSmem) + 1024; }

// one block per SM must fit (checked once per device)
static bool decode_few_resident() {
    static int cached[64] = {0};          // 0 unknown, 1 yes, -1 no
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    if (cached[dev] == 0) {
        const int smem = (int)decode_few_smem_bytes();
        int n = 0;
        bool ok = cudaFuncSetAttribute(decode_few_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) == cudaSuccess &&
                  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, decode_few_kernel, kFThreads, smem) == cudaSuccess && n >= 1;
        if (!ok) (void)cudaGetLastError();
        cached[dev] = ok ? 1 : -1;
    }
    return cached[dev] == 1;
}

bool decode_few_supported(const DecodeParams& p, int weight_dtype) {
    if (weight_dtype != FK_BF16 || p.hidden_dtype != FK_BF16) return false;
    if (p.T < 2 || p.T > kFMaxT) return false;
    if (p.H != kFH || p.I != kFI) return false;
    if (p.top_k < 1 || p.top_k > FK_MAX_TOP_K || p.E < p.top_k || p.E > FK_MAX_EXPERTS) return false;
    if (p.resid_in != nullptr) return false;                                   // the layer-stack form is single-token only
    if ((size_t)p.T * p.E > FK_MAX_EXPERTS) return false;                      // tagged logit words of the workspace
    const int G = sm_count();
    if (G < kFH / kFTile) return false;                                        // every output tile needs a block
    if ((p.E + G - 1) / G + (p.shared_gate ? 1 : 0) > kFMaxRouterRows) return false;
    if (((p.E + G - 1) / G + (p.shared_gate ? 1 : 0)) * p.T > 32) return false;      // one lane per (row, token)
    if ((kFUnits / 2 * kFAtomsPerExpert + G - 1) / G + 1 > kFMaxAtoms) return false;       // atoms of a block per half
    if (p.act_rows == nullptr || (reinterpret_cast<uintptr_t>(p.act_rows) & 15)) return false;
    uintptr_t bits = reinterpret_cast<uintptr_t>(p.hidden) | reinterpret_cast<uintptr_t>(p.norm_weight) |
                     reinterpret_cast<uintptr_t>(p.router_weight) | reinterpret_cast<uintptr_t>(p.gate_up) |
                     reinterpret_cast<uintptr_t>(p.down) | reinterpret_cast<uintptr_t>(p.shared_gate_up) |
                     reinterpret_cast<uintptr_t>(p.shared_down) | reinterpret_cast<uintptr_t>(p.shared_gate) |
                     reinterpret_cast<uintptr_t>(p.tagged) | reinterpret_cast<uintptr_t>(p.actw);
    if (bits & 15) return false;
    return decode_few_resident();
}

int launch_decode_few(const DecodeParams& p, cudaStream_t stream) {
    // same switch as the single-token kernel: a cooperative launch guarantees that all blocks are resident together,
    // at the price of the overlap with the previous kernel's tail
    static const bool cooperative = [] { const char* e = getenv("FKMOE_D1_COOPERATIVE"); return e && e[0] == '1'; }();
    const int smem = (int)decode_few_smem_bytes();
    FK_CUDA_OK(cudaFuncSetAttribute(decode_few_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "decode_few attr");
    // gate_up: [2 halves x 16 rows x 64 columns] boxes; down: [16 rows x 2 x 64 columns] boxes (shared expert: [16 x 64]);
    // 128-byte swizzle, cached per weight pointer
    CUtensorMap gu{}, sgu{}, dn{}, sdn{};
    const bool maps = gate_up_pair_map(p.gate_up, (uint64_t)p.E, p.I, p.H, kFTile, &gu) &&
                      column_pair_map(p.down, (uint64_t)p.E * p.H, p.I, kFTile, &dn) &&
                      gate_up_pair_map(p.shared_gate_up ? p.shared_gate_up : p.gate_up, 1, p.I, p.H, kFTile, &sgu) &&
                      weight_tensor_map(p.shared_down ? p.shared_down : p.down, (uint64_t)p.H, p.I, kFTile, &sdn);
    if (!maps) return FK_ERR_UNSUPPORTED;
    DecodeParams q = p;
    if (q.wait_cycles <= 0) q.wait_cycles = wait_limit_cycles();
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(sm_count());
    cfg.blockDim = dim3(kFThreads);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (cooperative) {
        attr[0].id = cudaLaunchAttributeCooperative;
        attr[0].val.cooperative = 1;
        cfg.numAttrs = 1;
    } else {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.numAttrs = pdl_enabled() ? 1 : 0;
    }
    cfg.attrs = attr;
    FK_CUDA_OK(cudaLaunchKernelEx(&cfg, decode_few_kernel, gu, sgu, dn, sdn, q), "decode_few launch");
    note_launch();
    return FK_OK;
}

}  // namespace fk
