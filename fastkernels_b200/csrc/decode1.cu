// Whole MoE layer for ONE token in one launch (bf16 weights and activations, H = 2048, I = 512), one block per SM.
//
// The layer has three dependent steps (router -> gate_up of the selected experts -> down), and at this size
// every dependent step costs about as much as streaming its weights.  The kernel is laid out around the
// dependences and around the instruction count of the warps that consume the stream:
//
//   start   every block issues ALL of its routing-independent copies at once: its router rows, its gate_up tiles
//           of the shared expert (ring stages) and the shared expert's down tile (a buffer of its own), before it
//           even has the token.  Weights are constants, so with programmatic dependent launch these copies run
//           while the kernel before this one in the stream drains.
//   logits  each router row's logit is published as one 64-bit word (launch tag << 32 | logit bits).  A select
//           warp in every block polls the E words until all carry this launch's tag: arrival and data are one
//           load, no fence, no counter, no second round trip.  The same warp then runs softmax + top-k on the
//           values it already holds in registers, and the producer warp starts the experts' copies at once.
//   B       the selected experts' gate and up tiles stream through the 16-stage ring; the down tiles follow in
//           the same queue as ring slots free up (their addresses depend on the ids only), so HBM stays busy
//           across the second grid-wide dependence.
//   sync    the SwiGLU activations travel like the logits: one 64-bit word each (tag << 32 | bf16 head << 16 |
//           bf16 remainder), and every warp polls just the words of its own K-slice.  (A counter barrier cost
//           3 us here: a fence under load, the counter's round trip, then an 18 KB copy of all activations.)
//   C       down tiles of the block's 16 output rows, summed in slot order with the routing weights, plus the
//           gated shared expert (and the residual).
//
// Consumers.  Warp w owns columns [256 w, 256 w + 256) of the hidden dimension (phase B) and [64 w, 64 w + 64) of
// the intermediate dimension (phase C).  A stage is 8 KB of weights in 128-byte-swizzled TMA boxes of 16 rows x 64
// columns: in phase B 16 gate rows and their 16 up rows over 128 columns (two copies through a 3-D view of the
// gate_up tensor, each bringing a gate box and its up box: copies of 2 KB streamed at 5.5 TB/s in a stand-alone
// probe, copies of 4 KB at 6.1), in phase C the down tiles of four slots.  Boxes are read with ldmatrix and
// multiplied on the tensor cores (mma.sync m16n8k16, bf16 in, fp32 accumulate): the sixteen weight rows are the
// M rows, the token is column 0 of N.  Seven of the eight N columns are wasted, and
// it is still five times fewer instructions than unpacking bf16 pairs and issuing one FMA per weight, which is what
// bounded this kernel before (each warp issued ~4300 instructions at ~6 stall cycles each).  Products of bf16
// values are exact in fp32, so the sums differ from a CUDA-core dot product only in their order.  The fp32 SwiGLU
// activations enter the down MMAs as a bf16 head plus a bf16 remainder (relative error 2^-17).  The eight K-slices
// of a tile meet in shared memory.  The router rows (at most three per block) stay on the CUDA cores, one K-slice
// per warp, because their operand x * (offset + norm_weight) is an fp32 value.
//
// The launch is not cooperative: 148 blocks of one block per SM become resident together as soon as the SMs are
// free, and every wait on another block is bounded (it gives up, raises the error word and lets the kernel
// finish).  That allows the programmatic-dependent-launch attribute, which a cooperative launch does not take.
// FKMOE_D1_COOPERATIVE=1 selects a cooperative launch without the overlap.
//
// Reference math: src/fastkernels/reference/qwen36_real.py:329-354.

#include <cuda.h>

#include <cstdlib>

#include "common.cuh"
#include "decode_common.cuh"
#include "kernels.cuh"
#include "tcgen05.cuh"
#include "topk.cuh"

namespace fk {

constexpr int kD1H = 2048, kD1I = 512;           // the shape this kernel is built for
constexpr int kD1Stages = 16;
constexpr int kD1StageBytes = 8192;
constexpr int kD1Consumers = 8;                  // warps
// Stage `it` lives in slot it % kD1Stages and is consumed by warp it % kD1Consumers.  The slot count must be a
// multiple of the warp count: then a slot always belongs to the same warp, which meets its laps in order.  With
// any other ratio another warp can reach lap k of a slot while lap k-1 is still in flight (bulk copies complete
// out of order, e.g. after a TLB miss), and a one-bit phase parity cannot tell "lap k landed" from "lap k-1 has
// not landed yet": the warp would read the slot early and release it twice.
static_assert(kD1Stages % kD1Consumers == 0, "every ring slot must belong to one consumer warp");
static_assert(kD1H == kD1Consumers * 256 && kD1I == kD1Consumers * 64, "one K-slice per consumer warp");
constexpr int kD1Threads = (kD1Consumers + 2) * 32;   // consumers + producer warp + select warp
constexpr int kD1Tile = 16;                      // MMA M: gate (or up) rows per stage, output rows per block
constexpr int kD1MaxRouterRows = 4;              // router rows of a block, the shared-expert gate vector included
constexpr int kD1MaxAtoms = 4;                   // gate_up atoms (16 gate/up pairs of one expert) per block
constexpr int kD1ActElems = (FK_MAX_TOP_K + 1) * kD1I;
constexpr int kD1IdValid = 1 << 30;              // flag bit of D1Smem::ids

struct D1Smem {
    unsigned char stage[kD1Stages][kD1StageBytes];                // 1 KB aligned: the swizzle is a function of the address
    unsigned char sdown[kD1Consumers][2048];                      // the shared expert's down tile, one [16 x 64] box per warp
    unsigned char rrow[kD1MaxRouterRows][kD1H * 2];               // router rows as stored
    unsigned char xraw[kD1H * 4];                                 // the token as stored (bf16), or the fp32 residual stream
    unsigned char uraw[kD1H * 4];                                 // fp32 update of the previous layer (stack mode)
    unsigned char nw[kD1H * 2];                                   // bf16 norm weights
    unsigned char xb[kD1H * 2];                                   // stack mode: the normed token in bf16
    unsigned char act_hi[kD1ActElems * 2];                        // all blocks' activations, bf16 head ...
    unsigned char act_lo[kD1ActElems * 2];                        // ... and bf16 remainder
    float bpart[2 * kD1MaxAtoms][kD1Consumers][kD1Tile];          // phase B: K-slice sums per stage
    float cpart[FK_MAX_TOP_K + 1][kD1Consumers][kD1Tile];         // phase C: K-slice sums per slot (slot top_k = shared expert)
    float rpart[kD1MaxRouterRows + 1][kD1Consumers];              // router rows: K-slice sums; last row: sum of squares
    float sopart[kD1Consumers];                                   // stack mode: K-slice sums of squares of the residual
    uint64_t full[kD1Stages];
    uint64_t empty[kD1Stages];
    uint64_t xready;                              // the token, the norm weights and the launch tag are in shared memory
    uint64_t rrfull;                              // the router rows have landed
    uint64_t sdfull;                              // sdown has landed
    uint64_t rdone;                               // every warp has written its router K-slice sums
    uint64_t ids_ready;                           // ids / wnorm written by the select warp
    float wnorm[FK_MAX_TOP_K];                    // renormalised routing weights
    int ids[FK_MAX_TOP_K];                        // expert | kD1IdValid, written round by round while the select warp runs
    unsigned tag;                                 // this launch's tag for the published logits
    int abort_flag;
};

// Static split of the work among the G blocks.
//   router   block b takes rows b, b + G, ...; the last block also takes the shared-expert gate vector.
//   gate_up  "atoms" of 16 gate/up pairs of one expert: first the shared expert's (I/16), then the routed experts'
//            (top_k * I/16, in the order of d1_routed_atom), dealt evenly.  (The blocks meet between gate_up and down, so each of
//            the two phases has to be balanced by itself: giving the blocks without an output tile more atoms
//            made everybody wait for them.)
//   down     block b < H/16 owns output rows [16 b, 16 b + 16); the other blocks leave after gate_up.
struct D1Plan {
    int nrr;            // router rows of this block (gate vector included)
    int gate_row;       // index of the gate vector among them, or -1
    int atom0, atoms;   // first global atom, number of atoms
    int shared_atoms;   // global atoms [0, shared_atoms) belong to the shared expert
    int tile;           // output tile, or -1
    int nB;             // ring stages of phase B per warp (2 per atom)
    int nC;             // ring stages of phase C per warp (4 slots per stage)
};

__device__ __forceinline__ D1Plan make_plan(const DecodeParams& p, int b, int G) {
    D1Plan pl;
    pl.nrr = b < p.E ? (p.E - b + G - 1) / G : 0;
    pl.gate_row = (p.shared_gate != nullptr && b == G - 1) ? pl.nrr : -1;
    if (pl.gate_row >= 0) pl.nrr += 1;
    const int per_expert = kD1I / kD1Tile;
    pl.shared_atoms = p.shared_gate_up ? per_expert : 0;
    const int total = pl.shared_atoms + p.top_k * per_expert;
    const int tiles = kD1H / kD1Tile;                      // G >= tiles is checked on the host
    const int q = total / G, r = total - q * G;
    pl.tile = b < tiles ? b : -1;
    pl.atom0 = b * q + min(b, r);
    pl.atoms = q + (b < r ? 1 : 0);
    pl.nB = 2 * pl.atoms;
    pl.nC = pl.tile >= 0 ? (p.top_k + 3) / 4 : 0;
    return pl;
}

// The q-th routed gate_up atom in dealing order -> its position slot * (I / 16) + pair16.  The winners arrive slot by
// slot while the select warp runs its rounds, so consecutive atoms alternate between the first and the last slots:
// every block then holds one atom it can start early, and all blocks finish the phase together.
__device__ __forceinline__ int d1_routed_atom(int q, int nq) { return (q & 1) ? nq - 1 - (q >> 1) : (q >> 1); }

// optional trace: p.trace[block][slot] = nanosecond timestamp of a phase boundary (32 words per block;
// words 8 and 9 hold the SM cycle counter at start and exit); the slots are listed in include/fkmoe.h
#define D1_TRACE(slot) do { if (p.trace) p.trace[(size_t)blockIdx.x * 32 + (slot)] = global_ns(); } while (0)

// "The mbarriers are initialised": the producer warp arrives on named barrier 2 without waiting, every other warp
// waits there once before its first use of an mbarrier.
__device__ __forceinline__ void barriers_ready_arrive() { asm volatile("bar.arrive 2, %0;" ::"r"(kD1Threads) : "memory"); }
__device__ __forceinline__ void barriers_ready_wait() { asm volatile("bar.sync 2, %0;" ::"r"(kD1Threads) : "memory"); }

// The expert of routing slot `sl` (the select warp publishes expert | kD1IdValid round by round; the rounds run while
// the first slots' copies are already on their way).  0 if it never came: the launch then reports a time-out.
__device__ __forceinline__ int d1_id(D1Smem& s, int sl) {
    return *reinterpret_cast<volatile int*>(&s.ids[sl]) & (kD1IdValid - 1);
}

// Select warp: wait until every expert's logit of this launch has been published, then softmax + top-k on the
// values the lanes already hold (lane L owns experts j*32 + L).  Writes ids / renormalised weights to shared memory
// (and to the outputs from block 0).
template <int EPL>
__device__ __forceinline__ void poll_and_select(const DecodeParams& p, D1Smem& s, int lane, bool write_global) {
    const unsigned tag = s.tag;
    float v[EPL];
    const long long t0 = clock64();
    bool complete = true;
    for (;;) {
        unsigned long long w[EPL];
#pragma unroll
        for (int j = 0; j < EPL; ++j) {               // all loads in flight together: one round trip per poll
            const int e = j * 32 + lane;
            w[j] = e < p.E ? ld_relaxed_u64(p.tagged + e) : 0ull;
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
        __nanosleep(32);       // 148 warps polling without a pause keep the publishing stores waiting for microseconds
    }
    complete = __all_sync(kFull, complete);
    if (lane == 0) D1_TRACE(18);
    if (!complete && lane == 0) s.abort_flag = 1;
    int my_i;
    float my_w;
    // every winner is handed to the producer warp as soon as its round is over: the blocks whose gate_up tiles belong
    // to the first slots start their copies a microsecond before the last round and the weights are done
    topk_warp_regs<EPL>(v, p.E, p.top_k, lane, my_i, my_w, [&](int r, int expert) {
        if (lane == 0) *reinterpret_cast<volatile int*>(&s.ids[r]) = expert | kD1IdValid;     // id and "valid" in one word: no fence
    });
    if (lane < p.top_k) {
        s.wnorm[lane] = my_w;
        if (write_global) {
            p.topk_ids[lane] = my_i;
            p.topk_weights[lane] = my_w;
            if (p.ids_mirror) p.ids_mirror[lane] = my_i;
            if (p.weights_mirror) p.weights_mirror[lane] = my_w;
        }
    }
    __syncwarp();
}

__global__ void __launch_bounds__(kD1Threads, 1)
decode1_kernel(const __grid_constant__ CUtensorMap gu_map, const __grid_constant__ CUtensorMap sgu_map,
               const __grid_constant__ CUtensorMap dn_map, const __grid_constant__ CUtensorMap sdn_map, DecodeParams p) {
    extern __shared__ unsigned char smem_raw[];
    D1Smem& s = *reinterpret_cast<D1Smem*>(smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = gridDim.x, blk = blockIdx.x;
    constexpr int H = kD1H, I = kD1I;
    pdl_trigger();            // the next kernel in the stream may start its own constant loads as SMs free up
    if (tid == 0) { D1_TRACE(0); if (p.trace) p.trace[(size_t)blk * 32 + 8] = (unsigned long long)clock64(); }

    const D1Plan pl = make_plan(p, blk, G);
    const bool has_shared = p.shared_gate_up != nullptr;
    const int shared_slot = p.top_k;                       // index of the shared expert in the activation arrays

    if (warp == kD1Consumers) {
        // ------------------------------------------------------------------ producer warp
        if (lane < kD1Stages) {
            mbar_init(&s.full[lane], 1);
            mbar_init(&s.empty[lane], 1);
        }
        if (lane < FK_MAX_TOP_K) s.ids[lane] = 0;
        if (lane == 0) {
            mbar_init(&s.xready, 2);              // the copies' transaction count + the tag
            mbar_init(&s.rrfull, 1);
            mbar_init(&s.sdfull, 1);
            mbar_init(&s.rdone, kD1Consumers);
            mbar_init(&s.ids_ready, 1);
            s.abort_flag = 0;
            prefetch_tensormap(&gu_map);
            prefetch_tensormap(&dn_map);
        }
        mbar_init_fence();
        __syncwarp();
        barriers_ready_arrive();                  // does not wait
        // routing-independent copies that do not go through the ring: the block's router rows ...
        if (lane == 0) mbar_expect_tx(&s.rrfull, (uint32_t)(pl.nrr * H * 2));
        __syncwarp();
        if (lane < pl.nrr) {
            const void* src = lane == pl.gate_row ? p.shared_gate
                                                  : (const void*)(reinterpret_cast<const __nv_bfloat16*>(p.router_weight) + (size_t)(blk + lane * G) * H);
            bulk_load(s.rrow[lane], src, (uint32_t)H * 2, &s.rrfull);
        }
        // ... and the shared expert's down tile of the block's output rows
        if (has_shared && pl.tile >= 0) {
            if (lane == 16) mbar_expect_tx(&s.sdfull, kD1Consumers * 2048);
            __syncwarp();
            if (lane >= 16 && lane < 16 + kD1Consumers)
                tma_load_2d(s.sdown[lane - 16], &sdn_map, (lane - 16) * 64, pl.tile * kD1Tile, &s.sdfull);
        }
        // Lane l owns ring slot l: the lanes issue up to kD1Stages stages side by side.  One loop (one copy of the
        // issue code) serves all phases.  Its first lap issues the stages that depend neither on the routing nor
        // on the kernel before this one (the shared expert's gate_up tiles); the token follows as soon as that
        // kernel has completed; stages whose addresses depend on the ids wait for the select warp; the down tiles
        // are issued as ring slots free up.
        const uint64_t wpolicy = l2_evict_first_policy();      // expert weights are read once per call: first out of L2
        const int nstatic = 2 * max(0, min(pl.atoms, pl.shared_atoms - pl.atom0)) * kD1Consumers;   // stages of shared atoms
        const int total = (pl.nB + pl.nC) * kD1Consumers;
        bool token_issued = false;
#pragma unroll 1
        for (int base = 0; base < total || !token_issued; base += kD1Stages) {
#pragma unroll 1
            for (int half = 0; half < 2; ++half) {
                const int it = base + lane;
                if (half == 1) {
                    if (!token_issued) {
                        token_issued = true;
                        if (lane == 0) D1_TRACE(1);
                        pdl_wait();                               // the token (and the barrier words) may come from the kernel before
                        if (lane == 0) D1_TRACE(20);
                        if (lane == 0) {
                            // One copy of the token and of the norm weights per block.  (Plain loads by every consumer
                            // warp of every block all hit the same few L2 lines and took 4 us to come back.)
                            if (p.resid_in) {
                                const uint32_t rb = (uint32_t)H * 4u;
                                mbar_expect_tx(&s.xready, rb + (p.update_in ? rb : 0u) + (uint32_t)H * 2u);
                                bulk_load(s.xraw, p.resid_in, rb, &s.xready);
                                if (p.update_in) bulk_load(s.uraw, p.update_in, rb, &s.xready);
                            } else {
                                mbar_expect_tx(&s.xready, (uint32_t)H * 4u);
                                bulk_load(s.xraw, p.hidden, (uint32_t)H * 2u, &s.xready);
                            }
                            bulk_load(s.nw, p.norm_weight, (uint32_t)H * 2u, &s.xready);
                            // this launch's tag: one load per block, handed to the other warps with the token
                            s.tag = ld_relaxed_u32(p.bar + 3) + 1u;
                            mbar_arrive(&s.xready);
                        }
                        __syncwarp();
                    }
                }
                // Every lane polls its own slot and issues the moment the slot is free and the ids its addresses need
                // are known: at the turn from gate_up to down the copies of a freed slot must not wait for the
                // slowest slot of the lap (nor for a sleeping poll loop: that cost a microsecond there).
                bool pending = lane < kD1Stages && it < total && ((it < nstatic) == (half == 0));
                const int n = it >> 3, w = it & 7;                // stage n of warp w
                const int slot = it % kD1Stages;
                const uint32_t par = (it / kD1Stages) & 1u;
                int q = -1, id_last = -1;                         // routed atom; the last routing slot whose id is needed
                if (pending) {
                    if (n >= pl.nB) {
                        id_last = min((n - pl.nB) * 4 + 4, p.top_k) - 1;
                    } else if (pl.atom0 + (n >> 1) >= pl.shared_atoms) {
                        q = d1_routed_atom(pl.atom0 + (n >> 1) - pl.shared_atoms, p.top_k * (I / kD1Tile));
                        id_last = q / (I / kD1Tile);
                    }
                }
                const long long t0 = clock64();
                while (__any_sync(kFull, pending)) {
                    bool go = false;
                    if (pending) {
                        go = mbar_try_wait(&s.empty[slot], par ^ 1u);          // passes at once on a slot's first lap
                        if (go && id_last >= 0) go = (*reinterpret_cast<volatile int*>(&s.ids[id_last]) & kD1IdValid) != 0;
                        if (!go && clock64() - t0 > kWaitCycles) { s.abort_flag = 1; go = true; }
                    }
                    if (go) {
                        pending = false;
                        unsigned char* dst = s.stage[slot];
                        if (n < pl.nB) {
                            // half n & 1 of atom n / 2: columns [256 w + 128 (n & 1), + 128) of the 16 gate rows and
                            // of their up rows, as two copies of [2 halves x 16 rows x 64 columns] (4 KB each)
                            const CUtensorMap* map;
                            int y, z;
                            if (q < 0) {
                                map = &sgu_map;
                                y = (pl.atom0 + (n >> 1)) * kD1Tile;
                                z = 0;
                            } else {
                                map = &gu_map;
                                y = (q % (I / kD1Tile)) * kD1Tile;
                                z = 2 * d1_id(s, id_last);
                            }
                            mbar_expect_tx(&s.full[slot], kD1StageBytes);
#pragma unroll
                            for (int op = 0; op < 2; ++op)
                                tma_load_3d_hint(dst + op * 4096, map, w * 256 + (n & 1) * 128 + op * 64, y, z, &s.full[slot], wpolicy);
                        } else {
                            // down tiles of four slots, columns [64 w, 64 w + 64) of the block's 16 output rows
                            const int c = n - pl.nB;
                            const int nu = min(4, p.top_k - c * 4);
                            mbar_expect_tx(&s.full[slot], (uint32_t)nu * 2048u);
                            for (int u = 0; u < nu; ++u)
                                tma_load_2d_hint(dst + u * 2048, &dn_map, w * 64, d1_id(s, c * 4 + u) * H + pl.tile * kD1Tile, &s.full[slot], wpolicy);
                        }
                        if (it == nstatic) D1_TRACE(4);
                    } else if (pending) {
                        __nanosleep(20);          // this warp shares its scheduler with warps that have work
                    }
                }
            }
        }
        if (lane == 0) D1_TRACE(14);
    } else if (warp == kD1Consumers + 1) {
        // ------------------------------------------------------------------ select warp
        barriers_ready_wait();
        pdl_wait();
        mbar_wait_spin(&s.xready, 0, kWaitCycles, &s.abort_flag);      // the tag travels with the token
        if (p.E <= 256) poll_and_select<8>(p, s, lane, blk == 0);
        else poll_and_select<32>(p, s, lane, blk == 0);
        if (lane == 0) { mbar_arrive(&s.ids_ready); D1_TRACE(19); }
    } else {
        // ------------------------------------------------------------------ consumer warps
        const int cthreads = kD1Consumers * 32;
        const int gid = lane >> 2, tig = lane & 3;
        // the router bias of this block's rows is a constant: fetched before the token arrives
        float bias_v = 0.f;
        if (warp == 0 && p.router_bias && lane < pl.nrr && lane != pl.gate_row) bias_v = __ldg(p.router_bias + blk + lane * G);
        barriers_ready_wait();
        pdl_wait();
        mbar_wait_spin(&s.xready, 0, kWaitCycles, &s.abort_flag);
        if (tid == 0) D1_TRACE(2);

        // ---- the token: this lane's 8 columns of the warp's K-slice
        const int c0 = warp * 256 + lane * 8;
        float xv[8];
        const unsigned char* xsrc = s.xraw;                    // bf16 source of the MMA B operand
        if (p.resid_in) {
            // layer-stack mode: the new residual stream is resid_in + update_in; the block stores its 16 columns of
            // it, and the token is its unit-gain RMS norm rounded to bf16, exactly what a separate norm kernel
            // would have handed over
            const uint4 a = lds128(s.xraw + (size_t)c0 * 4), b = lds128(s.xraw + (size_t)c0 * 4 + 16);
            xv[0] = __uint_as_float(a.x); xv[1] = __uint_as_float(a.y); xv[2] = __uint_as_float(a.z); xv[3] = __uint_as_float(a.w);
            xv[4] = __uint_as_float(b.x); xv[5] = __uint_as_float(b.y); xv[6] = __uint_as_float(b.z); xv[7] = __uint_as_float(b.w);
            if (p.update_in) {
                const uint4 c = lds128(s.uraw + (size_t)c0 * 4), d = lds128(s.uraw + (size_t)c0 * 4 + 16);
                xv[0] += __uint_as_float(c.x); xv[1] += __uint_as_float(c.y); xv[2] += __uint_as_float(c.z); xv[3] += __uint_as_float(c.w);
                xv[4] += __uint_as_float(d.x); xv[5] += __uint_as_float(d.y); xv[6] += __uint_as_float(d.z); xv[7] += __uint_as_float(d.w);
            }
            if (pl.tile >= 0 && c0 >= pl.tile * kD1Tile && c0 < (pl.tile + 1) * kD1Tile) {
                *reinterpret_cast<float4*>(p.resid_out + c0) = make_float4(xv[0], xv[1], xv[2], xv[3]);
                *reinterpret_cast<float4*>(p.resid_out + c0 + 4) = make_float4(xv[4], xv[5], xv[6], xv[7]);
            }
            float so = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) so = fmaf(xv[i], xv[i], so);
            so = warp_sum(so);
            if (lane == 0) s.sopart[warp] = so;
            named_bar_sync(1, cthreads);
            float tot = 0.f;
#pragma unroll
            for (int w = 0; w < kD1Consumers; ++w) tot += s.sopart[w];
            const float inv = rsqrtf(tot / (float)H + p.resid_eps);
            __nv_bfloat162 packed[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                packed[i] = __floats2bfloat162_rn(xv[2 * i] * inv, xv[2 * i + 1] * inv);
                const float2 f = __bfloat1622float2(packed[i]);
                xv[2 * i] = f.x; xv[2 * i + 1] = f.y;
            }
            *reinterpret_cast<uint4*>(s.xb + (size_t)c0 * 2) = *reinterpret_cast<const uint4*>(packed);
            __syncwarp();                                      // the warp reads back only its own K-slice
            xsrc = s.xb;
        } else {
            const uint4 v = lds128(s.xraw + (size_t)c0 * 2);
            xv[0] = bf16lo(v.x); xv[1] = bf16hi(v.x); xv[2] = bf16lo(v.y); xv[3] = bf16hi(v.y);
            xv[4] = bf16lo(v.z); xv[5] = bf16hi(v.z); xv[6] = bf16lo(v.w); xv[7] = bf16hi(v.w);
        }

        // ---- router rows (and the shared-expert gate vector): K-slice sums on the CUDA cores
        {
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) ss = fmaf(xv[i], xv[i], ss);
            const uint4 g = lds128(s.nw + (size_t)c0 * 2);
            const float o = p.norm_offset;
            float xg[8];
            xg[0] = xv[0] * (o + bf16lo(g.x)); xg[1] = xv[1] * (o + bf16hi(g.x)); xg[2] = xv[2] * (o + bf16lo(g.y)); xg[3] = xv[3] * (o + bf16hi(g.y));
            xg[4] = xv[4] * (o + bf16lo(g.z)); xg[5] = xv[5] * (o + bf16hi(g.z)); xg[6] = xv[6] * (o + bf16lo(g.w)); xg[7] = xv[7] * (o + bf16hi(g.w));
            mbar_wait(&s.rrfull, 0, &s.abort_flag);
            // all rows' K-slice sums are reduced together (independent shuffle chains), then lane r keeps row r
            float racc[kD1MaxRouterRows + 1];
#pragma unroll
            for (int r = 0; r < kD1MaxRouterRows; ++r) {
                racc[r] = 0.f;
                if (r < pl.nrr) {
                    const uint4 w = lds128(s.rrow[r] + (size_t)c0 * 2);
                    const bool gate = r == pl.gate_row;            // the gate vector meets the raw token
                    float a0, a1;
                    a0 = bf16lo(w.x) * (gate ? xv[0] : xg[0]);       a1 = bf16hi(w.x) * (gate ? xv[1] : xg[1]);
                    a0 = fmaf(bf16lo(w.y), gate ? xv[2] : xg[2], a0); a1 = fmaf(bf16hi(w.y), gate ? xv[3] : xg[3], a1);
                    a0 = fmaf(bf16lo(w.z), gate ? xv[4] : xg[4], a0); a1 = fmaf(bf16hi(w.z), gate ? xv[5] : xg[5], a1);
                    a0 = fmaf(bf16lo(w.w), gate ? xv[6] : xg[6], a0); a1 = fmaf(bf16hi(w.w), gate ? xv[7] : xg[7], a1);
                    racc[r] = a0 + a1;
                }
            }
            racc[kD1MaxRouterRows] = ss;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
                for (int r = 0; r <= kD1MaxRouterRows; ++r) racc[r] += __shfl_xor_sync(kFull, racc[r], o);
            }
            if (lane == 0) {
#pragma unroll
                for (int r = 0; r <= kD1MaxRouterRows; ++r) s.rpart[r][warp] = racc[r];
                mbar_arrive(&s.rdone);
            }
            __syncwarp();
            if (warp == 0) {
                // the eight K-slices meet here, in warp order
                mbar_wait_spin(&s.rdone, 0, kWaitCycles, &s.abort_flag);
                if (lane < pl.nrr) {
                    float acc = 0.f, sq = 0.f;
#pragma unroll
                    for (int w = 0; w < kD1Consumers; ++w) { acc += s.rpart[lane][w]; sq += s.rpart[kD1MaxRouterRows][w]; }
                    if (lane == pl.gate_row) {
                        atomicExch(p.actw + (size_t)(FK_MAX_TOP_K + 1) * I,
                                   ((unsigned long long)s.tag << 32) | (unsigned long long)__float_as_uint(sigmoidf_(acc)));
                    } else {
                        const int e = blk + lane * G;
                        float logit = acc * rsqrtf(sq / (float)H + p.eps);
                        if (p.router_bias) logit += bias_v;
                        // an atomic is performed at L2 at once; a plain store was seen by the pollers a microsecond later
                        atomicExch(p.tagged + e, ((unsigned long long)s.tag << 32) | (unsigned long long)__float_as_uint(logit));
                        p.logits[e] = logit;
                    }
                }
                if (lane == 0) D1_TRACE(3);
            }
        }

        // ---- phase B: gate and up tiles against the token (column 0 of the MMA's B operand lives in lanes 0..3)
        uint32_t bx[16][2];
#pragma unroll
        for (int ks = 0; ks < 16; ++ks) {
            const unsigned char* src = xsrc + (size_t)(warp * 256 + ks * 16 + 2 * tig) * 2;
            bx[ks][0] = gid == 0 ? d1_lds32(src) : 0u;
            bx[ks][1] = gid == 0 ? d1_lds32(src + 16) : 0u;
        }
#pragma unroll 1
        for (int j = 0; j < pl.atoms; ++j) {
            // a stage holds four boxes: gate and up rows over columns [0, 64) of the stage, then over [64, 128)
            float g0 = 0.f, g2 = 0.f, u0 = 0.f, u2 = 0.f;       // tile rows gid and gid + 8 (lanes with tig == 0)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int it = (2 * j + h) * kD1Consumers + warp;
                const int slot = it % kD1Stages;
                mbar_wait(&s.full[slot], (it / kD1Stages) & 1u, &s.abort_flag);
                if (tid == 0 && j == 0 && h == 0) D1_TRACE(11);
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
                const float gs0 = (c[0][0] + c[1][0]) + (c[2][0] + c[3][0]), gs2 = (c[0][2] + c[1][2]) + (c[2][2] + c[3][2]);
                const float us0 = (c[4][0] + c[5][0]) + (c[6][0] + c[7][0]), us2 = (c[4][2] + c[5][2]) + (c[6][2] + c[7][2]);
                g0 += gs0; g2 += gs2; u0 += us0; u2 += us2;
                if (lane == 0) d1_release(&s.empty[slot], (gs0 + gs2) + (us0 + us2));
            }
            if (tig == 0) {
                s.bpart[2 * j][warp][gid] = g0;
                s.bpart[2 * j][warp][gid + 8] = g2;
                s.bpart[2 * j + 1][warp][gid] = u0;
                s.bpart[2 * j + 1][warp][gid + 8] = u2;
            }
        }
        // the K-slices of every tile meet; SwiGLU; each activation is published as one tagged word (an atomic is
        // performed at L2 at once and nobody waits for it)
        named_bar_sync(1, cthreads);
        const unsigned tag = s.tag;
        if (tid < pl.atoms * kD1Tile) {
            const int j = tid >> 4, r = tid & 15;
            float gsum = 0.f, usum = 0.f;
#pragma unroll
            for (int w = 0; w < kD1Consumers; ++w) { gsum += s.bpart[2 * j][w][r]; usum += s.bpart[2 * j + 1][w][r]; }
            const float act = silu_mul(gsum, usum);
            const int g = pl.atom0 + j;
            int idx;
            if (g < pl.shared_atoms) idx = shared_slot * I + g * kD1Tile + r;
            else idx = d1_routed_atom(g - pl.shared_atoms, p.top_k * (I / kD1Tile)) * kD1Tile + r;     // slot * I + pair
            const __nv_bfloat16 hi = __float2bfloat16_rn(act);
            const __nv_bfloat16 lo = __float2bfloat16_rn(act - __bfloat162float(hi));
            const unsigned payload = ((unsigned)__bfloat16_as_ushort(hi) << 16) | (unsigned)__bfloat16_as_ushort(lo);
            atomicExch(p.actw + idx, ((unsigned long long)tag << 32) | (unsigned long long)payload);
        }
        if (tid == 0) D1_TRACE(5);

        if (pl.tile >= 0) {
            // ---- phase C: the block's 16 output rows
            // what the output rows need from global memory is fetched while the activations are on their way
            float resid_v = 0.f;
            if (tid < kD1Tile * kD1Consumers && p.layer_hidden && !p.resid_in)
                resid_v = load_any(p.hidden, p.hidden_dtype, (size_t)(pl.tile * kD1Tile + (tid >> 3)));
            // This warp's K-slice of every slot's activations (64 words per slot, two per lane), polled until all
            // carry this launch's tag; lane 0 also takes the shared-expert gate.
            const int nslots = p.top_k + (has_shared ? 1 : 0);
            const bool want_gate = has_shared && p.shared_gate != nullptr;
            float gate_v = 1.f;
            {
                unsigned long long w[2 * (FK_MAX_TOP_K + 1)];
                unsigned long long gw = 0ull;
                const unsigned long long* src = p.actw + warp * 64 + lane;
                const long long t0 = clock64();
                for (;;) {
#pragma unroll
                    for (int sl = 0; sl <= FK_MAX_TOP_K; ++sl) {
                        w[2 * sl] = sl < nslots ? ld_relaxed_u64(src + (size_t)sl * I) : 0ull;
                        w[2 * sl + 1] = sl < nslots ? ld_relaxed_u64(src + (size_t)sl * I + 32) : 0ull;
                    }
                    if (want_gate && lane == 0) gw = ld_relaxed_u64(p.actw + (size_t)(FK_MAX_TOP_K + 1) * I);
                    bool ok = !(want_gate && lane == 0) || (unsigned)(gw >> 32) == tag;
#pragma unroll
                    for (int sl = 0; sl <= FK_MAX_TOP_K; ++sl)
                        ok = ok & (sl >= nslots || ((unsigned)(w[2 * sl] >> 32) == tag && (unsigned)(w[2 * sl + 1] >> 32) == tag));
                    if (__all_sync(kFull, ok)) break;
                    if (clock64() - t0 > (s.abort_flag ? min(p.wait_cycles, kWaitCyclesAfterAbort) : p.wait_cycles)) { s.abort_flag = 1; break; }
                    __nanosleep(64);
                }
#pragma unroll
                for (int sl = 0; sl <= FK_MAX_TOP_K; ++sl) {
                    if (sl < nslots) {
#pragma unroll
                        for (int h2 = 0; h2 < 2; ++h2) {
                            const unsigned pay = (unsigned)w[2 * sl + h2];
                            const size_t el = (size_t)sl * I + warp * 64 + lane + 32 * h2;
                            reinterpret_cast<unsigned short*>(s.act_hi)[el] = (unsigned short)(pay >> 16);
                            reinterpret_cast<unsigned short*>(s.act_lo)[el] = (unsigned short)(pay & 0xffffu);
                        }
                    }
                }
                gate_v = want_gate ? __uint_as_float((unsigned)__shfl_sync(kFull, (unsigned)gw, 0)) : 1.f;
                __syncwarp();                              // the warp reads back only its own K-slice
            }
            if (tid == 0) D1_TRACE(12);
            // [16 x 64] down boxes of up to two slots against those slots' activations (head and remainder): K-slice
            // sums.  All loads of both boxes are written out first, then four independent MMA chains.
            auto down_boxes = [&](int sl0, uint32_t addr0, int sl1, uint32_t addr1) -> float {
                const bool two = sl1 >= 0;
                uint32_t bh[2][4][2], bl[2][4][2], a[2][4][4];
#pragma unroll
                for (int b = 0; b < 2; ++b) {
                    const size_t off = ((size_t)(b == 0 ? sl0 : (two ? sl1 : sl0)) * I + warp * 64 + 2 * tig) * 2;
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        bh[b][kk][0] = gid == 0 ? d1_lds32(s.act_hi + off + kk * 32) : 0u;
                        bh[b][kk][1] = gid == 0 ? d1_lds32(s.act_hi + off + kk * 32 + 16) : 0u;
                        bl[b][kk][0] = gid == 0 ? d1_lds32(s.act_lo + off + kk * 32) : 0u;
                        bl[b][kk][1] = gid == 0 ? d1_lds32(s.act_lo + off + kk * 32 + 16) : 0u;
                    }
                }
                box_load(a[0], addr0, lane);
                box_load(a[1], two ? addr1 : addr0, lane);
                // eight independent MMAs per box (a dependent MMA waits ~100 cycles for the one before it)
                float c[2][8][4];
#pragma unroll
                for (int b = 0; b < 2; ++b) {
#pragma unroll
                    for (int q = 0; q < 8; ++q) c[b][q][0] = c[b][q][1] = c[b][q][2] = c[b][q][3] = 0.f;
                }
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
                    for (int b = 0; b < 2; ++b) {
                        d1_mma(c[b][kk], a[b][kk], bh[b][kk][0], bh[b][kk][1]);
                        d1_mma(c[b][4 + kk], a[b][kk], bl[b][kk][0], bl[b][kk][1]);
                    }
                }
                float dep = 0.f;
#pragma unroll
                for (int b = 0; b < 2; ++b) {
                    // head sums first, then the remainders: a fixed order
                    const float v0 = ((c[b][0][0] + c[b][1][0]) + (c[b][2][0] + c[b][3][0])) + ((c[b][4][0] + c[b][5][0]) + (c[b][6][0] + c[b][7][0]));
                    const float v2 = ((c[b][0][2] + c[b][1][2]) + (c[b][2][2] + c[b][3][2])) + ((c[b][4][2] + c[b][5][2]) + (c[b][6][2] + c[b][7][2]));
                    const int sl = b == 0 ? sl0 : sl1;
                    if (tig == 0 && (b == 0 || two)) {
                        s.cpart[sl][warp][gid] = v0;
                        s.cpart[sl][warp][gid + 8] = v2;
                    }
                    dep += v0 + v2;
                }
                return dep;
            };
            if (has_shared) mbar_wait(&s.sdfull, 0, &s.abort_flag);
            bool shared_pending = has_shared;
#pragma unroll 1
            for (int cst = 0; cst < pl.nC; ++cst) {
                const int it = (pl.nB + cst) * kD1Consumers + warp;
                const int slot = it % kD1Stages;
                mbar_wait(&s.full[slot], (it / kD1Stages) & 1u, &s.abort_flag);
                const uint32_t base = smem_u32(s.stage[slot]);
                const int nu = min(4, p.top_k - cst * 4);
                float dep = 0.f;
#pragma unroll 1
                for (int u = 0; u < nu; u += 2)
                    dep += down_boxes(cst * 4 + u, base + u * 2048, u + 1 < nu ? cst * 4 + u + 1 : -1, base + (u + 1) * 2048);
                if (lane == 0) d1_release(&s.empty[slot], dep);
            }
            if (shared_pending) down_boxes(shared_slot, smem_u32(s.sdown[warp]), -1, 0u);
            named_bar_sync(1, cthreads);
            if (tid == 0) D1_TRACE(13);
            if (tid < kD1Tile * kD1Consumers) {
                // thread (row, w) weights K-slice w of every slot, then the eight slices of a row meet by shuffles:
                // a fixed order, so the result does not depend on scheduling
                const int row = tid >> 3, w = tid & 7;
                mbar_wait(&s.ids_ready, 0, &s.abort_flag);
                float acc = 0.f;
                for (int sl = 0; sl < p.top_k; ++sl) acc = fmaf(s.wnorm[sl], s.cpart[sl][w][row], acc);
                if (has_shared) acc = fmaf(gate_v, s.cpart[shared_slot][w][row], acc);      // gate_v is 1 without a gate
                acc += __shfl_xor_sync(kFull, acc, 1);
                acc += __shfl_xor_sync(kFull, acc, 2);
                acc += __shfl_xor_sync(kFull, acc, 4);
                if (w == 0) {
                    const int h = pl.tile * kD1Tile + row;
                    p.out[h] = acc;
                    if (p.layer_hidden && !p.resid_in) p.layer_hidden[h] = resid_v + acc;
                }
            }
            if (tid == 0) D1_TRACE(15);
        }
    }

    // Nothing to re-arm on the way out: the exchange words are told apart by the launch tag, which only grows.
    __syncthreads();
    if (tid == 0) {
        D1_TRACE(7);
        if (p.trace) p.trace[(size_t)blk * 32 + 9] = (unsigned long long)clock64();
        if (s.abort_flag && p.error_word) atomicExch(p.error_word, 2);
        // Block 0 owns an output tile, so it has seen every block's activations, and a block publishes those after it
        // has read the launch tag: all blocks have read it by now, and block 0 advances it for the next launch.
        if (blk == 0) p.bar[3] = s.tag;
    }
}

static size_t decode1_smem_bytes() { return sizeof(D1Smem) + 1024; }

// one block per SM must fit (checked once per device)
static bool decode1_resident() {
    static int cached[64] = {0};          // 0 unknown, 1 yes, -1 no
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    if (cached[dev] == 0) {
        const int smem = (int)decode1_smem_bytes();
        int n = 0;
        bool ok = cudaFuncSetAttribute(decode1_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) == cudaSuccess &&
                  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, decode1_kernel, kD1Threads, smem) == cudaSuccess && n >= 1;
        if (!ok) (void)cudaGetLastError();
        cached[dev] = ok ? 1 : -1;
    }
    return cached[dev] == 1;
}

bool decode1_supported(const DecodeParams& p, int weight_dtype) {
    if (weight_dtype != FK_BF16 || p.hidden_dtype != FK_BF16) return false;
    if (p.H != kD1H || p.I != kD1I) return false;
    if (p.top_k < 1 || p.top_k > FK_MAX_TOP_K || p.E < p.top_k || p.E > FK_MAX_EXPERTS) return false;
    const int G = sm_count();
    const int tiles = kD1H / kD1Tile;
    if (G < tiles) return false;                                              // every output tile needs a block
    if ((p.E + G - 1) / G + (p.shared_gate ? 1 : 0) > kD1MaxRouterRows) return false;
    const int total = (p.shared_gate_up ? kD1I / kD1Tile : 0) + p.top_k * (kD1I / kD1Tile);
    if ((total + G - 1) / G > kD1MaxAtoms) return false;
    uintptr_t bits = reinterpret_cast<uintptr_t>(p.hidden) | reinterpret_cast<uintptr_t>(p.norm_weight) |
                     reinterpret_cast<uintptr_t>(p.router_weight) | reinterpret_cast<uintptr_t>(p.gate_up) |
                     reinterpret_cast<uintptr_t>(p.down) | reinterpret_cast<uintptr_t>(p.shared_gate_up) |
                     reinterpret_cast<uintptr_t>(p.shared_down) | reinterpret_cast<uintptr_t>(p.shared_gate) |
                     reinterpret_cast<uintptr_t>(p.tagged) | reinterpret_cast<uintptr_t>(p.actw);
    bits |= reinterpret_cast<uintptr_t>(p.resid_in) | reinterpret_cast<uintptr_t>(p.update_in) | reinterpret_cast<uintptr_t>(p.resid_out);
    if (bits & 15) return false;
    return decode1_resident();
}

int launch_decode1(const DecodeParams& p, cudaStream_t stream) {
    static const bool cooperative = [] { const char* e = getenv("FKMOE_D1_COOPERATIVE"); return e && e[0] == '1'; }();
    const int smem = (int)decode1_smem_bytes();
    FK_CUDA_OK(cudaFuncSetAttribute(decode1_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "decode1 attr");
    // gate_up: [2 halves x 16 rows x 64 columns] boxes; down: [16 rows x 64 columns] boxes; 128-byte swizzle, cached per weight pointer
    CUtensorMap gu{}, sgu{}, dn{}, sdn{};
    const bool maps = gate_up_pair_map(p.gate_up, (uint64_t)p.E, p.I, p.H, kD1Tile, &gu) &&
                      weight_tensor_map(p.down, (uint64_t)p.E * p.H, p.I, kD1Tile, &dn) &&
                      gate_up_pair_map(p.shared_gate_up ? p.shared_gate_up : p.gate_up, 1, p.I, p.H, kD1Tile, &sgu) &&
                      weight_tensor_map(p.shared_down ? p.shared_down : p.down, (uint64_t)p.H, p.I, kD1Tile, &sdn);
    if (!maps) return FK_ERR_UNSUPPORTED;
    DecodeParams q = p;
    if (q.wait_cycles <= 0) q.wait_cycles = wait_limit_cycles();
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(sm_count());
    cfg.blockDim = dim3(kD1Threads);
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
    FK_CUDA_OK(cudaLaunchKernelEx(&cfg, decode1_kernel, gu, sgu, dn, sdn, q), "decode1 launch");
    note_launch();
    return FK_OK;
}

}  // namespace fk
