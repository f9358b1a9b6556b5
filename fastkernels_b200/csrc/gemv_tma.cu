// bf16 weight-streaming grouped GEMV fed by bulk (TMA) copies through shared-memory rings.
//
// Work unit = (pass, tile): a pass is up to 8 packed rows (tokens) of one expert (4 with the CUDA-core consumers;
// the pass list is written by the permute kernel), a tile is 16 gate/up pairs (gate_up) or 128 output rows (down).
// Units are dealt round-robin to one persistent block per SM, so a hot expert spreads over many
// blocks; its weights cross HBM once and the other passes find them in L2.
//
// Block = 16 consumer warps (two groups of 8 that take alternate weight stages) + a weight
// producer warp + an activation producer warp.  The weight producer issues 32 KB bulk copies of
// weight rows into a 4-stage ring; the activation producer looks up the pass, writes a small
// header (first row, row count) and bulk-copies the pass's activation rows into a 2-slot ring.
// Consumers never touch global memory except to store results: they wait on mbarriers, read
// 16-byte shared-memory vectors (lane = 8 consecutive columns of a 256-column slice), keep the
// activations in registers, fold partial sums with a transposing shuffle reduction and meet the
// other slices of the row in shared memory behind a named barrier of their group.
// A stage is released only after the values read from it have been used (the arrive carries a data
// dependence on the sums), so a refill cannot overtake a pending shared-memory read.
//
// GU = true : gate_up rows + SwiGLU -> act[row, i]     (a stage holds 4*RG gate rows + 4*RG up rows)
// GU = false: down rows             -> y[row, h]       (a stage holds 8*RG rows)
// with K = KCH*256 columns per row, RG = 8/KCH row groups per stage, 32 KB per stage either way.
//
// Reference math: src/fastkernels/reference/qwen36_real.py:343-347.

#include <cuda.h>

#include "common.cuh"
#include "kernels.cuh"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace fk {

constexpr int kStageBytes = 32768;          // weight bytes per stage
constexpr int kRowPad = 16;                 // gate_up rows sit 16 bytes further apart in shared memory than in HBM:
                                            // rows then start in different banks (tensor-core fragment loads)
constexpr int kStageAlloc = kStageBytes + 64 * kRowPad;
constexpr int kStages = 4;
constexpr int kXSlotBytes = 32768 + 8 * 16;  // 4 fp32 rows or 8 bf16 rows of 2048 columns at most, rows padded apart
constexpr int kXSlots = 2;
constexpr int kGroupWarps = 8;
constexpr int kGroups = 2;
constexpr int kConsumerWarps = kGroups * kGroupWarps;
constexpr int kStreamThreads = (kConsumerWarps + 2 + kGroups) * 32;   // + two producer warps + one epilogue warp per group
constexpr int kDownTile = 128;

struct StreamSmem {
    unsigned char stage[kStages][kStageAlloc];
    unsigned char xslot[kXSlots][kXSlotBytes];
    float partial[kGroups][2][kGroupWarps][128];
    int4 header[kXSlots];                    // (expert or -1, first packed row, rows, first token)
    int4 pmeta[kGroups][2];                  // per partial buffer: (first packed row, rows valid, tile, step)
    uint64_t pfull[kGroups][2];              // partial sums of a stage are complete (8 consumer warps arrive)
    uint64_t pempty[kGroups][2];             // the epilogue warp has read them
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t xfull[kXSlots];
    uint64_t xempty[kXSlots];
    int abort_flag;
    int units;                               // passes x tiles, fetched once per block
};

template <int V> struct Lg2 { static constexpr int value = 1 + Lg2<V / 2>::value; };
template <> struct Lg2<1> { static constexpr int value = 0; };

// After the call, v[0] of lane L holds the warp-wide sum of the value with index L >> (5 - log2 V).
template <int V>
__device__ __forceinline__ void transpose_reduce(float (&v)[V], int lane) {
    constexpr int L = Lg2<V>::value;
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

__device__ __forceinline__ void unpack_bf16x8(const uint4& w, float (&f)[8]) {
    f[0] = bf16lo(w.x); f[1] = bf16hi(w.x); f[2] = bf16lo(w.y); f[3] = bf16hi(w.y);
    f[4] = bf16lo(w.z); f[5] = bf16hi(w.z); f[6] = bf16lo(w.w); f[7] = bf16hi(w.w);
}

// mbarrier arrive that cannot be scheduled before `dep` has been computed.
__device__ __forceinline__ void mbar_arrive_after(uint64_t* bar, float dep) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)), "f"(dep) : "memory");
}

// pairs (gate_up) or rows (down) per unit: at least two stages, so that both groups see every unit
__host__ __device__ constexpr int stream_tile(int kch, bool gu) {
    return gu ? ((8 / kch) * 8 > 16 ? (8 / kch) * 8 : 16) : ((8 / kch) * 16 > kDownTile ? (8 / kch) * 16 : kDownTile);
}

__host__ __device__ constexpr int elem_bytes(int dtype) { return dtype == FK_F32 ? 4 : 2; }

// 8 consecutive activation values (columns col0..col0+7 of row t) from an activation slot.
__device__ __forceinline__ void load8_slot(const unsigned char* row, int dtype, int col0, float (&o)[8]) {
    if (dtype == FK_F32) {
        uint4 a = lds128(row + (size_t)col0 * 4), b = lds128(row + (size_t)col0 * 4 + 16);
        o[0] = __uint_as_float(a.x); o[1] = __uint_as_float(a.y); o[2] = __uint_as_float(a.z); o[3] = __uint_as_float(a.w);
        o[4] = __uint_as_float(b.x); o[5] = __uint_as_float(b.y); o[6] = __uint_as_float(b.z); o[7] = __uint_as_float(b.w);
    } else if (dtype == FK_BF16) {
        uint4 v = lds128(row + (size_t)col0 * 2);
        unpack_bf16x8(v, o);
    } else {
        uint4 v = lds128(row + (size_t)col0 * 2);
        const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 f = __half22float2(h[i]);
            o[2 * i] = f.x; o[2 * i + 1] = f.y;
        }
    }
}

// The weight stages of one unit for consumer group `g`, NT activation rows in registers.
template <int NT, int KCH, bool GU>
__device__ __forceinline__ void consume_unit(const ExpertParams& p, StreamSmem& s, const unsigned char* xrows, int xdtype,
                                             int row_pos, int nvalid, int tile, uint32_t& it, int& pbuf, uint32_t& nstage,
                                             uint64_t* xempty, int g, int w8, int lane) {
    constexpr int RG = 8 / KCH;
    constexpr int K = KCH * 256;
    constexpr int TILE = stream_tile(KCH, GU);
    constexpr int PER_STAGE = GU ? 4 * RG : 8 * RG;
    constexpr int STEPS = TILE / PER_STAGE;
    constexpr int RC = NT == 4 ? 4 : 8;                 // rows per reduction chunk
    constexpr int V = RC * NT;
    constexpr int SH = 5 - Lg2<V>::value;
    const int kw = w8 % KCH, rg = w8 / KCH;
    const int col0 = kw * 256 + lane * 8;

    float x[NT][8];
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        if (t < nvalid) {
            load8_slot(xrows + (size_t)t * (K * elem_bytes(xdtype) + (GU ? kRowPad : 0)), xdtype, col0, x[t]);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) x[t][i] = 0.f;
        }
    }
    bool x_released = false;

#pragma unroll 1
    for (int step = 0; step < STEPS; ++step, ++it) {
        if ((int)(it & 1u) != g) continue;
        const int stage = it % kStages;
        const uint32_t par = (it / kStages) & 1u;
        mbar_wait(&s.full[stage], par, &s.abort_flag);
        const unsigned char* base = s.stage[stage];
        uint4 w[8];
        if (GU) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                w[q] = lds128(base + (size_t)(rg * 4 + q) * (K * 2 + kRowPad) + (size_t)col0 * 2);
                w[4 + q] = lds128(base + (size_t)(4 * RG + rg * 4 + q) * (K * 2 + kRowPad) + (size_t)col0 * 2);
            }
        } else {
#pragma unroll
            for (int r = 0; r < 8; ++r) w[r] = lds128(base + ((size_t)(rg * 8 + r) * K + col0) * 2);
        }

        // the partial buffer must have been drained by the epilogue warp (two stages of this group ago)
        mbar_wait(&s.pempty[g][pbuf], ((nstage >> 1) & 1u) ^ 1u, &s.abort_flag);
        float* part = s.partial[g][pbuf][w8];
        float dep = 0.f;
#pragma unroll
        for (int c = 0; c < 8 / RC; ++c) {
            float acc[V];
#pragma unroll
            for (int r = 0; r < RC; ++r) {
                float wf[8];
                unpack_bf16x8(w[c * RC + r], wf);
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    float a = 0.f;
#pragma unroll
                    for (int i = 0; i < 8; ++i) a = fmaf(wf[i], x[t][i], a);
                    acc[r * NT + t] = a;
                }
            }
            transpose_reduce<V>(acc, lane);
            if ((lane & ((1 << SH) - 1)) == 0) part[c * V + (lane >> SH)] = acc[0];
            dep += acc[0];
        }
        // every value read from the stage (and from the activation slot) has been consumed by now
        dep = __shfl_sync(kFull, dep, 0) + dep;
        if (lane == 0) {
            mbar_arrive_after(&s.empty[stage], dep);
            if (!x_released) mbar_arrive_after(xempty, dep);
        }
        x_released = true;

        // hand the partial sums to the group's epilogue warp; the consumers go straight to their next stage
        if (w8 == 0 && lane == 0) s.pmeta[g][pbuf] = make_int4(row_pos, nvalid, tile, step);
        __syncwarp();
        if (lane == 0) mbar_arrive(&s.pfull[g][pbuf]);
        ++nstage;
        pbuf ^= 1;
    }
}

// bf16 tensor-core variant of the gate_up consumer (activations in bf16): the 8 weight rows of the warp's
// row group are the M rows of m16n8k16 MMAs (rows 8..15 of the tile are zero), up to 8 tokens are its N
// columns, and the warp's 256-column K slice is 16 MMAs.  The MMAs replace 8 unpack + 8*tokens FMA
// instructions per 8 weights per lane, which is what kept the CUDA-core version from reaching the copy
// rate; products of bf16 values are exact in fp32 either way.  Partial sums land as [row 0..7][token 0..7].
__device__ __forceinline__ void mma_bf16_16x8x16(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t lds32(const void* smem_ptr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(smem_ptr)));
    return v;
}

template <int KCH>
__device__ __forceinline__ void consume_unit_mma(const ExpertParams& p, StreamSmem& s, const unsigned char* xrows,
                                                 int row_pos, int nvalid, int tile, uint32_t& it, int& pbuf, uint32_t& nstage,
                                                 uint64_t* xempty, int g, int w8, int lane) {
    constexpr int RG = 8 / KCH;
    constexpr int K = KCH * 256;
    constexpr int TILE = stream_tile(KCH, true);
    constexpr int PER_STAGE = 4 * RG;
    constexpr int STEPS = TILE / PER_STAGE;
    constexpr int WSTRIDE = K * 2 + kRowPad;
    const int kw = w8 % KCH, rg = w8 / KCH;
    const int gid = lane >> 2, tig = lane & 3;          // fragment coordinates: row / token = gid, k pair = tig
    // B fragments: token gid, this warp's K slice, 16 k-steps x 2 registers
    uint32_t bf[16][2];
    {
        const unsigned char* xr = xrows + (size_t)gid * WSTRIDE + (size_t)(kw * 256 + 2 * tig) * 2;
#pragma unroll
        for (int ks = 0; ks < 16; ++ks) {
            bf[ks][0] = gid < nvalid ? lds32(xr + ks * 32) : 0u;
            bf[ks][1] = gid < nvalid ? lds32(xr + ks * 32 + 16) : 0u;
        }
    }
    bool x_released = false;
    // weight row of this lane inside the stage: rows 0..3 of the fragment are gate rows, 4..7 the up rows
    const int srow = gid < 4 ? rg * 4 + gid : 4 * RG + rg * 4 + (gid - 4);
#pragma unroll 1
    for (int step = 0; step < STEPS; ++step, ++it) {
        if ((int)(it & 1u) != g) continue;
        const int stage = it % kStages;
        const uint32_t par = (it / kStages) & 1u;
        mbar_wait(&s.full[stage], par, &s.abort_flag);
        const unsigned char* wr = s.stage[stage] + (size_t)srow * WSTRIDE + (size_t)(kw * 256 + 2 * tig) * 2;
        float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < 16; ks += 2) {
            mma_bf16_16x8x16(c0, lds32(wr + ks * 32), lds32(wr + ks * 32 + 16), bf[ks][0], bf[ks][1]);
            mma_bf16_16x8x16(c1, lds32(wr + (ks + 1) * 32), lds32(wr + (ks + 1) * 32 + 16), bf[ks + 1][0], bf[ks + 1][1]);
        }
        const float v0 = c0[0] + c1[0], v1 = c0[1] + c1[1];      // row gid, tokens 2*tig and 2*tig+1
        const float dep = v0 + v1;
        if (lane == 0) {
            mbar_arrive_after(&s.empty[stage], dep);
            if (!x_released) mbar_arrive_after(xempty, dep);
        }
        x_released = true;
        mbar_wait(&s.pempty[g][pbuf], ((nstage >> 1) & 1u) ^ 1u, &s.abort_flag);
        float* part = s.partial[g][pbuf][w8];
        *reinterpret_cast<float2*>(part + gid * 8 + 2 * tig) = make_float2(v0, v1);
        if (w8 == 0 && lane == 0) s.pmeta[g][pbuf] = make_int4(row_pos, nvalid | (1 << 16), tile, step);
        __syncwarp();
        if (lane == 0) mbar_arrive(&s.pfull[g][pbuf]);
        ++nstage;
        pbuf ^= 1;
    }
}

// Tensor-core variant of the down consumer (bf16 models).  The activations are the fp32 SwiGLU outputs;
// each is split into a bf16 head and a bf16 remainder (together 16 mantissa bits, relative error 2^-17),
// so every weight fragment feeds two MMAs.  A warp owns 16 output rows (a full M tile, fetched with one
// ldmatrix.x4 per k-step from the padded rows) and a 128-column K slice; the up to 8 tokens of a pass are the N columns.  Partial sums land as [row 0..15][token 0..7].
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_ptr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(smem_ptr)));
}
__device__ __forceinline__ void mma_bf16_full(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void split_bf16x2(float x, float y, uint32_t& head, uint32_t& rest) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
    const float2 hf = __bfloat1622float2(h);
    const __nv_bfloat162 l = __floats2bfloat162_rn(x - hf.x, y - hf.y);
    head = *reinterpret_cast<const uint32_t*>(&h);
    rest = *reinterpret_cast<const uint32_t*>(&l);
}

template <int KCH>
__device__ __forceinline__ void consume_unit_mma_down(const ExpertParams& p, StreamSmem& s, const unsigned char* xrows,
                                                      int row_pos, int nvalid, int tile, uint32_t& it, int& pbuf, uint32_t& nstage,
                                                      uint64_t* xempty, int g, int w8, int lane) {
    static_assert(KCH <= 4, "a stage must hold at least 16 rows");
    constexpr int K = KCH * 256;
    constexpr int TILE = stream_tile(KCH, false);
    constexpr int PER_STAGE = 64 / KCH;
    constexpr int STEPS = TILE / PER_STAGE;
    constexpr int KS = 2 * KCH;                          // 128-column K slices per 16-row tile
    const int rt = w8 / KS, ks = w8 % KS;
    const int gid = lane >> 2, tig = lane & 3;
    // B fragments: token gid, 8 k-steps, head and remainder
    uint32_t bh[8][2], bl[8][2];
    {
        const unsigned char* xr = xrows + (size_t)gid * (K * 4) + (size_t)(ks * 128 + 2 * tig) * 4;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            float2 v0 = make_float2(0.f, 0.f), v1 = make_float2(0.f, 0.f);
            if (gid < nvalid) {
                v0 = *reinterpret_cast<const float2*>(xr + q * 64);
                v1 = *reinterpret_cast<const float2*>(xr + q * 64 + 32);
            }
            split_bf16x2(v0.x, v0.y, bh[q][0], bl[q][0]);
            split_bf16x2(v1.x, v1.y, bh[q][1], bl[q][1]);
        }
    }
    bool x_released = false;
    // ldmatrix row address of this lane: matrices 0..3 = (rows 0-7, k 0-7), (rows 8-15, k 0-7), (rows 0-7, k 8-15), (rows 8-15, k 8-15).
    // A stage is K/64 slabs of [PER_STAGE rows x 128 bytes]; inside a slab the 16-byte chunk c of row r sits at chunk c ^ (r & 7).
    const int lrow = rt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
    const int lofs = (ks * 2) * (PER_STAGE * 128) + lrow * 128;
    const int lx = (lane >> 4) ^ (lane & 7);
#pragma unroll 1
    for (int step = 0; step < STEPS; ++step, ++it) {
        if ((int)(it & 1u) != g) continue;
        const int stage = it % kStages;
        const uint32_t par = (it / kStages) & 1u;
        mbar_wait(&s.full[stage], par, &s.abort_flag);
        const unsigned char* wr = s.stage[stage] + lofs;
        float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            uint32_t a[4];
            ldmatrix_x4(a, wr + (q >> 2) * (PER_STAGE * 128) + ((((q & 3) * 2) ^ lx) << 4));
            mma_bf16_full(c0, a, bh[q][0], bh[q][1]);
            mma_bf16_full(c1, a, bl[q][0], bl[q][1]);
        }
        const float2 lo = make_float2(c0[0] + c1[0], c0[1] + c1[1]);     // row gid,     tokens 2*tig, 2*tig+1
        const float2 hi = make_float2(c0[2] + c1[2], c0[3] + c1[3]);     // row gid + 8, same tokens
        const float dep = lo.x + hi.x;
        if (lane == 0) {
            mbar_arrive_after(&s.empty[stage], dep);
            if (!x_released) mbar_arrive_after(xempty, dep);
        }
        x_released = true;
        mbar_wait(&s.pempty[g][pbuf], ((nstage >> 1) & 1u) ^ 1u, &s.abort_flag);
        float* part = s.partial[g][pbuf][w8];
        *reinterpret_cast<float2*>(part + gid * 8 + 2 * tig) = lo;
        *reinterpret_cast<float2*>(part + (gid + 8) * 8 + 2 * tig) = hi;
        if (w8 == 0 && lane == 0) s.pmeta[g][pbuf] = make_int4(row_pos, nvalid | (2 << 16), tile, step);
        __syncwarp();
        if (lane == 0) mbar_arrive(&s.pfull[g][pbuf]);
        ++nstage;
        pbuf ^= 1;
    }
}

// Epilogue warp of group g: sums the K-slices of every output of a stage, applies SwiGLU (gate_up) and
// stores.  It runs beside the consumers, so the final sum and the global stores are off their path.
template <int KCH, bool GU>
__device__ __forceinline__ void epilogue_warp(const ExpertParams& p, StreamSmem& s, int g, int lane, uint32_t stages, int nt_unused) {
    constexpr int RG = 8 / KCH;
    constexpr int TILE = stream_tile(KCH, GU);
    constexpr int PER_STAGE = GU ? 4 * RG : 8 * RG;
    (void)nt_unused;
    for (uint32_t n = 0; n < stages; ++n) {
        const int pb = n & 1u;
        mbar_wait(&s.pfull[g][pb], (n >> 1) & 1u, &s.abort_flag);
        int4 m = s.pmeta[g][pb];                             // first packed row, rows valid, tile, step
        const int layout = m.y >> 16;                        // 1: tensor-core gate_up, partial[row 0..7][token 0..7]
        const bool mma_layout = layout == 1;                 // 2: tensor-core down,    partial[row 0..15][token 0..7]
        m.y &= 0xffff;
        if (!GU && layout == 2) {
            constexpr int KS = 2 * KCH;
            for (int idx = lane; idx < PER_STAGE * 8; idx += 32) {
                const int t = idx & 7, o = idx >> 3;
                const int rt = o >> 4, r16 = o & 15;
                float sum = 0.f;
#pragma unroll
                for (int k2 = 0; k2 < (KS <= 8 ? KS : 8); ++k2) sum += s.partial[g][pb][(rt * KS + k2) & 7][r16 * 8 + t];
                if (t < m.y) p.y[(size_t)(m.x + t) * p.H + m.z * TILE + m.w * PER_STAGE + o] = sum;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&s.pempty[g][pb]);
            continue;
        }
        const int NT = mma_layout ? 8 : (m.y == 1 ? 1 : (m.y == 2 ? 2 : 4));
        for (int idx = lane; idx < PER_STAGE * NT; idx += 32) {
            const int t = idx % NT;
            const int o = idx / NT;                          // output index inside the stage
            if (GU) {
                const int rg2 = o / 4, q = o - rg2 * 4;
                float gsum = 0.f, usum = 0.f;
#pragma unroll
                for (int k2 = 0; k2 < KCH; ++k2) {
                    gsum += s.partial[g][pb][rg2 * KCH + k2][q * NT + t];
                    usum += s.partial[g][pb][rg2 * KCH + k2][(4 + q) * NT + t];
                }
                if (t < m.y) p.act[(size_t)(m.x + t) * p.I + m.z * TILE + m.w * PER_STAGE + o] = silu_mul(gsum, usum);
            } else {
                const int rg2 = o / 8, r = o - rg2 * 8;
                float sum = 0.f;
#pragma unroll
                for (int k2 = 0; k2 < KCH; ++k2) sum += s.partial[g][pb][rg2 * KCH + k2][r * NT + t];
                if (t < m.y) p.y[(size_t)(m.x + t) * p.H + m.z * TILE + m.w * PER_STAGE + o] = sum;
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&s.pempty[g][pb]);
    }
}

// TM (down only): the weight stages are filled by tiled TMA copies through tensor maps (`wmap` for the
// routed experts' [E*H, I] matrix, `smap` for the shared expert's [H, I]) in the 128-byte swizzled layout
// that the tensor-core consumer's ldmatrix reads without bank conflicts.
template <int KCH, bool GU, bool TM>
__global__ void __launch_bounds__(kStreamThreads, 1) stream_gemv_kernel(const __grid_constant__ CUtensorMap wmap,
                                                                        const __grid_constant__ CUtensorMap smap, ExpertParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    // the swizzle pattern is a function of the shared-memory address: stages start on 1 KB boundaries
    StreamSmem& s = *reinterpret_cast<StreamSmem*>(smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u));
    constexpr int RG = 8 / KCH;
    constexpr int K = KCH * 256;
    constexpr int TILE = stream_tile(KCH, GU);
    constexpr int PER_STAGE = GU ? 4 * RG : 8 * RG;
    constexpr int STEPS = TILE / PER_STAGE;
    static_assert(STEPS % 2 == 0, "both consumer groups must see every unit");
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0) {
        for (int i = 0; i < kStages; ++i) {
            mbar_init(&s.full[i], 1);
            mbar_init(&s.empty[i], kGroupWarps);
        }
        for (int i = 0; i < kXSlots; ++i) {
            mbar_init(&s.xfull[i], 1);
            mbar_init(&s.xempty[i], kConsumerWarps);
        }
        for (int i = 0; i < kGroups * 2; ++i) {
            mbar_init(&s.pfull[i / 2][i % 2], kGroupWarps);
            mbar_init(&s.pempty[i / 2][i % 2], 1);
        }
        s.abort_flag = 0;
        mbar_init_fence();
    }
    if (GU) pdl_wait();       // pass list and packed order come from the permutation kernel
    // one thread fetches the pass count for the block (a load by every warp of every block queues thousands of
    // requests on one L2 line)
    if (tid == 0) s.units = __ldcg(p.meta + 1) * ((GU ? p.I : p.H) / TILE);
    __syncthreads();
    if (GU) {
        pdl_trigger();        // only now: the down kernel reads the pass list without waiting (below)
    } else {
        // The down kernel is released while the gate_up kernel still runs (which has itself waited for the
        // permutation).  Its blocks take over SMs as gate_up blocks leave, and their weight producers fill the
        // rings at once: weights and pass list are final.  Only the activation producer has to wait for gate_up.
        pdl_trigger();
    }

    const int tiles = (GU ? p.I : p.H) / TILE;
    const int units = s.units;
    const int xdtype = GU ? p.hidden_dtype : FK_F32;
    const int xrow_bytes = K * elem_bytes(xdtype);

    if (warp == kConsumerWarps) {
        // ---------------------------------------------------------------- weight producer
        {
            const uint64_t wpolicy = l2_evict_first_policy();
            uint32_t it = 0;
            int unit = blockIdx.x;
            // __ldcg: in the down kernel this warp does not wait for the kernel before it (see launch_experts_stream), so
            // the pass list must not be served from a line cached before that kernel's predecessor wrote it
            int4 next = unit < units ? __ldcg(p.passes + unit / tiles) : make_int4(0, 0, 0, 0);
            for (; unit < units; unit += gridDim.x) {
                const int4 pass = next;
                const int tile = unit % tiles;
                const int nu = unit + gridDim.x;
                if (nu < units) next = __ldcg(p.passes + nu / tiles);
                const __nv_bfloat16* W;
                if (pass.x < 0) {
                    W = reinterpret_cast<const __nv_bfloat16*>(GU ? p.shared_gate_up : p.shared_down);
                } else {
                    const size_t per_expert = GU ? (size_t)2 * p.I * p.H : (size_t)p.H * p.I;
                    W = reinterpret_cast<const __nv_bfloat16*>(GU ? p.gate_up : p.down) + (size_t)pass.x * per_expert;
                }
                for (int step = 0; step < STEPS; ++step, ++it) {
                    const int stage = it % kStages;
                    const uint32_t par = (it / kStages) & 1u;
                    unsigned char* sbuf = s.stage[stage];
                    if (lane == 0) {
                        mbar_wait(&s.empty[stage], par ^ 1u, &s.abort_flag);
                        mbar_expect_tx(&s.full[stage], kStageBytes);
                    }
                    __syncwarp();
                    const size_t first = (size_t)tile * TILE + (size_t)step * PER_STAGE;
                    if (GU) {
                        // one copy per weight row (gate rows first, then the up rows of the same pairs), rows padded apart
                        for (int r = lane; r < 2 * PER_STAGE; r += 32) {
                            const size_t grow = r < PER_STAGE ? first + r : (size_t)p.I + first + (r - PER_STAGE);
                            bulk_load_hint(sbuf + (size_t)r * (K * 2 + kRowPad), W + grow * K, K * 2, &s.full[stage], wpolicy);
                        }
                    } else if (TM) {
                        // one box of [PER_STAGE rows x 64 columns] per 128-byte column slab, 128-byte swizzle
                        const CUtensorMap* map = pass.x < 0 ? &smap : &wmap;
                        const int y = (pass.x < 0 ? 0 : pass.x * p.H) + (int)first;
                        for (int sl = lane; sl < K / 64; sl += 32)
                            tma_load_2d_hint(sbuf + (size_t)sl * (PER_STAGE * 128), map, sl * 64, y, &s.full[stage], wpolicy);
                    } else if (lane == 0) {
                        bulk_load(sbuf, W + first * K, kStageBytes, &s.full[stage]);
                    }
                }
            }
        }
    } else if (warp == kConsumerWarps + 1) {
        // ---------------------------------------------------------------- activation producer
        uint32_t ui = 0;
        int unit = blockIdx.x;
        int4 next = unit < units ? __ldcg(p.passes + unit / tiles) : make_int4(0, 0, 0, 0);
        if (!GU) pdl_wait();  // the activations are the gate_up kernel's output
        for (; unit < units; unit += gridDim.x, ++ui) {
            const int4 pass = next;
            const int nu = unit + gridDim.x;
            if (nu < units) next = __ldcg(p.passes + nu / tiles);
            const int slot = ui % kXSlots;
            const uint32_t par = (ui / kXSlots) & 1u;
            const void* src = nullptr;
            if (GU) {
                if (lane < pass.z) {
                    const int token = pass.x < 0 ? (pass.w + lane) : (p.order[pass.y + lane] / p.top_k);
                    src = reinterpret_cast<const unsigned char*>(p.hidden) + (size_t)token * xrow_bytes;
                }
            } else if (lane == 0) {
                src = p.act + (size_t)pass.y * K;      // the rows of a pass are consecutive in act
            }
            if (lane == 0) {
                mbar_wait(&s.xempty[slot], par ^ 1u, &s.abort_flag);
                s.header[slot] = pass;
                mbar_expect_tx(&s.xfull[slot], (uint32_t)(pass.z * xrow_bytes));
            }
            __syncwarp();
            if (GU) {
                if (lane < pass.z) bulk_load(s.xslot[slot] + (size_t)lane * (xrow_bytes + kRowPad), src, xrow_bytes, &s.xfull[slot]);
            } else if (lane == 0) {
                bulk_load(s.xslot[slot], src, (uint32_t)(pass.z * xrow_bytes), &s.xfull[slot]);
            }
        }
    } else if (warp >= kConsumerWarps + 2) {
        // ---------------------------------------------------------------- epilogue warps (one per group)
        const int g = warp - (kConsumerWarps + 2);
        const int my_units = units > (int)blockIdx.x ? (units - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
        epilogue_warp<KCH, GU>(p, s, g, lane, (uint32_t)my_units * (STEPS / 2), 0);
    } else {
        // ---------------------------------------------------------------- consumers
        const int g = warp / kGroupWarps, w8 = warp % kGroupWarps;
        int pbuf = 0;
        uint32_t it = 0, ui = 0, nstage = 0;
        for (int unit = blockIdx.x; unit < units; unit += gridDim.x, ++ui) {
            const int tile = unit % tiles;
            const int slot = ui % kXSlots;
            const uint32_t par = (ui / kXSlots) & 1u;
            mbar_wait(&s.xfull[slot], par, &s.abort_flag);
            const int4 pass = s.header[slot];
            const unsigned char* xrows = s.xslot[slot];
            if (GU && xdtype == FK_BF16)
                consume_unit_mma<KCH>(p, s, xrows, pass.y, pass.z, tile, it, pbuf, nstage, &s.xempty[slot], g, w8, lane);
            else if (TM)
                consume_unit_mma_down<(KCH <= 4 ? KCH : 4)>(p, s, xrows, pass.y, pass.z, tile, it, pbuf, nstage, &s.xempty[slot], g, w8, lane);
            else if (pass.z == 1) consume_unit<1, KCH, GU>(p, s, xrows, xdtype, pass.y, 1, tile, it, pbuf, nstage, &s.xempty[slot], g, w8, lane);
            else if (pass.z == 2) consume_unit<2, KCH, GU>(p, s, xrows, xdtype, pass.y, 2, tile, it, pbuf, nstage, &s.xempty[slot], g, w8, lane);
            else consume_unit<4, KCH, GU>(p, s, xrows, xdtype, pass.y, pass.z, tile, it, pbuf, nstage, &s.xempty[slot], g, w8, lane);
        }
        if (s.abort_flag && lane == 0 && p.error_word) atomicExch(p.error_word, 1);
    }
}

// Rows per pass the streaming kernels want from the permutation: the tensor-core consumers (bf16 models)
// take 8 tokens as the N columns of an MMA, the CUDA-core consumers keep 4 tokens in registers.
int stream_pass_rows(const ExpertParams& p) {
    CUtensorMap probe;
    const void* any = p.down ? p.down : p.shared_down;
    const bool mma = p.hidden_dtype == FK_BF16 && p.I <= 1024 && any != nullptr &&
                     weight_tensor_map(any, p.down ? (uint64_t)p.E * p.H : (uint64_t)p.H, p.I, 64 / (p.I / 256), &probe);
    return mma ? 8 : 4;
}

static bool kch_supported(int k) { return k == 256 || k == 512 || k == 1024 || k == 2048; }

bool stream_path_supported(const ExpertParams& p, int weight_dtype) {
    if (weight_dtype != FK_BF16) return false;
    if (!kch_supported(p.H) || !kch_supported(p.I)) return false;
    if (p.I % stream_tile(p.H / 256, true) != 0 || p.H % stream_tile(p.I / 256, false) != 0) return false;
    uintptr_t bits = reinterpret_cast<uintptr_t>(p.hidden) | reinterpret_cast<uintptr_t>(p.gate_up) |
                     reinterpret_cast<uintptr_t>(p.down) | reinterpret_cast<uintptr_t>(p.shared_gate_up) |
                     reinterpret_cast<uintptr_t>(p.shared_down);
    return (bits & 15) == 0;
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

template <int KCH, bool GU, bool TM>
static int launch_stream_t(const ExpertParams& p, cudaStream_t stream, const CUtensorMap& wmap, const CUtensorMap& smap) {
    auto kern = stream_gemv_kernel<KCH, GU, TM>;
    const int smem = (int)sizeof(StreamSmem) + 1024;
    FK_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "stream gemv attr");
    FK_CUDA_OK(launch_pdl(kern, dim3(sm_count()), dim3(kStreamThreads), (size_t)smem, stream, wmap, smap, p), "stream gemv launch");
    FK_LAUNCH_OK(GU ? "gate_up stream launch" : "down stream launch");
    return FK_OK;
}

template <int KCH>
static int launch_down(const ExpertParams& p, cudaStream_t stream) {
    CUtensorMap wmap{}, smap{};
    if (KCH <= 4 && p.hidden_dtype == FK_BF16) {
        // bf16 model: tensor-core consumer over swizzled stages, if the driver can encode the maps
        const void* any = p.down ? p.down : p.shared_down;
        const bool ok = weight_tensor_map(any, p.down ? (uint64_t)p.E * p.H : (uint64_t)p.H, p.I, 64 / KCH, &wmap) &&
                        weight_tensor_map(p.shared_down ? p.shared_down : any, (uint64_t)p.H, p.I, 64 / KCH, &smap);
        if (ok) return launch_stream_t<KCH, false, (KCH <= 4)>(p, stream, wmap, smap);
    }
    return launch_stream_t<KCH, false, false>(p, stream, wmap, smap);
}

// Launch order is part of the kernels' contract.  The down kernel is released by the gate_up kernel's trigger and
// reads the pass list (and overwrites y) WITHOUT waiting for gate_up to finish; only its activation producer waits.
// That is sound because (1) the gate_up kernel triggers only after its own griddepcontrol.wait, i.e. after the
// permutation that wrote the pass list has completed, and (2) every kernel earlier in the chain waits before it
// completes, so the previous call's combine (the reader of y) is done by then.  The down launch must therefore
// directly follow a gate_up launch of this file; a kernel that triggers before it waits must not be put between.
int launch_experts_stream(const ExpertParams& p, cudaStream_t stream) {
    if (p.T <= 0) return FK_OK;
    int st;
    const CUtensorMap none{};
    switch (p.H / 256) {
        case 1: st = launch_stream_t<1, true, false>(p, stream, none, none); break;
        case 2: st = launch_stream_t<2, true, false>(p, stream, none, none); break;
        case 4: st = launch_stream_t<4, true, false>(p, stream, none, none); break;
        case 8: st = launch_stream_t<8, true, false>(p, stream, none, none); break;
        default: return FK_ERR_UNSUPPORTED;
    }
    if (st != FK_OK) return st;
    stage_mark();   // end of gate_up
    switch (p.I / 256) {
        case 1: st = launch_down<1>(p, stream); break;
        case 2: st = launch_down<2>(p, stream); break;
        case 4: st = launch_down<4>(p, stream); break;
        case 8: st = launch_down<8>(p, stream); break;
        default: return FK_ERR_UNSUPPORTED;
    }
    if (st != FK_OK) return st;
    stage_mark();   // end of down
    return FK_OK;
}

}  // namespace fk
