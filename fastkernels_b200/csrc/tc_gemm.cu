// Grouped expert GEMM on the Blackwell tensor cores (tcgen05 + tensor memory), for expert groups
// that are too tall for the CUDA-core GEMV (>= 64 tokens in the batch).
//
// Swap-AB: the weight rows are the MMA's M dimension (128 rows per tile, K-major in shared memory,
// 128-byte swizzle, loaded by tiled TMA), the tokens of one pass are its N dimension (up to 64,
// rounded up to 16), K runs over the reduction dimension in chunks of 64.  A gate_up tile is 64 gate
// rows stacked on the 64 up rows of the same pairs (two 64-row TMA boxes into one operand tile), so
// one MMA per K step produces both halves: accumulator lanes 0..63 hold gate[p, t], lanes 64..127
// hold up[p, t].  The two up warps of the epilogue pass their values through shared memory to the
// two gate warps, which apply SwiGLU and store bf16 into the packed activation buffer that the down
// GEMM reads back through TMA.  (Tiles of 64 pairs keep the work units at 0.5 MiB: with 1 MiB units
// the last round over the 148 SMs ran a third full at 64 tokens.)  Two accumulator buffers: the MMAs
// of the next unit run while the epilogue drains the previous one.
//
// Block = 6 warps: warp 0 issues TMA (one lane), warp 1 owns tensor memory and issues the MMAs (one
// lane), warps 2..5 are the epilogue (one TMEM lane quarter each).  One persistent block per SM,
// units (pass x 128-row tile) dealt round-robin.  Every wait is bounded.
//
// Reference math: src/fastkernels/reference/qwen36_real.py:343-347.

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "kernels.cuh"
#include "tcgen05.cuh"

namespace fk {

// NMAX = tokens per pass (MMA N, rounded up to 16): 64 while experts see few tokens (more ring stages, the kernel is
// a weight stream), 128 when an expert sees dozens of tokens (expert parallel at 8 x 256 tokens: 64 per expert on
// average, and every pass beyond the first streams the expert's weights again).
constexpr int kTcStagesMax = 8;
constexpr int kTcThreads = 192;
constexpr int kTcTileBytes = 128 * 64 * 2;          // one 128-row x 64-column bf16 operand tile
// MT = weight tiles per unit (they share the unit's activation tile: with 2, the activations of a pass cross the SM
// boundary half as often).  Ring depth: what fits beside the barriers and the up-value buffer.
__host__ __device__ constexpr int tc_stages(bool gu, int nmax, int mt) {
    return mt == 2 ? 4 : (nmax == 64 ? (gu ? 7 : 8) : (gu ? 5 : 6));
}
__host__ __device__ constexpr int tc_b_bytes(int nmax) { return nmax * 64 * 2; }
constexpr int kTcUStride = 17;                      // row stride (floats) of the up-value exchange buffer (16 columns at a time)
constexpr int kTcUBytes = 2 * 64 * kTcUStride * (int)sizeof(float);

struct TcBarriers {
    uint64_t full[kTcStagesMax];
    uint64_t empty[kTcStagesMax];
    uint64_t tfull[2];
    uint64_t tempty[2];
    uint32_t tmem_base;
    int abort_flag;
    int units;
};

struct TcParams {
    const int4* passes;        // (expert or -1, first packed row, rows <= 64, first token)
    const int* meta;           // [1] = number of passes
    __nv_bfloat16* actb;       // GU: output [rows, I] bf16
    float* y;                  // down: output [rows, H] f32
    int* error_word;
    int H, I;
};

template <bool GU, int NMAX, int MT>
__global__ void __launch_bounds__(kTcThreads, 1)
tc_grouped_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap smap,
                  const __grid_constant__ CUtensorMap amap, TcParams p) {
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
    constexpr int kTcBBytes = tc_b_bytes(NMAX);
    constexpr int kTcTmemCols = 2 * MT * NMAX;            // two accumulator buffers of MT tiles
    static_assert(kTcTmemCols <= 512 && (kTcTmemCols & (kTcTmemCols - 1)) == 0, "tensor memory holds 512 columns");
    constexpr int kABytes = MT * kTcTileBytes;
    constexpr int kStageBytes = kABytes + kTcBBytes;
    constexpr int kNumStages = tc_stages(GU, NMAX, MT);
    TcBarriers& bar = *reinterpret_cast<TcBarriers*>(smem + kNumStages * kStageBytes);
    float* ubuf = reinterpret_cast<float*>(smem + kNumStages * kStageBytes + 1024);   // GU: [2][64][kTcUStride]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int K = GU ? p.H : p.I;
    const int chunks = K / 64;
    const int tiles = (GU ? p.I / 64 : p.H / 128) / MT;     // units per pass
    const int rows_per_expert = GU ? 2 * p.I : p.H;
    if (tid == 0) {
        for (int i = 0; i < kNumStages; ++i) { mbar_init(&bar.full[i], 1); mbar_init(&bar.empty[i], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&bar.tfull[i], 1); mbar_init(&bar.tempty[i], 4); }
        bar.abort_flag = 0;
        mbar_init_fence();
        prefetch_tensormap(&wmap);
        prefetch_tensormap(&smap);
        prefetch_tensormap(&amap);
    }
    if (warp == 1) tmem_alloc(&bar.tmem_base, kTcTmemCols);
    pdl_trigger();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = bar.tmem_base;
    pdl_wait();               // pass list and gathered activations come from the kernels before
    if (tid == 0) bar.units = p.meta[1] * tiles;      // one load per block, not one per warp
    __syncthreads();
    const int units = bar.units;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t it = 0;
            int4 next = (int)blockIdx.x < units ? p.passes[blockIdx.x / tiles] : make_int4(0, 0, 0, 0);
            for (int unit = blockIdx.x; unit < units; unit += gridDim.x) {
                const int4 pass = next;                      // looked up one unit ahead: off the copy-issue path
                if (unit + (int)gridDim.x < units) next = p.passes[(unit + gridDim.x) / tiles];
                const int mt = unit % tiles;
                const int npad = (pass.z + 15) & ~15;
                const CUtensorMap* wm = pass.x < 0 ? &smap : &wmap;
                const int wrow = (pass.x < 0 ? 0 : pass.x * rows_per_expert) + mt * MT * (GU ? 64 : 128);
                for (int c = 0; c < chunks; ++c, ++it) {
                    const int stage = it % kNumStages;
                    const uint32_t par = (it / kNumStages) & 1u;
                    mbar_wait(&bar.empty[stage], par ^ 1u, &bar.abort_flag);
                    unsigned char* st = smem + stage * kStageBytes;
                    // activations: whole 64-row boxes (rows past the pass belong to the next expert or are zero-filled
                    // past the end; the epilogue ignores them).  Boxes of 16 rows cost one TMA instruction per 2 KB.
                    const int nb64 = (npad + 63) / 64;
                    mbar_expect_tx(&bar.full[stage], kABytes + nb64 * 64 * 128);
#pragma unroll
                    for (int t = 0; t < MT; ++t) {
                        unsigned char* at = st + t * kTcTileBytes;
                        if (GU) {
                            tma_load_2d(at, wm, c * 64, wrow + t * 64, &bar.full[stage]);                            // 64 gate rows
                            tma_load_2d(at + kTcTileBytes / 2, wm, c * 64, wrow + t * 64 + p.I, &bar.full[stage]);   // 64 up rows
                        } else {
                            tma_load_2d(at, wm, c * 64, wrow + t * 128, &bar.full[stage]);
                        }
                    }
                    unsigned char* bt = st + kABytes;
                    for (int j = 0; j < nb64; ++j)
                        tma_load_2d(bt + j * 64 * 128, &amap, c * 64, pass.y + j * 64, &bar.full[stage]);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            uint32_t it = 0, ui = 0;
            for (int unit = blockIdx.x; unit < units; unit += gridDim.x, ++ui) {
                const int4 pass = p.passes[unit / tiles];
                const uint32_t npad = (uint32_t)((pass.z + 15) & ~15);
                const uint32_t idesc = umma_idesc_bf16(npad);
                const uint32_t acc = ui & 1u;
                mbar_wait(&bar.tempty[acc], ((ui >> 1) & 1u) ^ 1u, &bar.abort_flag);
                tc_fence_after_sync();
                const uint32_t d0 = tmem_base + acc * (uint32_t)(MT * NMAX);
                for (int c = 0; c < chunks; ++c, ++it) {
                    const int stage = it % kNumStages;
                    const uint32_t par = (it / kNumStages) & 1u;
                    mbar_wait(&bar.full[stage], par, &bar.abort_flag);
                    tc_fence_after_sync();
                    const unsigned char* st = smem + stage * kStageBytes;
                    const unsigned char* bt = st + kABytes;
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        const uint32_t accum = (c > 0 || kk > 0) ? 1u : 0u;
#pragma unroll
                        for (int t = 0; t < MT; ++t)
                            umma_bf16(d0 + t * NMAX, umma_smem_desc(st + t * kTcTileBytes + kk * 32), umma_smem_desc(bt + kk * 32), idesc, accum);
                    }
                    umma_commit(&bar.empty[stage]);      // the stage is free once these MMAs have read it
                }
                umma_commit(&bar.tfull[acc]);            // the accumulators are complete
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue warps
        const int q = warp & 3;                          // TMEM lane quarter this warp may read
        const int r = q * 32 + lane;                     // row of the 128-row tile
        uint32_t ui = 0, uc = 0;                         // units done; 16-column chunks handed over (selects the buffer)
        for (int unit = blockIdx.x; unit < units; unit += gridDim.x, ++ui) {
            const int4 pass = p.passes[unit / tiles];
            const int mt = unit % tiles;
            const int n = pass.z, npad = (n + 15) & ~15;
            const uint32_t acc = ui & 1u;
            mbar_wait(&bar.tfull[acc], (ui >> 1) & 1u, &bar.abort_flag);
            tc_fence_after_sync();
            const uint32_t taddr0 = tmem_base + ((uint32_t)(q * 32) << 16) + acc * (uint32_t)(MT * NMAX);
#pragma unroll 1
            for (int t = 0; t < MT; ++t) {
                const uint32_t taddr = taddr0 + t * NMAX;
                const int tile = mt * MT + t;
                if (GU) {
                    // lanes 64..127 hold the up rows: they reach the warps that hold the gate rows of the same pairs through
                    // shared memory, 16 columns at a time in two alternating buffers (one barrier per 16 columns)
                    for (int c16 = 0; c16 < npad / 16; ++c16, ++uc) {
                        float* ub = ubuf + (size_t)(uc & 1u) * 64 * kTcUStride;
                        float v[16];
                        tmem_ld16(taddr + c16 * 16, v);
                        if (q >= 2) {
#pragma unroll
                            for (int j = 0; j < 16; ++j) ub[(size_t)(r - 64) * kTcUStride + j] = v[j];
                        }
                        named_bar_sync(2, 128);
                        if (q < 2) {
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                const int tok = c16 * 16 + j;
                                if (tok < n) {
                                    const float u = ub[(size_t)r * kTcUStride + j];
                                    p.actb[(size_t)(pass.y + tok) * p.I + tile * 64 + r] = __float2bfloat16_rn(silu_mul(v[j], u));
                                }
                            }
                        }
                    }
                } else {
                    for (int c16 = 0; c16 < npad / 16; ++c16) {
                        float g[16];
                        tmem_ld16(taddr + c16 * 16, g);
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int tok = c16 * 16 + j;
                            if (tok < n) p.y[(size_t)(pass.y + tok) * p.H + tile * 128 + r] = g[j];
                        }
                    }
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar.tempty[acc]);
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTcTmemCols);
    }
    if (tid == 0 && bar.abort_flag && p.error_word) atomicExch(p.error_word, 3);
}

// packed bf16 activations: xg[pos] = hidden[token of packed row pos]; the shared expert's rows follow
__global__ void gather_rows_kernel(ExpertParams p, __nv_bfloat16* xg) {
    pdl_trigger();
    pdl_wait();
    const int routed = p.offsets[p.E];
    const int shared_rows = p.shared_gate_up ? p.shared_n : 0;
    const int chunks = p.H / 8;
    const long long total = (long long)(p.routes + shared_rows) * chunks;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int pos = (int)(i / chunks), c = (int)(i - (long long)pos * chunks);
        int token;
        if (pos >= p.routes) token = p.shared_tok0 + pos - p.routes;
        else if (pos < routed) token = p.order[pos] / p.top_k;
        else continue;
        const size_t src = (size_t)token * p.H + c * 8;
        uint4 out;
        if (p.hidden_dtype == FK_BF16) {
            out = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.hidden) + src);
        } else {
            __nv_bfloat162 h2[4];
#pragma unroll
            for (int k = 0; k < 4; ++k)
                h2[k] = __floats2bfloat162_rn(load_any(p.hidden, p.hidden_dtype, src + 2 * k), load_any(p.hidden, p.hidden_dtype, src + 2 * k + 1));
            out = *reinterpret_cast<uint4*>(h2);
        }
        *reinterpret_cast<uint4*>(xg + (size_t)pos * p.H + c * 8) = out;
    }
}

// ---------------------------------------------------------------------------------------------
// Host side: tensor maps (encoded through the driver entry point, cached) and launches
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    return fn;
}

struct MapKey {
    const void* base; uint64_t rows, cols; uint32_t box_rows;
    bool operator==(const MapKey& o) const { return base == o.base && rows == o.rows && cols == o.cols && box_rows == o.box_rows; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        return std::hash<const void*>()(k.base) ^ (k.rows * 1000003ull) ^ (k.cols * 10007ull) ^ k.box_rows;
    }
};

// 2-D bf16 tensor [rows, cols] row-major, box = [box_rows, 64 columns], 128-byte swizzle, zero fill outside
bool weight_tensor_map(const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, CUtensorMap* out) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;
    MapKey key{base, rows, cols, box_rows};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return true; }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * 2};
    cuuint32_t box[2] = {64, box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUtensorMap m;
    CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, m);
    *out = m;
    return true;
}

// 3-D view of a bf16 gate_up tensor [experts][2][half_rows][cols] (gate rows, then up rows, per expert):
// coordinates (column, row within the half, 2 * expert + half); box = [2 halves][box_rows][64 columns], 128-byte
// swizzle.  One copy brings box_rows gate rows together with their up rows: half as many copies for the same bytes.
bool gate_up_pair_map(const void* base, uint64_t experts, uint64_t half_rows, uint64_t cols, uint32_t box_rows, CUtensorMap* out) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;
    MapKey key{base, experts * half_rows, cols, box_rows | (uint32_t)(half_rows << 8)};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return true; }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[3] = {cols, half_rows, 2 * experts};
    cuuint64_t strides[2] = {cols * 2, half_rows * cols * 2};
    cuuint32_t box[3] = {64, box_rows, 2};
    cuuint32_t elem[3] = {1, 1, 1};
    CUtensorMap m;
    CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, m);
    *out = m;
    return true;
}

// 3-D view of a row-major bf16 matrix [rows][cols] as (64 columns, column group, row): box = [box_rows][2 groups][64
// columns], 128-byte swizzle.  One copy brings box_rows x 128 columns; in shared memory row r holds its two 128-byte
// groups one after the other (line 2 r + g), and the swizzle goes by that line number.
bool column_pair_map(const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, CUtensorMap* out) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;
    MapKey key{base, rows, cols, box_rows};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return true; }
    EncodeTiledFn fn = encode_fn();
    if (!fn || cols % 128 != 0) return false;
    cuuint64_t dims[3] = {64, cols / 64, rows};
    cuuint64_t strides[2] = {128, cols * 2};
    cuuint32_t box[3] = {64, 2, box_rows};
    cuuint32_t elem[3] = {1, 1, 1};
    CUtensorMap m;
    CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, m);
    *out = m;
    return true;
}

bool tc_path_supported(const ExpertParams& p, int weight_dtype) {
    if (weight_dtype != FK_BF16) return false;
    if (p.H % 128 != 0 || p.I % 64 != 0 || p.H < 128 || p.I < 64) return false;
    uintptr_t bits = reinterpret_cast<uintptr_t>(p.hidden) | reinterpret_cast<uintptr_t>(p.gate_up) |
                     reinterpret_cast<uintptr_t>(p.down) | reinterpret_cast<uintptr_t>(p.shared_gate_up) |
                     reinterpret_cast<uintptr_t>(p.shared_down);
    if (bits & 15) return false;
    return encode_fn() != nullptr;
}

// gather -> gate_up GEMM (+SwiGLU) -> down GEMM; the pass list in p.passes must hold passes of <= NMAX rows
template <int NMAX, int MT>
static int launch_experts_tc_t(const ExpertParams& p, __nv_bfloat16* xg, __nv_bfloat16* actb, cudaStream_t stream) {
    if (p.T <= 0) return FK_OK;
    const uint64_t rows = (uint64_t)p.routes + (p.shared_gate_up ? p.shared_n : 0);
    CUtensorMap w_gu, s_gu, a_x, w_dn, s_dn, a_act;
    const void* dummy_gu = p.gate_up ? p.gate_up : p.shared_gate_up;
    const void* dummy_dn = p.down ? p.down : p.shared_down;
    const uint64_t e_rows = p.gate_up ? (uint64_t)p.E : 0;
    bool ok = weight_tensor_map(dummy_gu, p.gate_up ? e_rows * 2 * p.I : 2 * p.I, p.H, 64, &w_gu) &&
              weight_tensor_map(p.shared_gate_up ? p.shared_gate_up : dummy_gu, 2 * (uint64_t)p.I, p.H, 64, &s_gu) &&
              weight_tensor_map(xg, rows, p.H, 64, &a_x) &&
              weight_tensor_map(dummy_dn, p.down ? e_rows * p.H : p.H, p.I, 128, &w_dn) &&
              weight_tensor_map(p.shared_down ? p.shared_down : dummy_dn, (uint64_t)p.H, p.I, 128, &s_dn) &&
              weight_tensor_map(actb, rows, p.I, 64, &a_act);
    if (!ok) return FK_ERR_UNSUPPORTED;

    {
        long long total = (long long)rows * (p.H / 8);
        int blocks = (int)((total + 255) / 256);
        if (blocks > sm_count() * 8) blocks = sm_count() * 8;
        FK_CUDA_OK(launch_pdl(gather_rows_kernel, dim3(blocks), dim3(256), 0, stream, p, xg), "gather rows launch");
        FK_LAUNCH_OK("gather rows launch");
    }
    stage_mark();   // end of the row gather
    TcParams tp{};
    tp.passes = p.passes; tp.meta = p.meta; tp.actb = actb; tp.y = p.y; tp.error_word = p.error_word; tp.H = p.H; tp.I = p.I;
    {
        auto kern = tc_grouped_kernel<true, NMAX, MT>;
        const int smem = tc_stages(true, NMAX, MT) * (MT * kTcTileBytes + tc_b_bytes(NMAX)) + 1024 + kTcUBytes + 1024;
        FK_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "tc gate_up attr");
        FK_CUDA_OK(launch_pdl(kern, dim3(sm_count()), dim3(kTcThreads), (size_t)smem, stream, w_gu, s_gu, a_x, tp), "tc gate_up launch");
        FK_LAUNCH_OK("tc gate_up launch");
    }
    stage_mark();   // end of gate_up
    {
        auto kern = tc_grouped_kernel<false, NMAX, MT>;
        const int smem = tc_stages(false, NMAX, MT) * (MT * kTcTileBytes + tc_b_bytes(NMAX)) + 1024 + 1024;
        FK_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "tc down attr");
        FK_CUDA_OK(launch_pdl(kern, dim3(sm_count()), dim3(kTcThreads), (size_t)smem, stream, w_dn, s_dn, a_act, tp), "tc down launch");
        FK_LAUNCH_OK("tc down launch");
    }
    stage_mark();   // end of down
    return FK_OK;
}

// pass_rows 64: one weight tile per unit (experts that see a few tokens: the kernel is a weight stream);
// pass_rows 128: 128-token passes and two weight tiles per unit (experts that see dozens of tokens: what crosses the
// SM boundary per expert drops from two passes x (weights + 8 x activations) to weights + 4 x activations).
int launch_experts_tc(const ExpertParams& p, __nv_bfloat16* xg, __nv_bfloat16* actb, int pass_rows, cudaStream_t stream) {
    const bool pairs_ok = (p.I / 64) % 2 == 0 && (p.H / 128) % 2 == 0;
    if (pass_rows > 64) return pairs_ok ? launch_experts_tc_t<128, 2>(p, xg, actb, stream) : launch_experts_tc_t<128, 1>(p, xg, actb, stream);
    return launch_experts_tc_t<64, 1>(p, xg, actb, stream);
}

}  // namespace fk
