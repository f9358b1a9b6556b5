// Expert histogram, exclusive offsets and the stable expert-major permutation of the T*k routes.
//
// One block of 8 warps (few routes) or 32 warps.  Each warp owns a contiguous segment of the flattened id array; a
// per-warp histogram in shared memory turns into per-warp base offsets, so rows land in
// flat-index order inside every expert group (order == argsort(ids.flatten(), stable)).
// Oracle: reference_expert_histogram (src/fastkernels/reference/moe.py:24-30) for the counts;
// the packing itself has no reference implementation.

#include "common.cuh"
#include "kernels.cuh"

namespace fk {

constexpr int kPermWarps = 32;

__device__ __forceinline__ int local_expert(const PermuteParams& p, int r) {
    long long id = p.ids64 ? p.ids64[r] : (long long)p.ids32[r];
    long long lid = id - p.expert_base;
    if (lid < 0 || lid >= p.E) {
        if (p.skip_foreign) return -1;
        lid = lid < 0 ? 0 : p.E - 1;      // clamp, as the reference kernels do
    }
    return (int)lid;
}

__global__ void __launch_bounds__(kPermWarps * 32) permute_kernel(PermuteParams p) {
    extern __shared__ int sm[];
    const int E = p.E, R = p.routes;
    const int NW = blockDim.x >> 5;        // warps in this launch (8 or kPermWarps)
    int* whist = sm;                       // [NW][E]
    int* offs = sm + NW * E;               // [E+1]
    __shared__ int warp_cnt[kPermWarps], warp_flag[kPermWarps];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    pdl_trigger();
    for (int i = tid; i < NW * E; i += blockDim.x) whist[i] = 0;
    pdl_wait();               // the ids come from the router
    __syncthreads();

    const int seg = (R + NW - 1) / NW;
    const int seg_lo = min(R, warp * seg), seg_hi = min(R, seg_lo + seg);
    // The local expert of every route is kept in shared memory for the placement pass (when it fits), and the ids are
    // fetched four groups at a time: with thousands of routes the kernel was two serial chains of global loads.
    short* lid_cache = p.cache_routes >= R ? reinterpret_cast<short*>(offs + E + 2) : nullptr;
    for (int base = seg_lo; base < seg_hi; base += 128) {
        int lid[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int r = base + j * 32 + lane;
            lid[j] = r < seg_hi ? local_expert(p, r) : -1;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int r = base + j * 32 + lane;
            if (lid[j] >= 0) atomicAdd(&whist[warp * E + lid[j]], 1);
            if (lid_cache && r < seg_hi) lid_cache[r] = (short)lid[j];
        }
    }
    __syncthreads();

    // per expert (E <= blockDim.x): running sum over warps -> warp base offsets; total -> count
    {
        const int e = tid;
        int c = 0;
        if (e < E) {
            for (int w = 0; w < NW; ++w) {
                int v = whist[w * E + e];
                whist[w * E + e] = c;
                c += v;
            }
            p.counts[e] = c;
        }
        // block-wide exclusive scan of the counts and of the "touched" flags
        const int f = c > 0 ? 1 : 0;
        int ic = c, iflag = f;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int a = __shfl_up_sync(kFull, ic, o), b = __shfl_up_sync(kFull, iflag, o);
            if (lane >= o) { ic += a; iflag += b; }
        }
        if (lane == 31) { warp_cnt[warp] = ic; warp_flag[warp] = iflag; }
        __syncthreads();
        int pre_c = 0, pre_f = 0;
        for (int w = 0; w < warp; ++w) { pre_c += warp_cnt[w]; pre_f += warp_flag[w]; }
        const int excl_c = pre_c + ic - c, excl_f = pre_f + iflag - f;
        if (e < E) {
            offs[e] = excl_c;
            if (f && p.touched) p.touched[excl_f] = e;
        }
        if (tid == blockDim.x - 1) {           // threads past E carry zeros, so these are the totals
            offs[E] = excl_c + c;
            if (p.meta) p.meta[0] = excl_f + f;
            if (p.touched) p.touched[excl_f + f] = -1;
        }
        // pass list: an expert with c rows is visited in ceil(c/PR) passes of up to PR rows
        if (p.passes) {
            __syncthreads();                   // warp_cnt is reused for the pass-count scan
            const int PR = p.pass_rows > 0 ? p.pass_rows : 4;
            const int np = (c + PR - 1) / PR;
            int ip = np;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                int a = __shfl_up_sync(kFull, ip, o);
                if (lane >= o) ip += a;
            }
            if (lane == 31) warp_cnt[warp] = ip;
            __syncthreads();
            int pre = 0;
            for (int w = 0; w < warp; ++w) pre += warp_cnt[w];
            const int first = pre + ip - np;
            for (int j = 0; j < np; ++j) p.passes[first + j] = make_int4(e, excl_c + PR * j, min(PR, c - PR * j), 0);
            __shared__ int routed_passes;
            if (tid == blockDim.x - 1) routed_passes = first + np;
            __syncthreads();
            const int sp = (p.shared_tokens + PR - 1) / PR;
            for (int j = tid; j < sp; j += blockDim.x)
                p.passes[routed_passes + j] = make_int4(-1, p.routes + PR * j, min(PR, p.shared_tokens - PR * j), p.shared_tok0 + PR * j);
            if (tid == 0 && p.meta) p.meta[1] = routed_passes + sp;
        }
    }
    __syncthreads();
    for (int e = tid; e <= E; e += blockDim.x) p.offsets[e] = offs[e];

    // stable placement
    for (int base = seg_lo; base < seg_hi; base += 32) {
        int r = base + lane;
        int lid = -1;
        if (r < seg_hi) lid = lid_cache ? (int)lid_cache[r] : local_expert(p, r);
        unsigned peers = __match_any_sync(kFull, lid);
        int pos = -1;
        if (lid >= 0) {
            int rank = __popc(peers & ((1u << lane) - 1u));
            pos = offs[lid] + whist[warp * E + lid] + rank;
        }
        __syncwarp();
        if (lid >= 0) {
            if (lane == __ffs(peers) - 1) whist[warp * E + lid] += __popc(peers);
            p.order[pos] = r;
        }
        if (r < seg_hi && p.inv) p.inv[r] = pos;
        __syncwarp();
    }
}

int launch_permute(const PermuteParams& p, cudaStream_t stream) {
    if (p.E < 1 || p.E > FK_MAX_EXPERTS || p.routes < 0) return FK_ERR_ARG;
    // a short dependency chain matters more than width while there are few routes; E must fit the block
    const int warps = (p.routes <= 768 && p.E <= 256) ? 8 : kPermWarps;
    size_t smem = sizeof(int) * ((size_t)warps * p.E + p.E + 2);
    PermuteParams q = p;
    q.cache_routes = 0;
    const size_t cache = ((size_t)p.routes * sizeof(short) + 15) & ~size_t(15);
    if (p.E < 32767 && smem + cache <= 200 * 1024) {      // local expert ids of all routes next to the histograms
        q.cache_routes = p.routes;
        smem += cache;
    }
    FK_CUDA_OK(cudaFuncSetAttribute(permute_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "permute attr");
    FK_CUDA_OK(launch_pdl(permute_kernel, dim3(1), dim3(warps * 32), smem, stream, q), "permute launch");
    FK_LAUNCH_OK("permute launch");
    return FK_OK;
}

// ---------------------------------------------------------------------------------------------
// Stand-alone histogram (any E): block-private shared histogram when it fits, else global atomics.
// ---------------------------------------------------------------------------------------------
template <typename IT>
__global__ void histogram_kernel(const IT* __restrict__ ids, long long n, int E, int* __restrict__ counts, int use_smem) {
    extern __shared__ int h[];
    if (use_smem) {
        for (int i = threadIdx.x; i < E; i += blockDim.x) h[i] = 0;
        __syncthreads();
    }
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        long long id = (long long)ids[i];
        if (id >= 0 && id < E) atomicAdd(use_smem ? &h[id] : &counts[id], 1);
    }
    if (use_smem) {
        __syncthreads();
        for (int i = threadIdx.x; i < E; i += blockDim.x)
            if (h[i]) atomicAdd(&counts[i], h[i]);
    }
}

int launch_histogram(const void* ids, int ids_are_int64, long long count, int E, int* counts, cudaStream_t stream) {
    if (E < 1 || count < 0) return FK_ERR_ARG;
    FK_CUDA_OK(cudaMemsetAsync(counts, 0, sizeof(int) * (size_t)E, stream), "histogram memset");
    if (count == 0) return FK_OK;
    int use_smem = E <= 8192;
    size_t smem = use_smem ? sizeof(int) * (size_t)E : 0;
    int blocks = (int)((count + 1023) / 1024);
    if (blocks > 296) blocks = 296;
    if (ids_are_int64)
        histogram_kernel<long long><<<blocks, 256, smem, stream>>>(reinterpret_cast<const long long*>(ids), count, E, counts, use_smem);
    else
        histogram_kernel<int><<<blocks, 256, smem, stream>>>(reinterpret_cast<const int*>(ids), count, E, counts, use_smem);
    FK_LAUNCH_OK("histogram launch");
    return FK_OK;
}

}  // namespace fk
