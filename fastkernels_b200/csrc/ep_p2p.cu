// Expert-parallel exchange over peer memory: dispatch, combine and reduce kernels.
//
// Every rank owns one exchange buffer that all ranks of the node have mapped (CUDA IPC over NVLink):
//   header   64 x u32   [0..8)  dispatch arrival epochs, one word per source rank (written by that rank)
//                       [8..16) combine arrival epochs, one word per source rank
//                       [16] dispatch epoch of this rank   [17] combine epoch of this rank
//                       [18] dispatch ticket   [19] combine ticket   [20] error word
//   hidden   [world*T, H]   activations of every rank's tokens, rank-major
//   ids      [world*T, k]   i32 global expert ids
//   weights  [world*T, k]   f32 routing weights
//   partial  [world, T, H]  f32: slice g holds rank g's partial rows for THIS rank's tokens; a row is written only
//                           if rank g holds one of the token's experts (or is the home rank running the shared
//                           expert): the home rank derives the same set from the token's ids and reads nothing else
//
// Dispatch: each rank stores its own rows into slot `rank` of every buffer (plain 16-byte stores to peer
// memory); every block fences at device scope and takes a ticket, and the last block to finish fences at system
// scope, publishes the rank's new epoch in every buffer's flag word (release) and then waits until every rank's
// epoch has arrived in its own buffer (acquire).  The combine
// does the same with the partial rows.  Epochs only grow and live in device memory, so a captured graph
// replays correctly.  A buffer is never overwritten while a peer still reads it: rank A can only start call
// n+1 after it has seen every rank's combine flag of call n, and a rank raises that flag after its own
// local-expert kernels (the readers of its dispatch slots) have finished; A's partial slots are read by the
// home rank's reduce of call n, which precedes that rank's dispatch flag of call n+1, which A waits for
// before it writes partials again.
//
// Reference semantics: src/fastkernels/reference/qwen36_real.py:329-354 on the gathered tokens; the
// reference itself has no multi-GPU code.

#include "common.cuh"
#include "kernels.cuh"
#include "tma.cuh"

namespace fk {

__host__ __device__ inline size_t ep_align(size_t v) { return (v + 255) & ~size_t(255); }

EpLayout ep_layout(int world, int tokens, int hidden, int top_k, int hidden_dtype) {
    EpLayout l{};
    const size_t es = hidden_dtype == FK_F32 ? 4 : 2;
    size_t o = 256;
    l.hidden = o; o += ep_align((size_t)world * tokens * hidden * es);
    l.ids = o; o += ep_align((size_t)world * tokens * top_k * 4);
    l.weights = o; o += ep_align((size_t)world * tokens * top_k * 4);
    l.partial = o; o += ep_align((size_t)world * tokens * hidden * 4);
    l.total = o;
    return l;
}

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Called by the threads of ONE block after every block of the grid has fenced its stores (ticket): thread r
// publishes this rank's next epoch to rank r and waits for rank r's epoch in the own buffer.  `slot0` is 0 for
// the dispatch words, 8 for the combine words; `counter` is the matching epoch word of this rank.
__device__ __forceinline__ void ep_signal_and_wait(const EpPeers& ep, int slot0, int counter) {
    __shared__ unsigned epoch_s;
    unsigned* mine = ep.header[ep.rank];
    if (threadIdx.x == 0) {
        const unsigned e = mine[counter] + 1u;
        mine[counter] = e;
        epoch_s = e;
    }
    __syncthreads();
    const unsigned epoch = epoch_s;
    if ((int)threadIdx.x < ep.world) {
        const int r = threadIdx.x;
        st_release_sys(ep.header[r] + slot0 + ep.rank, epoch);
        const unsigned* flag = mine + slot0 + r;
        const long long t0 = clock64();
        // epochs only grow; the signed difference keeps the comparison right across a wrap
        while ((int)(ld_acquire_sys(flag) - epoch) < 0) {
            __nanosleep(64);
            if (clock64() - t0 > ep.wait_cycles) {
                atomicCAS(reinterpret_cast<int*>(mine + 20), 0, slot0 == 0 ? 1 : 2);     // the first wait that gave up is kept
                break;
            }
        }
    }
    __syncthreads();
}

// True in every thread of the last block of the grid to get here (self-resetting ticket).
//
// Ordering of all blocks' stores to peer memory before the flag that the last block raises: a block's threads meet at
// a barrier; the thread that takes the ticket fences at DEVICE scope first (fence + ticket: a release towards the
// other blocks of this GPU); the last block's ticket + fence is the matching acquire, and that fence is at SYSTEM
// scope, followed by st.release.sys of the flag.  Every block's stores thereby precede the flag in causality order,
// which is what a peer that acquires the flag relies on.  A system-scope fence in every block is not needed for that
// and is what these kernels used to spend their time in: it took 6-9 us per block (all blocks at once) against
// 0.5-1.7 us for the device-scope fence (dispatch of 1 MB: 10 -> 4.7 us from start to flag; combine: 19 -> 11 us).
__device__ __forceinline__ bool ep_last_block(unsigned* ticket) {
    __shared__ int last_s;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned total = gridDim.x * gridDim.y;
        const unsigned t = atomicAdd(ticket, 1u);
        last_s = (t == total - 1u);
        if (last_s) {
            *ticket = 0u;              // re-arm for the next launch
            __threadfence_system();
        }
    }
    __syncthreads();
    return last_s != 0;
}

// grid (chunks, world): block column r stores this rank's rows into rank r's buffer
__global__ void __launch_bounds__(256) ep_dispatch_kernel(EpDispatchParams p) {
    pdl_trigger();
    pdl_wait();
    const EpPeers& ep = p.peers;
    const int r = blockIdx.y;
    unsigned char* dst_base = reinterpret_cast<unsigned char*>(ep.header[r]);
    const size_t row_bytes = (size_t)p.H * p.elem_bytes;
    // activations: 16-byte vectors
    {
        const uint4* src = reinterpret_cast<const uint4*>(p.hidden);
        uint4* dst = reinterpret_cast<uint4*>(dst_base + p.layout.hidden + (size_t)ep.rank * p.T * row_bytes);
        const size_t n = (size_t)p.T * row_bytes / 16;
        for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) dst[i] = src[i];
    }
    // routing: ids narrowed to i32, weights as they are
    {
        int* dst_ids = reinterpret_cast<int*>(dst_base + p.layout.ids) + (size_t)ep.rank * p.T * p.top_k;
        float* dst_w = reinterpret_cast<float*>(dst_base + p.layout.weights) + (size_t)ep.rank * p.T * p.top_k;
        const int n = p.T * p.top_k;
        for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
            dst_ids[i] = (int)p.ids[i];
            dst_w[i] = p.weights[i];
        }
    }
    if (ep_last_block(ep.header[ep.rank] + 18)) ep_signal_and_wait(ep, 0, 16);
}

// Ordered combine whose rows go to the tokens' home ranks: token t of the gathered batch belongs to rank
// t / T_local; this rank's partial for it lands in slice `rank` of that rank's partial buffer.
__global__ void __launch_bounds__(256) combine_ep_kernel(ExpertParams p) {
    pdl_trigger();
    pdl_wait();
    const EpPeers& ep = p.ep;
    const int H4 = p.H >> 2;
    const long long total = (long long)p.T * H4;
    for (long long i = (blockIdx.x + (long long)blockIdx.y * gridDim.x) * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * gridDim.y * blockDim.x) {
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
        if (shared) { acc.x += gate * sh.x; acc.y += gate * sh.y; acc.z += gate * sh.z; acc.w += gate * sh.w; }
        // a token none of whose experts live here (and that is not one of this rank's own, shared-expert tokens)
        // gets no row from this rank: its home rank knows from the token's ids and skips the slot
        bool any = shared;
#pragma unroll
        for (int s = 0; s < FK_MAX_TOP_K; ++s) any = any || pos[s] >= 0;
        if (!any) continue;
        const int home = t / ep.tokens, tl = t - home * ep.tokens;
        float* dst = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(ep.header[home]) + ep.partial_offset) +
                     ((size_t)ep.rank * ep.tokens + tl) * p.H + h;
        *reinterpret_cast<float4*>(dst) = acc;
    }
    if (ep_last_block(ep.header[ep.rank] + 19)) ep_signal_and_wait(ep, 8, 17);
}

// out[t] = sum over the ranks g (ascending) that hold one of token t's experts, plus this rank when it ran the shared
// expert for t, of partial[g][t]  (+ hidden[t] into layer_hidden).  Slots of other ranks were not written.
__global__ void __launch_bounds__(256) ep_reduce_kernel(const float* partial, int world, int rank, int T, int H, const long long* ids,
                                                        int top_k, int experts_per_rank, int own_always, float* out,
                                                        float* layer_hidden, const void* hidden, int hidden_dtype) {
    pdl_trigger();
    pdl_wait();
    const int H4 = H >> 2;
    const long long total = (long long)T * H4;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const size_t o = (size_t)i * 4;
        const int t = (int)(i / H4);
        unsigned mask = own_always ? (1u << rank) : 0u;
        for (int s = 0; s < top_k; ++s) {
            const long long e = ids[(size_t)t * top_k + s];
            if (e >= 0 && e < (long long)experts_per_rank * world) mask |= 1u << (int)(e / experts_per_rank);
        }
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int g = 0; g < world; ++g) {
            if (!((mask >> g) & 1u)) continue;
            const float4 v = *reinterpret_cast<const float4*>(partial + (size_t)g * T * H + o);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        *reinterpret_cast<float4*>(out + o) = acc;
        if (layer_hidden) {
            float4 r;
            r.x = load_any(hidden, hidden_dtype, o) + acc.x; r.y = load_any(hidden, hidden_dtype, o + 1) + acc.y;
            r.z = load_any(hidden, hidden_dtype, o + 2) + acc.z; r.w = load_any(hidden, hidden_dtype, o + 3) + acc.w;
            *reinterpret_cast<float4*>(layer_hidden + o) = r;
        }
    }
}

int launch_ep_dispatch(const EpDispatchParams& p, cudaStream_t stream) {
    const size_t vecs = (size_t)p.T * p.H * p.elem_bytes / 16;
    int bx = (int)((vecs + 255) / 256);
    if (bx < 1) bx = 1;
    if (bx > 64) bx = 64;
    FK_CUDA_OK(launch_pdl(ep_dispatch_kernel, dim3(bx, p.peers.world), dim3(256), 0, stream, p), "ep dispatch launch");
    FK_LAUNCH_OK("ep dispatch launch");
    return FK_OK;
}

int launch_combine_ep(const ExpertParams& p, cudaStream_t stream) {
    const long long total = (long long)p.T * (p.H / 4);
    int blocks = (int)((total + 255) / 256);
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (blocks < 1) blocks = 1;
    FK_CUDA_OK(launch_pdl(combine_ep_kernel, dim3(blocks, 1), dim3(256), 0, stream, p), "ep combine launch");
    FK_LAUNCH_OK("ep combine launch");
    return FK_OK;
}

int launch_ep_reduce(const float* partial, int world, int rank, int T, int H, const long long* ids, int top_k, int experts_per_rank,
                     int own_always, float* out, float* layer_hidden, const void* hidden, int hidden_dtype, cudaStream_t stream) {
    const long long total = (long long)T * (H / 4);
    int blocks = (int)((total + 255) / 256);
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (blocks < 1) blocks = 1;
    FK_CUDA_OK(launch_pdl(ep_reduce_kernel, dim3(blocks), dim3(256), 0, stream, partial, world, rank, T, H, ids, top_k,
                          experts_per_rank, own_always, out, layer_hidden, hidden, hidden_dtype), "ep reduce launch");
    FK_LAUNCH_OK("ep reduce launch");
    return FK_OK;
}

}  // namespace fk
