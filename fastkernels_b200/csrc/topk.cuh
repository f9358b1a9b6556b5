// Warp-level softmax + top-k with renormalised weights (ties go to the lower expert index).
// Reference semantics: src/fastkernels/reference/qwen36_real.py:335-337.
#pragma once

#include "common.cuh"

namespace fk {

// softmax + top-k of one token's logits held in registers: lane L owns the experts j*32 + L (j < EPL, E <= 32*EPL).
// After the call lane r < top_k holds the r-th winner in (my_i, my_w); my_w is renormalised over the winners.
// Reference: probs = softmax(logits); top-k of probs; weights = selected / sum(selected) (qwen36_real.py:335-337).
// Every router kernel of the library selects through this one function, so they agree bit for bit on equal logits.
struct TopkNoHook {
    __device__ __forceinline__ void operator()(int, int) const {}
};
// on_round(r, expert) is called by every lane as soon as the r-th winner is known (a caller that can start work
// per winner does not have to wait for the last round and the weights).
template <int EPL, typename Hook = TopkNoHook>
__device__ __forceinline__ void topk_warp_regs(float (&v)[EPL], int E, int top_k, int lane, int& my_i, float& my_w,
                                               Hook on_round = Hook()) {
    // Selection works on the logits: softmax is monotonic, so the k largest probabilities are the k largest logits,
    // and the renormalised weight of a winner, p_i / sum of the winners' p_j, is exp(l_i - m) / sum of the winners'
    // exp(l_j - m): the normaliser of the full softmax cancels, and only k exponentials are needed instead of E.
    // An fp32 orders like the unsigned integer (bits ^ sign-extended mask): key 0 is kept for padding and for
    // experts already taken.  Each round is two hardware warp reductions (max of the keys, then min of the indices
    // that hold that key, which is the lower-index tie rule); lane r keeps the r-th winner.
    unsigned key[EPL];
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
        const unsigned u = __float_as_uint(v[j]);
        const unsigned k = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
        key[j] = (j * 32 + lane < E) ? max(k, 1u) : 0u;
    }
    unsigned my_k = 1u;
    my_i = 0;
#pragma unroll 1
    for (int r = 0; r < top_k; ++r) {
        unsigned best = 0u;
#pragma unroll
        for (int j = 0; j < EPL; ++j) best = max(best, key[j]);
        const unsigned mk = __reduce_max_sync(kFull, best);
        unsigned cand = 0x7fffffffu;
#pragma unroll
        for (int j = EPL - 1; j >= 0; --j) cand = (key[j] == mk) ? (unsigned)(j * 32 + lane) : cand;   // lowest j wins
        const unsigned bi = __reduce_min_sync(kFull, cand);
#pragma unroll
        for (int j = 0; j < EPL; ++j) key[j] = ((unsigned)(j * 32 + lane) == bi) ? 0u : key[j];
        if (lane == r) { my_k = mk; my_i = (int)bi; }
        on_round(r, (int)bi);
    }
    // lanes 0..k-1 hold the winners in descending order: lane 0 has the maximum
    const unsigned ku = (my_k & 0x80000000u) ? (my_k & 0x7fffffffu) : ~my_k;
    const float logit = __uint_as_float(ku);
    const float m = __shfl_sync(kFull, logit, 0);
    const float ex = lane < top_k ? expf(logit - m) : 0.f;
    const float total = warp_sum(ex);
    my_w = ex / total;
}

// softmax + top-k of one token's logits by one warp.  EPL = experts per lane (E <= 32*EPL).
template <int EPL>
__device__ void topk_warp(const float* __restrict__ logits_row, int E, int top_k, long long* ids_out,
                          int* ids32_out, float* weights_out, float* weights_out2 = nullptr, long long* ids_out2 = nullptr) {
    const int lane = threadIdx.x & 31;
    float v[EPL];
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
        int e = j * 32 + lane;
        v[j] = e < E ? __ldcg(logits_row + e) : -INFINITY;
    }
    int my_i;
    float w;
    topk_warp_regs<EPL>(v, E, top_k, lane, my_i, w);
    if (lane < top_k) {
        if (ids_out) ids_out[lane] = my_i;
        if (ids_out2) ids_out2[lane] = my_i;
        if (ids32_out) ids32_out[lane] = my_i;
        if (weights_out) weights_out[lane] = w;
        if (weights_out2) weights_out2[lane] = w;
    }
}

}  // namespace fk
