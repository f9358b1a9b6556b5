// Warp-level softmax + top-k with renormalised weights (ties go to the lower expert index).
// Reference semantics: src/fastkernels/reference/qwen36_real.py:335-337.
#pragma once

#include "common.cuh"

namespace fk {

// softmax + top-k of one token's logits by one warp.  EPL = experts per lane (E <= 32*EPL).
template <int EPL>
__device__ void topk_warp(const float* __restrict__ logits_row, int E, int top_k, long long* ids_out,
                          int* ids32_out, float* weights_out, float* weights_out2 = nullptr, long long* ids_out2 = nullptr) {
    const int lane = threadIdx.x & 31;
    float v[EPL];
    float m = -INFINITY;
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
        int e = j * 32 + lane;
        v[j] = e < E ? __ldcg(logits_row + e) : -INFINITY;
        m = fmaxf(m, v[j]);
    }
    m = warp_max(m);
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
        int e = j * 32 + lane;
        v[j] = e < E ? expf(v[j] - m) : 0.f;
        s += v[j];
    }
    s = warp_sum(s);
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
        int e = j * 32 + lane;
        v[j] = e < E ? v[j] / s : -1.f;      // probabilities; padding can never win
    }
    // k rounds of warp arg-max; lane r keeps the r-th winner.  Probabilities are non-negative floats,
    // so their bit patterns order like unsigned integers: each round is two hardware warp reductions
    // (max of the keys, then min of the indices that hold that key, which is the lower-index tie rule).
    // key = bits + 1 for a live candidate, 0 for padding and for experts already taken.
    unsigned key[EPL];
#pragma unroll
    for (int j = 0; j < EPL; ++j) key[j] = (j * 32 + lane < E) ? __float_as_uint(v[j]) + 1u : 0u;
    float my_v = 0.f, total = 0.f;
    int my_i = 0;
#pragma unroll 1
    for (int r = 0; r < top_k; ++r) {
        unsigned best = 0u;
#pragma unroll
        for (int j = 0; j < EPL; ++j) best = max(best, key[j]);
        const unsigned m = __reduce_max_sync(kFull, best);
        unsigned cand = 0x7fffffffu;
#pragma unroll
        for (int j = EPL - 1; j >= 0; --j) cand = (key[j] == m) ? (unsigned)(j * 32 + lane) : cand;   // lowest j wins
        const unsigned bi = __reduce_min_sync(kFull, cand);
#pragma unroll
        for (int j = 0; j < EPL; ++j) key[j] = ((unsigned)(j * 32 + lane) == bi) ? 0u : key[j];
        const float bv = __uint_as_float(m - 1u);
        if (lane == r) { my_v = bv; my_i = (int)bi; }
        total += bv;
    }
    if (lane < top_k) {
        const float w = my_v / total;
        if (ids_out) ids_out[lane] = my_i;
        if (ids_out2) ids_out2[lane] = my_i;
        if (ids32_out) ids32_out[lane] = my_i;
        if (weights_out) weights_out[lane] = w;
        if (weights_out2) weights_out2[lane] = w;
    }
}

}  // namespace fk
