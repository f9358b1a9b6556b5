// Parameter blocks and host launchers of the individual kernels (internal to libfkmoe).
#pragma once

#include "common.cuh"

namespace fk {

struct RouterParams {
    const void* hidden;
    int hidden_dtype;
    const void* norm_weight;
    const void* router_weight;
    const float* router_bias;          // optional
    const void* shared_gate_weight;    // optional
    float* logits;
    long long* topk_ids;
    float* topk_weights;
    int* ids32;                        // optional int32 copy of the ids (workspace)
    float* shared_gate_out;            // optional f32 [T]
    long long* ids_mirror;             // optional second copy of ids / weights (e.g. the caller's pinned host buffers)
    float* weights_mirror;
    unsigned* tickets;
    int T, H, E, top_k;
    float eps, norm_offset;
};
int launch_router(const RouterParams& p, int weight_dtype, cudaStream_t stream);
int launch_router_noalloc(RouterParams p, int weight_dtype, cudaStream_t stream);   // tickets in a static device array

struct PermuteParams {
    const long long* ids64;   // one of ids64 / ids32 is set
    const int* ids32;
    int routes;               // T*k
    int E;                    // local experts
    int expert_base;          // ids are global; local id = id - expert_base
    int skip_foreign;         // 1: ids outside the local range are dropped, 0: clamped into range
    int* counts;              // [E]
    int* offsets;             // [E+1]
    int* touched;             // [E+1] (optional)
    int* order;               // [routes]: packed row -> route (rows beyond offsets[E] are unused)
    int* inv;                 // [routes]: route -> packed row, -1 if dropped (optional)
    int* meta;                // [0] = number of experts with count>0, [1] = number of passes (optional)
    int4* passes;             // optional GEMV pass list: routed experts ascending, then the shared expert
    int shared_tokens;        // tokens the shared expert sees (0: no shared expert)
    int shared_tok0;          // first of them
    int pass_rows;            // rows per pass: 4 or 8 for the GEMV kernels, 64 for the tensor-core GEMM
    int cache_routes;         // set by the launcher: routes whose local expert ids fit in shared memory (0: none)
};
int launch_permute(const PermuteParams& p, cudaStream_t stream);
int launch_histogram(const void* ids, int ids_are_int64, long long count, int E, int* counts, cudaStream_t stream);

// Expert-parallel exchange over peer memory (ep_p2p.cu)
struct EpLayout {              // byte offsets inside one rank's exchange buffer (256-byte header first)
    size_t hidden, ids, weights, partial, total;
};
EpLayout ep_layout(int world, int tokens, int hidden, int top_k, int hidden_dtype);

struct EpPeers {
    unsigned* header[8];       // exchange buffer of every rank as mapped in this process
    size_t partial_offset;     // EpLayout::partial
    int world, rank;           // world == 0: not expert parallel
    int tokens;                // tokens per rank
    long long wait_cycles;     // limit of a wait on a peer's flag
};

struct EpDispatchParams {
    EpPeers peers;
    EpLayout layout;
    const void* hidden;        // this rank's [T,H]
    const long long* ids;      // [T,k] global expert ids
    const float* weights;      // [T,k]
    int T, H, top_k, elem_bytes;
};
int launch_ep_dispatch(const EpDispatchParams& p, cudaStream_t stream);
int launch_ep_reduce(const float* partial, int world, int rank, int T, int H, const long long* ids, int top_k, int experts_per_rank,
                     int own_always, float* out, float* layer_hidden, const void* hidden, int hidden_dtype, cudaStream_t stream);

struct ExpertParams {
    const void* hidden;
    int hidden_dtype;
    const void* gate_up;          // [E,2I,H]
    const void* down;             // [E,H,I]
    const void* shared_gate_up;   // optional
    const void* shared_down;
    int T, H, E, I, top_k;
    int routes;                   // T*k
    int shared_tok0, shared_n;    // the shared expert runs on tokens [shared_tok0, shared_tok0 + shared_n)
    const int* counts;
    const int* offsets;
    const int* touched;
    const int* order;
    const int* inv;
    const int* meta;
    const int4* passes;
    const float* topk_weights;    // [T,k]
    const float* shared_gate;     // optional f32 [T] (already sigmoid)
    float* act;                   // [(routes+T), I]
    float* y;                     // [(routes+T), H]
    float* out;                   // [T,H]
    float* layer_hidden;          // optional [T,H]
    int* error_word;              // optional: set to non-zero when a bounded device-side wait gave up
    EpPeers ep;                   // ep.world > 0: the combine stores every token's row into its home rank's buffer
};
int launch_combine_ep(const ExpertParams& p, cudaStream_t stream);
// shape-agnostic kernels (any dtype, any H/I)
int launch_experts_generic(const ExpertParams& p, int weight_dtype, cudaStream_t stream);
// bf16 grouped GEMV fed by bulk copies through a shared-memory ring (H, I in {256, 512, 1024, 2048})
bool stream_path_supported(const ExpertParams& p, int weight_dtype);
int launch_experts_stream(const ExpertParams& p, cudaStream_t stream);
int stream_pass_rows(const ExpertParams& p);    // 8 when both streaming kernels run their tensor-core consumers, else 4
// tcgen05 grouped GEMM (bf16, H and I multiples of 128); needs a pass list of <= 64-row passes
bool tc_path_supported(const ExpertParams& p, int weight_dtype);
int launch_experts_tc(const ExpertParams& p, __nv_bfloat16* xg, __nv_bfloat16* actb, int pass_rows, cudaStream_t stream);   // pass_rows 64 or 128
// ordered weighted combine of the per-row outputs (+ shared expert, + residual)
int launch_combine(const ExpertParams& p, cudaStream_t stream);

// one token, whole layer, one launch (bf16 weights)
struct DecodeParams {
    const void* hidden;
    int hidden_dtype;
    const void* norm_weight;
    const void* router_weight;
    const float* router_bias;
    const void* gate_up;
    const void* down;
    const void* shared_gate_up;   // optional
    const void* shared_down;
    const void* shared_gate;      // optional
    float* logits;                // [E]
    long long* topk_ids;          // [k]
    float* topk_weights;          // [k]
    long long* ids_mirror;        // optional second copy of ids / weights (the caller's pinned host buffers)
    float* weights_mirror;
    float* out;                   // [H]
    float* layer_hidden;          // optional [H]
    unsigned* bar;                // workspace [4]: word 3 is the launch epoch (the tag of the next launch minus one)
    unsigned long long* tagged;   // workspace [E]: (launch tag << 32 | logit bits), how the blocks exchange the logits
    unsigned long long* actw;     // workspace [(k+1)*I + 1]: (tag << 32 | bf16 head << 16 | bf16 remainder) per SwiGLU
                                  //   activation of the k slots and the shared expert; last word: the shared gate (fp32 bits)
    uint32_t* act_rows;           // decode_few: workspace [36][I / 2] pairs of bf16, the activations of its (expert, token) rows
    int* error_word;
    unsigned long long* trace;    // optional [blocks][16] nanosecond timestamps of the phase boundaries
    int H, E, I, top_k;
    int T;                        // tokens: 1 for the single-token kernel, 2..4 for decode_few (all arrays then have T rows)
    float eps, norm_offset;
    long long wait_cycles;        // limit of every wait on another block (0: the library's current limit)

    // layer-stack mode (resid_in != null): the token is RMSNorm(resid_in + update_in) with unit gain, rounded to the
    // activation dtype of `hidden_dtype`; `hidden` is not read; resid_out receives resid_in + update_in
    const float* resid_in;        // [H] fp32 residual stream
    const float* update_in;       // [H] fp32 update of the previous layer, or null
    float* resid_out;             // [H] (a different buffer than resid_in: other blocks still read that one)
    float resid_eps;
};
bool decode1_supported(const DecodeParams& p, int weight_dtype);
int launch_decode1(const DecodeParams& p, cudaStream_t stream);
// the same layer call for two to four tokens in one launch (decode_few.cu)
bool decode_few_supported(const DecodeParams& p, int weight_dtype);
int launch_decode_few(const DecodeParams& p, cudaStream_t stream);
int sm_count();
// Limit, in SM clock cycles, of device-side waits on other blocks or ranks (fk_set_wait_limit_cycles; about a second by default)
long long wait_limit_cycles();

int launch_residual_norm(float* x, const float* update, void* normed, int out_dtype, int T, int H, float eps, cudaStream_t stream);

int launch_swiglu(const void* gate_up, void* out, int dtype, long long rows, int I, cudaStream_t stream);

}  // namespace fk
