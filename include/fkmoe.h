/* fkmoe.h -- C ABI of libfkmoe.so: the Qwen3.6 MoE decode layer on B200 (sm_100a).
 *
 * Every entry point takes raw DEVICE pointers (unless its name ends in _host),
 * sizes, a dtype code and a CUDA stream (passed as void*; NULL = legacy default
 * stream).  Entry points never allocate, never synchronise and never throw:
 * they enqueue kernels on `stream` and return an fk_status.  Scratch memory is
 * a caller-owned workspace of fk_moe_workspace_bytes() bytes that must have been
 * cleared once with fk_moe_workspace_init() and must not be shared by calls
 * that overlap on the GPU.
 *
 * Each declaration names the reference interface it replaces; paths are
 * relative to the reference project's root (suryavanshi/fastkernels).
 *
 * Layouts (all row-major contiguous, weights in one dtype per call):
 *   hidden [T,H]   norm_weight [H]   router_weight [E,H]
 *   expert_gate_up [E,2I,H] (gate rows 0..I-1, up rows I..2I-1)   expert_down [E,H,I]
 *   shared_gate_up [2I,H]   shared_down [H,I]   shared_gate [H]
 *   logits f32 [T,E]   topk_ids i64 [T,k]   topk_weights f32 [T,k]   out f32 [T,H]
 */
#ifndef FKMOE_H
#define FKMOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum fk_dtype { FK_F32 = 0, FK_BF16 = 1, FK_F16 = 2 };

enum fk_status {
    FK_OK = 0,
    FK_ERR_ARG = 1,          /* null pointer, bad size, limit exceeded */
    FK_ERR_UNSUPPORTED = 2,  /* dtype / shape combination not built */
    FK_ERR_WORKSPACE = 3,    /* workspace too small or misaligned */
    FK_ERR_CUDA = 4,         /* a CUDA runtime call failed (launch error) */
    FK_ERR_TIMEOUT = 5       /* a bounded device-side wait gave up */
};

/* Limits carried over from the reference wrappers
 * (src/fastkernels/kernels/triton/qwen36_router.py:280-288, qwen36_expert.py:850, :1137). */
#define FK_MAX_TOP_K 8
#define FK_MAX_HIDDEN 4096
#define FK_MAX_EXPERTS 1024
#define FK_MAX_INTERMEDIATE 1024

typedef struct fk_moe_dims {
    int32_t tokens;        /* T */
    int32_t hidden;        /* H */
    int32_t experts;       /* E (routed experts held by this call's weight tensors) */
    int32_t intermediate;  /* I */
    int32_t top_k;         /* k */
} fk_moe_dims;

/* flags for fk_moe_call.flags */
#define FK_FLAG_FORCE_GENERIC 1u   /* use the shape-agnostic kernels even where a fast path exists */
#define FK_FLAG_FORCE_GEMV 2u      /* never use the tensor-core grouped GEMM */
#define FK_FLAG_FORCE_TENSOR 4u    /* use the tensor-core grouped GEMM whenever the shape allows */
#define FK_FLAG_NO_FUSED_DECODE 8u /* T<=4: run the staged kernels instead of the single-launch kernels (one token; two to four) */
#define FK_FLAG_TRACE 64u          /* T<=4 single-launch kernels: write per-block phase timestamps at the start of the workspace's y
                                      region, u64 [blocks][32] (fk_moe_trace_offset() gives the offset).  Nanoseconds of
                                      the global timer in slots 0 entry, 1 constant copies issued, 20 the kernel before
                                      has completed, 2 token in shared memory, 3 this block's logits published, 18 all
                                      logits seen, 19 experts selected, 4 producer has the ids, 11 first ring stage
                                      landed, 5 this block's activations published, 12 the activations this block needs
                                      are in shared memory, 14 last copy issued, 13 down tiles done, 15 output stored,
                                      7 exit (0 where a block skips the step); SM cycle counter in 8 (entry) and 9 (exit).
                                      Two to four tokens: 19 is "distinct experts listed", 21 / 5 this block has published the
                                      first / second half of the experts, 22 / 25 every block has, 26 / 27 first down stage
                                      landed / done; no 1, 8, 9.
                                      Ignored when the record (blocks * 256 bytes) does not fit the y region. */
#define FK_FLAG_SKIP_FOREIGN 16u   /* ids outside [expert_base, expert_base+E) are skipped instead of clamped */
#define FK_FLAG_WIDE_PASSES 128u   /* tcgen05 path: 128 tokens per pass and two weight tiles per unit instead of 64 and one */

typedef struct fk_moe_call {
    fk_moe_dims dims;
    int32_t hidden_dtype;          /* fk_dtype of `hidden` */
    int32_t weight_dtype;          /* fk_dtype of every weight tensor */
    float eps;                     /* RMSNorm epsilon (reference default 1e-6) */
    float norm_offset;             /* router norm gain is (norm_offset + norm_weight); reference default 1.0 */
    uint32_t flags;
    int32_t expert_base;           /* expert-parallel shard: ids in [expert_base, expert_base+E) are local,
                                      others are skipped (0 for a whole layer) */
    int32_t shared_token_base;     /* fk_moe_experts: run the shared expert only on tokens [base, base+count);  */
    int32_t shared_token_count;    /* count 0 = all tokens (expert parallel: the rank's own tokens among the gathered ones) */
    const void* hidden;
    const void* norm_weight;
    const void* router_weight;
    const float* router_bias;      /* optional f32 [E] added to the logits, or NULL */
    const void* expert_gate_up;
    const void* expert_down;
    const void* shared_gate_up;    /* NULL: no shared expert */
    const void* shared_down;
    const void* shared_gate;       /* NULL: shared expert is not gated */
    const int64_t* topk_ids_in;    /* fk_moe_experts only: routing given by the caller */
    const float* topk_weights_in;
    float* out;                    /* f32 [T,H]: the MoE update */
    float* layer_hidden;           /* optional f32 [T,H]: hidden + update, or NULL */
    float* logits;                 /* f32 [T,E] */
    int64_t* topk_ids;             /* i64 [T,k] */
    float* topk_weights;           /* f32 [T,k] */
    void* workspace;
    size_t workspace_bytes;
} fk_moe_call;

/* Library identification and error text. */
int fk_version(void);
const char* fk_status_string(int status);
/* Text of the last CUDA error seen by this thread inside the library ("" if none). */
const char* fk_last_cuda_error(void);

/* Number of kernels this library has launched in this process (all threads, all entry points). */
uint64_t fk_launch_count(void);

/* Profiling aid, not a hot path: runs fk_moe_layer with CUDA events recorded on `stream`
 * between its stages, WAITS for the last one, and writes the stage durations in milliseconds
 * to stage_ms (room for 11) and their number to *stages.  Staged path: router, permute,
 * [row gather, tensor-core path only], gate_up, down, combine; single-token kernel: one stage.  No counterpart in the reference (it times with a host clock around
 * a Python loop, e.g. bench/qwen36_real_moe_microbench.py:101-119). */
int fk_moe_layer_timed(const fk_moe_call* call, void* stream, float* stage_ms, int* stages);
/* The same for fk_moe_experts: permute (with the shared-gate kernel, if any), [row gather], gate_up, down, combine. */
int fk_moe_experts_timed(const fk_moe_call* call, void* stream, float* stage_ms, int* stages);

/* Limit of every device-side wait on another block or another rank, in SM clock cycles (default: about one
 * second; 0 restores the default).  A wait that runs out never traps and never spins on: the kernel raises an
 * error word, finishes with undefined output, and the next fk_moe_status / fk_ep_status call reports it.
 * Process-wide; applies to calls enqueued afterwards.  No counterpart in the reference, which has no
 * device-side waits (each of its stages is a separate launch, e.g.
 * src/fastkernels/kernels/triton/qwen36_expert.py:1249-1308). */
int fk_set_wait_limit_cycles(long long cycles);

/* Synchronises the device and reports whether a bounded device-side wait of a call that used `workspace`
 * gave up since the last fk_moe_status on it: FK_OK, or FK_ERR_TIMEOUT with *code (may be NULL) = 1 grouped
 * GEMV kernels, 2 single-token kernel, 3 tensor-core grouped GEMM.  The word is cleared, so the workspace
 * can be used again.  No counterpart in the reference (see fk_set_wait_limit_cycles). */
int fk_moe_status(void* workspace, size_t workspace_bytes, int* code);

/* Byte offset inside the workspace of the FK_FLAG_TRACE record for these dims. */
size_t fk_moe_trace_offset(const fk_moe_dims* dims);

/* Scratch size for a call with these dims (0 on invalid dims); and the one-time clear. */
size_t fk_moe_workspace_bytes(const fk_moe_dims* dims);
int fk_moe_workspace_init(void* workspace, size_t bytes, void* stream);

/* Router: RMSNorm * (norm_offset + w) -> GEMV [E,H] -> (+bias) -> softmax -> top-k (ties to the
 * lower expert index) -> renormalise.  Uses call->{hidden,norm_weight,router_weight,router_bias,
 * logits,topk_ids,topk_weights}.
 * Replaces triton_qwen36_moe_router_decode / triton_qwen36_batched_moe_router_decode
 * (src/fastkernels/kernels/triton/qwen36_router.py:193, :260); oracle
 * src/fastkernels/reference/qwen36_real.py:333-337. */
int fk_moe_router(const fk_moe_call* call, void* stream);

/* The router for callers that cannot allocate device memory.  No counterpart in the reference.
 * Some hosts may not call cudaMalloc at all: a plugin whose device memory is entirely owned and
 * budgeted by its framework, a serving loop with a latency bound that must never enter the
 * allocator, a sandboxed extension that is only handed input and output buffers.  fk_moe_router needs a workspace (for its per-tile completion
 * tickets) that such a caller has nowhere to get from.  This variant keeps the tickets in a fixed
 * 4 KB array inside the library image (every GPU that loads the library holds it until exit), so the
 * caller passes only inputs and outputs: call->workspace is ignored.  It calls no cudaMalloc, no
 * cudaFree and no allocating library routine.
 *   - at most FK_NOALLOC_MAX_TOKENS tokens per call; more is refused with FK_ERR_ARG and a message
 *     in fk_last_cuda_error();
 *   - the first call on each device looks the array's device address up (with that device current);
 *     make that first call before any stream capture begins; the address is kept per device ordinal
 *     for the life of the process, so do not call this after a cudaDeviceReset of that device;
 *   - all calls on a device share the one array, cleared on `stream` at the start of every call:
 *     calls that overlap on the GPU (different streams) race on it, so keep them on one stream or
 *     otherwise ordered. */
#define FK_NOALLOC_MAX_TOKENS 4096
int fk_moe_router_noalloc(const fk_moe_call* call, void* stream);

/* Routed experts (+ optional shared expert, + optional sigmoid gate) for routing given in
 * call->topk_ids_in / topk_weights_in; writes call->out (and layer_hidden if set).
 * Replaces triton_qwen36_{,batched_}routed_experts_decode and
 * triton_qwen36_{,batched_}routed_shared_experts_decode
 * (src/fastkernels/kernels/triton/qwen36_expert.py:889, :969, :1096, :1181); oracle
 * src/fastkernels/reference/qwen36_real.py:339-353.  Out-of-range expert ids are clamped
 * as the reference kernels do (qwen36_expert.py:485) unless expert_base/E select a shard. */
int fk_moe_experts(const fk_moe_call* call, void* stream);

/* Whole layer: router -> routed + shared experts (-> residual).
 * Replaces triton_qwen36_moe_decode / triton_qwen36_batched_moe_decode
 * (qwen36_expert.py:1312, :1353) and triton_qwen36_batched_moe_layer_decode
 * (src/fastkernels/kernels/triton/qwen36_layer.py:55); oracle qwen36_real_moe_update
 * (src/fastkernels/reference/qwen36_real.py:329-354). */
int fk_moe_layer(const fk_moe_call* call, void* stream);

/* Same as fk_moe_layer, but hidden/out/layer_hidden/logits/topk_ids/topk_weights are HOST
 * pointers (pinned memory recommended); weights and workspace stay device pointers.
 * layer_hidden, logits, topk_ids and topk_weights may be NULL: that result is then not copied back.
 * `staging` is a device buffer of fk_moe_host_staging_bytes(dims, hidden_dtype) bytes.  The copies are enqueued on
 * `stream`; the caller synchronises the stream before reading the results. */
size_t fk_moe_host_staging_bytes(const fk_moe_dims* dims, int hidden_dtype);
int fk_moe_layer_host(const fk_moe_call* call, void* staging, size_t staging_bytes, void* stream);

/* Single expert MLP for one token: out f32 [H] = Wd (silu(Wg x) * (Wu x)).
 * Replaces triton_qwen36_single_expert_mlp_decode (qwen36_expert.py:817). */
int fk_single_expert_mlp(const void* hidden, int hidden_dtype, const void* gate_up, const void* down,
                         int weight_dtype, float* out, int hidden_size, int intermediate,
                         void* workspace, size_t workspace_bytes, void* stream);

/* Layer boundary of a stack of MoE layers: x[t,:] += update[t,:] (fp32, in place; update may be NULL),
 * then normed[t,:] = x[t,:] * rsqrt(mean(x[t,:]^2) + eps) in `out_dtype` (unit gain).
 * The reference composes layers in Python (hidden + update, src/fastkernels/kernels/triton/qwen36_layer.py:94-105,
 * then the next block's norm, src/fastkernels/reference/qwen36_real.py:23-28); this is that step as one kernel. */
int fk_residual_rmsnorm(float* x, const float* update, void* normed, int out_dtype, int tokens, int hidden_size,
                        float eps, void* stream);

/* out[n,c] = silu(gate_up[n,c]) * gate_up[n,I+c], fp32 math, stored in the input dtype.
 * Replaces triton_fused_swiglu (src/fastkernels/kernels/triton/moe.py:67); oracle
 * reference_fused_swiglu (src/fastkernels/reference/moe.py:16). */
int fk_fused_swiglu(const void* gate_up, void* out, int dtype, int64_t rows, int intermediate, void* stream);

/* counts[e] = number of ids equal to e (ids outside [0,E) are ignored); counts is int32 [E].
 * Replaces triton_expert_histogram (src/fastkernels/kernels/triton/moe.py:87); oracle
 * reference_expert_histogram (src/fastkernels/reference/moe.py:24). */
int fk_expert_histogram(const void* ids, int ids_are_int64, int64_t count, int num_experts,
                        int32_t* counts, void* stream);

/* Histogram, exclusive offsets and the stable expert-major order of the T*k routes:
 * order = argsort(ids.flatten(), stable).  counts i32 [E], offsets i32 [E+1], order i32 [T*k].
 * The reference has no packing function (docs/QWEN36_MEGAKERNEL_PLAN.md:142-149 lists it as
 * future work); this is the packing step its grouped-expert plan describes. */
int fk_moe_permute(const int64_t* topk_ids, int tokens, int top_k, int num_experts,
                   int32_t* counts, int32_t* offsets, int32_t* order,
                   void* workspace, size_t workspace_bytes, void* stream);

/* One token through one layer of a stack, x_next = x + MoE(RMSNorm(x)) with the previous layer's update still
 * to be added: resid_out = resid_in + update_in (update_in may be NULL), the layer runs on the unit-gain RMS norm
 * (norm_eps) of resid_out rounded to c->hidden_dtype, and c->out receives this layer's update (to be passed as
 * update_in of the next call).  c->hidden is not read.  resid_out must not be resid_in.  The residual add and the
 * norm happen inside the single-token kernel, so a stack needs one launch per layer.  dims.tokens must be 1 and the
 * shapes those of the fused kernel, else FK_ERR_UNSUPPORTED (use fk_residual_rmsnorm + fk_moe_layer then).
 * Counterpart in the reference: the per-layer residual add of its decode loop
 * (src/fastkernels/kernels/triton/qwen36_layer.py:94-105) and the norm feeding the MoE block (:167-190). */
int fk_moe_layer_residual(const fk_moe_call* c, const float* resid_in, const float* update_in, float* resid_out,
                          float norm_eps, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Expert-parallel layer over peer memory (one node, one process per GPU, NVLink).
 * The reference has no distributed code (no torch.distributed / NCCL / MPI call site anywhere; its plan
 * lists expert-parallel dispatch as future work, docs/QWEN35_KERNEL_PLAN.md:83).  Semantics: those of
 * triton_qwen36_batched_moe_decode (src/fastkernels/kernels/triton/qwen36_expert.py:1353) applied to the
 * concatenation of all ranks' tokens, with rank r holding experts [r*E/world, (r+1)*E/world).
 *
 * Every rank owns one exchange buffer (fk_ep_buffer_create) and maps every other rank's buffer through a
 * CUDA IPC handle (fk_ep_buffer_open).  fk_moe_layer_ep then runs the whole layer for this rank in one
 * call: router on the rank's own tokens; a dispatch kernel that stores activations and routing of those
 * tokens into every rank's buffer and exchanges arrival flags; the local experts on all gathered tokens;
 * a combine kernel that stores each token's partial row straight into its home rank's buffer and
 * exchanges flags again; a fixed-order sum of the world partials.  No collective library call and no host
 * synchronisation are involved, so the call can be captured in a CUDA graph.  All ranks must make the
 * same sequence of calls.  Waits on peers are bounded (about a second); a rank that gives up sets the
 * error word read by fk_ep_status and finishes with undefined output.
 * --------------------------------------------------------------------------------------------- */
#define FK_EP_MAX_RANKS 8
#define FK_EP_HANDLE_BYTES 64

typedef struct fk_ep_comm {
    int32_t rank, world;
    int32_t tokens_per_rank;           /* fixed for the life of the buffers */
    int32_t reserved;
    void* base[FK_EP_MAX_RANKS];       /* exchange buffer of rank r as mapped in THIS process (own: base[rank]) */
    size_t bytes;                      /* size of each buffer */
} fk_ep_comm;

/* Bytes of one rank's exchange buffer (0 for bad arguments). */
size_t fk_ep_buffer_bytes(int world, int tokens_per_rank, int hidden, int top_k, int hidden_dtype);
/* Allocates (cudaMalloc) and clears a buffer on the current device and returns its IPC handle. */
int fk_ep_buffer_create(size_t bytes, void** buffer, void* handle_out);
/* Maps another process's buffer from its handle / unmaps it / frees an own buffer. */
int fk_ep_buffer_open(const void* handle, void** buffer);
int fk_ep_buffer_close(void* buffer);
int fk_ep_buffer_destroy(void* buffer);
/* One expert-parallel layer call for this rank.  `c` describes the rank's own tokens (dims.tokens ==
 * comm->tokens_per_rank, dims.experts == the GLOBAL expert count, expert_gate_up / expert_down == the rank's
 * block of experts); outputs as for fk_moe_layer.  The workspace must hold
 * fk_moe_workspace_bytes({world*tokens, hidden, experts/world, intermediate, top_k}). */
int fk_moe_layer_ep(const fk_moe_call* c, const fk_ep_comm* comm, void* stream);
/* Synchronises the device and returns the buffer's error word in *error (0: no wait ever gave up; 1: the wait
 * for the ranks' dispatched rows, 2: the wait for their partial rows; the first one that gave up is kept). */
int fk_ep_status(const fk_ep_comm* comm, int* error);
/* Clears an OWN exchange buffer's header (arrival epochs, tickets, error word) after a failed call, once every
 * rank has stopped using the buffers; all ranks reset theirs before the next fk_moe_layer_ep. Synchronises. */
int fk_ep_buffer_reset(void* buffer);
/* fk_moe_layer_ep with CUDA events between its stages (profiling aid, waits for the call): router, dispatch +
 * wait, permutation, [row gather, tensor-core path only], gate_up, down, combine + wait, reduce.
 * stage_ms has room for 11 values. */
int fk_moe_layer_ep_timed(const fk_moe_call* c, const fk_ep_comm* comm, void* stream, float* stage_ms, int* stages);

#ifdef __cplusplus
}
#endif
#endif /* FKMOE_H */
