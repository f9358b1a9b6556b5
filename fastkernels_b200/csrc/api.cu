// C ABI of libfkmoe (declarations and reference citations: include/fkmoe.h).

#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "kernels.cuh"
#include "tma.cuh"

namespace fk {

static thread_local char g_last_error[256] = "";
static unsigned long long g_launches = 0;
thread_local StageTimer* g_stage_timer = nullptr;

bool pdl_enabled() {
    static const bool on = [] { const char* e = getenv("FKMOE_NO_PDL"); return !(e && e[0] == '1'); }();
    return on;
}

void note_launch() { __atomic_fetch_add(&g_launches, 1ull, __ATOMIC_RELAXED); }

static long long g_wait_cycles = kWaitCycles;
long long wait_limit_cycles() { return __atomic_load_n(&g_wait_cycles, __ATOMIC_RELAXED); }

void note_cuda_error(cudaError_t e, const char* where) {
    snprintf(g_last_error, sizeof(g_last_error), "%s: %s", where, cudaGetErrorString(e));
    (void)cudaGetLastError();   // clear the sticky-less error so later calls are not blamed for it
}

static bool dims_ok(const fk_moe_dims& d, bool need_routing) {
    if (d.tokens < 0 || d.hidden < 1 || d.hidden > FK_MAX_HIDDEN) return false;
    if (d.experts < 1 || d.experts > FK_MAX_EXPERTS) return false;
    if (d.intermediate < 1 || d.intermediate > FK_MAX_INTERMEDIATE) return false;
    if (d.top_k < (need_routing ? 1 : 0) || d.top_k > FK_MAX_TOP_K) return false;
    if ((long long)d.tokens * (d.top_k > 0 ? d.top_k : 1) > (1 << 24)) return false;
    return true;
}

static bool dtype_ok(int dt) { return dt == FK_F32 || dt == FK_BF16 || dt == FK_F16; }

template <typename T>
static T* at(void* base, size_t off) { return reinterpret_cast<T*>(reinterpret_cast<char*>(base) + off); }

static int check_workspace(const fk_moe_call* c, Workspace& w) {
    w = workspace_layout(c->dims);
    if (c->workspace == nullptr || c->workspace_bytes < w.total) return FK_ERR_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(c->workspace) & 255) return FK_ERR_WORKSPACE;
    return FK_OK;
}

// permutation + expert kernels + combine for routing already present in ids/weights
static int run_experts(const fk_moe_call* c, const Workspace& w, const long long* ids, const float* weights,
                       const float* shared_gate_sig, cudaStream_t stream, const int* ids32 = nullptr,
                       const EpPeers* ep_peers = nullptr, int avg_rows_per_expert = 0) {
    const fk_moe_dims& d = c->dims;
    void* ws = c->workspace;
    PermuteParams pp{};
    pp.ids64 = ids;
    pp.ids32 = ids32;
    pp.routes = d.tokens * d.top_k;
    pp.E = d.experts;
    pp.expert_base = c->expert_base;
    pp.skip_foreign = (c->flags & FK_FLAG_SKIP_FOREIGN) ? 1 : 0;
    pp.counts = at<int>(ws, w.counts);
    pp.offsets = at<int>(ws, w.offsets);
    pp.touched = at<int>(ws, w.touched);
    pp.order = at<int>(ws, w.order);
    pp.inv = at<int>(ws, w.inv);
    pp.meta = at<int>(ws, w.meta);
    pp.passes = at<int4>(ws, w.passes);
    // the shared expert may be asked for a sub-range of the tokens (expert parallel: the home rank's own tokens)
    int sh_n = c->shared_token_count > 0 ? c->shared_token_count : d.tokens;
    int sh0 = c->shared_token_count > 0 ? c->shared_token_base : 0;
    if (sh0 < 0 || sh0 + sh_n > d.tokens) return FK_ERR_ARG;
    pp.shared_tokens = c->shared_gate_up ? sh_n : 0;
    pp.shared_tok0 = sh0;

    ExpertParams ep{};
    ep.hidden = c->hidden;
    ep.hidden_dtype = c->hidden_dtype;
    ep.gate_up = c->expert_gate_up;
    ep.down = c->expert_down;
    ep.shared_gate_up = c->shared_gate_up;
    ep.shared_down = c->shared_gate_up ? c->shared_down : nullptr;
    ep.T = d.tokens; ep.H = d.hidden; ep.E = d.experts; ep.I = d.intermediate; ep.top_k = d.top_k;
    ep.routes = pp.routes;
    ep.shared_tok0 = sh0; ep.shared_n = sh_n;
    // Path choice.  The weight-streaming kernels (8-token passes with their tensor-core consumers, 4-token passes with
    // the CUDA-core ones) win while an expert sees few tokens: below 64 tokens per call.  From 64 on the tcgen05
    // grouped GEMM (64-token passes) takes over: at 64 evenly routed tokens the two are level (189 vs 186 us), and
    // when a few experts draw most of the tokens the GEMM reads their weights once instead of once per 8 tokens
    // (64 tokens, eight hot experts: 135 vs 154 us).
    const bool generic = (c->flags & FK_FLAG_FORCE_GENERIC) != 0;
    const bool stream_ok = !generic && stream_path_supported(ep, c->weight_dtype);
    const int stream_rows = stream_ok ? stream_pass_rows(ep) : 4;
    const int stream_max_tokens = 63;
    const bool want_tc = !generic && !(c->flags & FK_FLAG_FORCE_GEMV) &&
                         ((c->flags & FK_FLAG_FORCE_TENSOR) || d.tokens > stream_max_tokens || !stream_ok);
    const bool use_tc = want_tc && (d.tokens >= 64 || (c->flags & FK_FLAG_FORCE_TENSOR)) && tc_path_supported(ep, c->weight_dtype);
    const bool use_stream = !use_tc && stream_ok;
    // Measured for one rank of 8 x 256 tokens: gate_up 57 us with 64-token passes, 75 us with 128-token passes and two
    // weight tiles per unit (fewer bytes cross the SM boundary, but four ring stages instead of seven and one round of
    // large units).  So the wide form stays an option, not a default.
    (void)avg_rows_per_expert;
    const int tc_rows = (c->flags & FK_FLAG_WIDE_PASSES) ? 128 : 64;
    pp.pass_rows = use_tc ? tc_rows : (use_stream ? stream_rows : 4);
    int st = launch_permute(pp, stream);
    if (st != FK_OK) return st;
    stage_mark();   // end of permute

    ep.counts = pp.counts; ep.offsets = pp.offsets; ep.touched = pp.touched;
    ep.order = pp.order; ep.inv = pp.inv; ep.meta = pp.meta; ep.passes = pp.passes;
    ep.topk_weights = weights;
    ep.shared_gate = shared_gate_sig;
    ep.act = at<float>(ws, w.act);
    ep.y = at<float>(ws, w.y);
    ep.out = c->out;
    ep.layer_hidden = c->layer_hidden;

    ep.error_word = at<int>(ws, w.meta) + 2;
    if (use_tc)
        st = launch_experts_tc(ep, at<__nv_bfloat16>(ws, w.xg), at<__nv_bfloat16>(ws, w.actb), tc_rows, stream);
    else if (use_stream)
        st = launch_experts_stream(ep, stream);
    else
        st = launch_experts_generic(ep, c->weight_dtype, stream);
    if (st != FK_OK) return st;
    if (ep_peers) {
        ep.ep = *ep_peers;
        st = launch_combine_ep(ep, stream);
    } else {
        st = launch_combine(ep, stream);
    }
    stage_mark();   // end of combine
    return st;
}

// sigmoid(g . x) per token for callers that skip the router (fk_moe_experts with a gate)
__global__ void shared_gate_kernel(const void* hidden, int hidden_dtype, const void* g, int weight_dtype, float* out,
                                   int T, int H) {
    const int lane = threadIdx.x & 31;
    const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (t >= T) return;
    float acc = 0.f;
    for (int h = lane; h < H; h += 32)
        acc = fmaf(load_any(g, weight_dtype, h), load_any(hidden, hidden_dtype, (size_t)t * H + h), acc);
    acc = warp_sum(acc);
    if (lane == 0) out[t] = sigmoidf_(acc);
}

template <typename F>
static int run_timed(void* stream, float* stage_ms, int* stages, F&& call) {
    if (!stage_ms || !stages) return FK_ERR_ARG;
    StageTimer t{};
    t.stream = (cudaStream_t)stream;
    for (int i = 0; i < 12; ++i) FK_CUDA_OK(cudaEventCreate(&t.ev[i]), "event create");
    g_stage_timer = &t;
    int st = call();
    g_stage_timer = nullptr;
    *stages = 0;
    if (st == FK_OK && t.used >= 2) {
        FK_CUDA_OK(cudaEventSynchronize(t.ev[t.used - 1]), "event sync");
        for (int i = 1; i < t.used; ++i) cudaEventElapsedTime(&stage_ms[i - 1], t.ev[i - 1], t.ev[i]);
        *stages = t.used - 1;
    }
    for (int i = 0; i < 12; ++i) cudaEventDestroy(t.ev[i]);
    return st;
}

}  // namespace fk

using namespace fk;

extern "C" {

int fk_version(void) { return 100; }

const char* fk_status_string(int status) {
    switch (status) {
        case FK_OK: return "ok";
        case FK_ERR_ARG: return "invalid argument";
        case FK_ERR_UNSUPPORTED: return "unsupported dtype or shape";
        case FK_ERR_WORKSPACE: return "workspace too small or misaligned";
        case FK_ERR_CUDA: return "CUDA error";
        case FK_ERR_TIMEOUT: return "device-side wait timed out";
        default: return "unknown status";
    }
}

const char* fk_last_cuda_error(void) { return g_last_error; }

uint64_t fk_launch_count(void) { return __atomic_load_n(&g_launches, __ATOMIC_RELAXED); }

int fk_moe_layer_timed(const fk_moe_call* c, void* stream, float* stage_ms, int* stages) {
    return run_timed(stream, stage_ms, stages, [&] { return fk_moe_layer(c, stream); });
}

int fk_moe_experts_timed(const fk_moe_call* c, void* stream, float* stage_ms, int* stages) {
    return run_timed(stream, stage_ms, stages, [&] { stage_mark(); return fk_moe_experts(c, stream); });
}

int fk_moe_layer_ep_timed(const fk_moe_call* c, const fk_ep_comm* comm, void* stream, float* stage_ms, int* stages) {
    return run_timed(stream, stage_ms, stages, [&] { return fk_moe_layer_ep(c, comm, stream); });
}

int fk_set_wait_limit_cycles(long long cycles) {
    if (cycles < 0) return FK_ERR_ARG;
    __atomic_store_n(&g_wait_cycles, cycles == 0 ? kWaitCycles : cycles, __ATOMIC_RELAXED);
    return FK_OK;
}

int fk_moe_status(void* workspace, size_t workspace_bytes, int* code) {
    Workspace w = workspace_layout(fk_moe_dims{0, 1, 1, 1, 0});
    if (workspace == nullptr || workspace_bytes < w.meta + 16 * sizeof(int)) return FK_ERR_ARG;
    int* word = at<int>(workspace, w.meta) + 2;
    int v = 0;
    FK_CUDA_OK(cudaDeviceSynchronize(), "status sync");
    FK_CUDA_OK(cudaMemcpy(&v, word, sizeof(int), cudaMemcpyDeviceToHost), "status read");
    if (code) *code = v;
    if (v == 0) return FK_OK;
    FK_CUDA_OK(cudaMemset(word, 0, sizeof(int)), "status clear");
    return FK_ERR_TIMEOUT;
}

size_t fk_moe_trace_offset(const fk_moe_dims* dims) {
    if (dims == nullptr || !dims_ok(*dims, false)) return 0;
    return workspace_layout(*dims).y;
}

size_t fk_moe_workspace_bytes(const fk_moe_dims* dims) {
    if (dims == nullptr || !dims_ok(*dims, false)) return 0;
    return workspace_layout(*dims).total;
}

int fk_moe_workspace_init(void* workspace, size_t bytes, void* stream) {
    if (workspace == nullptr) return FK_ERR_ARG;
    // only the self-resetting words need a defined start value; they sit at the front
    Workspace w = workspace_layout(fk_moe_dims{0, 1, 1, 1, 0});
    size_t head = w.ids32;
    if (bytes < head) return FK_ERR_WORKSPACE;
    FK_CUDA_OK(cudaMemsetAsync(workspace, 0, head, (cudaStream_t)stream), "workspace init");
    return FK_OK;
}

int fk_moe_router(const fk_moe_call* c, void* stream) {
    if (c == nullptr || !dims_ok(c->dims, true) || c->dims.top_k > c->dims.experts) return FK_ERR_ARG;
    if (!dtype_ok(c->hidden_dtype) || !dtype_ok(c->weight_dtype)) return FK_ERR_UNSUPPORTED;
    if (c->dims.tokens == 0) return FK_OK;
    if (!c->hidden || !c->norm_weight || !c->router_weight || !c->logits || !c->topk_ids || !c->topk_weights) return FK_ERR_ARG;
    Workspace w;
    int st = check_workspace(c, w);
    if (st != FK_OK) return st;
    RouterParams rp{};
    rp.hidden = c->hidden; rp.hidden_dtype = c->hidden_dtype;
    rp.norm_weight = c->norm_weight; rp.router_weight = c->router_weight; rp.router_bias = c->router_bias;
    rp.shared_gate_weight = nullptr; rp.shared_gate_out = nullptr;
    rp.logits = c->logits; rp.topk_ids = reinterpret_cast<long long*>(c->topk_ids); rp.topk_weights = c->topk_weights;
    rp.ids32 = nullptr;
    rp.tickets = at<unsigned>(c->workspace, w.tickets);
    rp.T = c->dims.tokens; rp.H = c->dims.hidden; rp.E = c->dims.experts; rp.top_k = c->dims.top_k;
    rp.eps = c->eps; rp.norm_offset = c->norm_offset;
    return launch_router(rp, c->weight_dtype, (cudaStream_t)stream);
}

int fk_moe_router_noalloc(const fk_moe_call* c, void* stream) {
    if (c == nullptr || !dims_ok(c->dims, true) || c->dims.top_k > c->dims.experts) return FK_ERR_ARG;
    if (!dtype_ok(c->hidden_dtype) || !dtype_ok(c->weight_dtype)) return FK_ERR_UNSUPPORTED;
    if (c->dims.tokens > FK_NOALLOC_MAX_TOKENS) {
        snprintf(g_last_error, sizeof(g_last_error), "fk_moe_router_noalloc: %d tokens exceed the built-in scratch (max %d)",
                 c->dims.tokens, FK_NOALLOC_MAX_TOKENS);
        return FK_ERR_ARG;
    }
    if (c->dims.tokens == 0) return FK_OK;
    if (!c->hidden || !c->norm_weight || !c->router_weight || !c->logits || !c->topk_ids || !c->topk_weights) return FK_ERR_ARG;
    RouterParams rp{};
    rp.hidden = c->hidden; rp.hidden_dtype = c->hidden_dtype;
    rp.norm_weight = c->norm_weight; rp.router_weight = c->router_weight; rp.router_bias = c->router_bias;
    rp.logits = c->logits; rp.topk_ids = reinterpret_cast<long long*>(c->topk_ids); rp.topk_weights = c->topk_weights;
    rp.T = c->dims.tokens; rp.H = c->dims.hidden; rp.E = c->dims.experts; rp.top_k = c->dims.top_k;
    rp.eps = c->eps; rp.norm_offset = c->norm_offset;
    return launch_router_noalloc(rp, c->weight_dtype, (cudaStream_t)stream);
}

int fk_moe_experts(const fk_moe_call* c, void* stream) {
    if (c == nullptr || !dims_ok(c->dims, false)) return FK_ERR_ARG;
    if (!dtype_ok(c->hidden_dtype) || !dtype_ok(c->weight_dtype)) return FK_ERR_UNSUPPORTED;
    if (c->dims.tokens == 0) return FK_OK;
    if (!c->hidden || !c->out) return FK_ERR_ARG;
    if (c->dims.top_k > 0 && (!c->topk_ids_in || !c->topk_weights_in || !c->expert_gate_up || !c->expert_down)) return FK_ERR_ARG;
    if ((c->shared_gate_up == nullptr) != (c->shared_down == nullptr)) return FK_ERR_ARG;
    Workspace w;
    int st = check_workspace(c, w);
    if (st != FK_OK) return st;
    cudaStream_t s = (cudaStream_t)stream;
    const float* gate_sig = nullptr;
    if (c->shared_gate_up && c->shared_gate) {
        float* g = at<float>(c->workspace, w.shared_gate);
        int warps_per_block = 8;
        int blocks = (c->dims.tokens + warps_per_block - 1) / warps_per_block;
        shared_gate_kernel<<<blocks, warps_per_block * 32, 0, s>>>(c->hidden, c->hidden_dtype, c->shared_gate, c->weight_dtype, g,
                                                                  c->dims.tokens, c->dims.hidden);
        FK_LAUNCH_OK("shared gate launch");
        gate_sig = g;
    }
    return run_experts(c, w, reinterpret_cast<const long long*>(c->topk_ids_in), c->topk_weights_in, gate_sig, s);
}

// What the public layer entry points add to a plain fk_moe_layer call.
struct LayerExtras {
    long long* ids_mirror = nullptr;       // fk_moe_layer_host: the caller's pinned ids / weights buffers, written by the
    float* weights_mirror = nullptr;       // routing kernels as a second copy
    const float* resid_in = nullptr;       // fk_moe_layer_residual: the residual stream handed to the single-token kernel
    const float* update_in = nullptr;
    float* resid_out = nullptr;
    float resid_eps = 0.f;
};

static int moe_layer_impl(const fk_moe_call* c, void* stream, const LayerExtras& x);

int fk_moe_layer(const fk_moe_call* c, void* stream) { return moe_layer_impl(c, stream, LayerExtras{}); }

static int moe_layer_impl(const fk_moe_call* c, void* stream, const LayerExtras& x) {
    if (c == nullptr || !dims_ok(c->dims, true) || c->dims.top_k > c->dims.experts) return FK_ERR_ARG;
    if (!dtype_ok(c->hidden_dtype) || !dtype_ok(c->weight_dtype)) return FK_ERR_UNSUPPORTED;
    if (c->dims.tokens == 0) return FK_OK;
    if (!c->hidden || !c->norm_weight || !c->router_weight || !c->expert_gate_up || !c->expert_down || !c->out ||
        !c->logits || !c->topk_ids || !c->topk_weights)
        return FK_ERR_ARG;
    if ((c->shared_gate_up == nullptr) != (c->shared_down == nullptr)) return FK_ERR_ARG;
    Workspace w;
    int st = check_workspace(c, w);
    if (st != FK_OK) return st;
    cudaStream_t s = (cudaStream_t)stream;
    const bool gated = c->shared_gate_up && c->shared_gate;
    RouterParams rp{};
    rp.hidden = c->hidden; rp.hidden_dtype = c->hidden_dtype;
    rp.norm_weight = c->norm_weight; rp.router_weight = c->router_weight; rp.router_bias = c->router_bias;
    rp.shared_gate_weight = gated ? c->shared_gate : nullptr;
    rp.shared_gate_out = gated ? at<float>(c->workspace, w.shared_gate) : nullptr;
    rp.logits = c->logits; rp.topk_ids = reinterpret_cast<long long*>(c->topk_ids); rp.topk_weights = c->topk_weights;
    rp.ids32 = nullptr;
    rp.ids_mirror = x.ids_mirror; rp.weights_mirror = x.weights_mirror;
    rp.tickets = at<unsigned>(c->workspace, w.tickets);
    rp.T = c->dims.tokens; rp.H = c->dims.hidden; rp.E = c->dims.experts; rp.top_k = c->dims.top_k;
    rp.eps = c->eps; rp.norm_offset = c->norm_offset;
    stage_mark();   // start
    if (c->dims.tokens <= 4 && !(c->flags & (FK_FLAG_NO_FUSED_DECODE | FK_FLAG_FORCE_GENERIC)) &&
        (c->dims.tokens == 1 || x.resid_in == nullptr)) {
        DecodeParams dp{};
        dp.hidden = c->hidden; dp.hidden_dtype = c->hidden_dtype;
        dp.norm_weight = c->norm_weight; dp.router_weight = c->router_weight; dp.router_bias = c->router_bias;
        dp.gate_up = c->expert_gate_up; dp.down = c->expert_down;
        dp.shared_gate_up = c->shared_gate_up; dp.shared_down = c->shared_gate_up ? c->shared_down : nullptr;
        dp.shared_gate = gated ? c->shared_gate : nullptr;
        dp.logits = c->logits; dp.topk_ids = reinterpret_cast<long long*>(c->topk_ids); dp.topk_weights = c->topk_weights;
        dp.out = c->out; dp.layer_hidden = c->layer_hidden;
        dp.ids_mirror = x.ids_mirror; dp.weights_mirror = x.weights_mirror;
        dp.resid_in = x.resid_in; dp.update_in = x.update_in; dp.resid_out = x.resid_out; dp.resid_eps = x.resid_eps;
        dp.bar = at<unsigned>(c->workspace, w.counters);
        dp.tagged = at<unsigned long long>(c->workspace, w.tagged);
        dp.actw = dp.tagged + FK_MAX_EXPERTS;
        dp.wait_cycles = wait_limit_cycles();
        dp.error_word = at<int>(c->workspace, w.meta) + 2;
        // the trace record is 256 bytes per block at the start of the y region: dropped when it does not fit there
        const bool trace_fits = (size_t)sm_count() * 256 <= w.xg - w.y;
        dp.trace = ((c->flags & FK_FLAG_TRACE) && trace_fits) ? at<unsigned long long>(c->workspace, w.y) : nullptr;
        dp.H = c->dims.hidden; dp.E = c->dims.experts; dp.I = c->dims.intermediate; dp.top_k = c->dims.top_k;
        dp.T = c->dims.tokens;
        // the few-token kernel's activation rows: in the y region (unused on this path), behind the trace record
        dp.act_rows = (w.xg - w.y >= (size_t)65536 + 36 * 1024 * 2) ? at<uint32_t>(c->workspace, w.y) + 16384 : nullptr;
        dp.eps = c->eps; dp.norm_offset = c->norm_offset;
        if (dp.T == 1 && decode1_supported(dp, c->weight_dtype)) {
            st = launch_decode1(dp, s);
            stage_mark();   // end of the fused kernel
            return st;
        }
        if (dp.T > 1 && decode_few_supported(dp, c->weight_dtype)) {
            st = launch_decode_few(dp, s);
            stage_mark();   // end of the fused kernel
            return st;
        }
    }
    if (x.resid_in) return FK_ERR_UNSUPPORTED;      // the residual form exists for the single-token kernel only
    st = launch_router(rp, c->weight_dtype, s);
    if (st != FK_OK) return st;
    stage_mark();   // end of router
    return run_experts(c, w, rp.topk_ids, c->topk_weights, rp.shared_gate_out, s);
}

int fk_moe_layer_residual(const fk_moe_call* c, const float* resid_in, const float* update_in, float* resid_out,
                          float norm_eps, void* stream) {
    if (c == nullptr || resid_in == nullptr || resid_out == nullptr || resid_out == resid_in) return FK_ERR_ARG;
    if (c->dims.tokens != 1) return FK_ERR_UNSUPPORTED;
    LayerExtras x;
    x.resid_in = resid_in; x.update_in = update_in; x.resid_out = resid_out; x.resid_eps = norm_eps;
    fk_moe_call call = *c;
    if (call.hidden == nullptr) call.hidden = resid_in;       // not read in this form; keeps the argument check simple
    call.layer_hidden = nullptr;
    return moe_layer_impl(&call, stream, x);
}

size_t fk_moe_host_staging_bytes(const fk_moe_dims* d, int hidden_dtype) {
    if (d == nullptr || !dims_ok(*d, true) || !dtype_ok(hidden_dtype)) return 0;
    size_t T = d->tokens, H = d->hidden, E = d->experts, k = d->top_k;
    size_t es = hidden_dtype == FK_F32 ? 4 : 2;
    return align256(T * H * es) + 2 * align256(T * H * 4) + align256(T * E * 4) + align256(T * k * 8) + align256(T * k * 4);
}

// Device-side alias of a pinned (page-locked, mapped) host buffer, or null for pageable memory.
static void* mapped_alias(void* host) {
    if (host == nullptr) return nullptr;
    cudaPointerAttributes attr{};
    if (cudaPointerGetAttributes(&attr, host) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    return attr.type == cudaMemoryTypeHost ? attr.devicePointer : nullptr;
}

int fk_moe_layer_host(const fk_moe_call* c, void* staging, size_t staging_bytes, void* stream) {
    if (c == nullptr || staging == nullptr) return FK_ERR_ARG;
    size_t need = fk_moe_host_staging_bytes(&c->dims, c->hidden_dtype);
    if (need == 0) return FK_ERR_ARG;
    if (staging_bytes < need || (reinterpret_cast<uintptr_t>(staging) & 255)) return FK_ERR_WORKSPACE;
    if (c->dims.tokens == 0) return FK_OK;
    if (!c->hidden || !c->out) return FK_ERR_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    size_t T = c->dims.tokens, H = c->dims.hidden, E = c->dims.experts, k = c->dims.top_k;
    size_t es = c->hidden_dtype == FK_F32 ? 4 : 2;
    size_t o = 0;
    auto take = [&](size_t bytes) { void* p = reinterpret_cast<char*>(staging) + o; o += align256(bytes); return p; };
    void* d_hidden = take(T * H * es);
    float* d_out = (float*)take(T * H * 4);
    float* d_layer = (float*)take(T * H * 4);
    float* d_logits = (float*)take(T * E * 4);
    int64_t* d_ids = (int64_t*)take(T * k * 8);
    float* d_w = (float*)take(T * k * 4);
    FK_CUDA_OK(cudaMemcpyAsync(d_hidden, c->hidden, T * H * es, cudaMemcpyHostToDevice, s), "h2d hidden");
    fk_moe_call dev = *c;
    // The output rows are written once, by the last kernel, and read by none: when the caller's buffers are pinned
    // the kernel stores them straight into host memory and the copy back (and its place in the stream) is saved.
    float* out_alias = (float*)mapped_alias(c->out);
    float* layer_alias = (float*)mapped_alias(c->layer_hidden);
    dev.hidden = d_hidden; dev.out = out_alias ? out_alias : d_out;
    dev.layer_hidden = c->layer_hidden ? (layer_alias ? layer_alias : d_layer) : nullptr;
    dev.logits = d_logits; dev.topk_ids = d_ids; dev.topk_weights = d_w;
    // ids and weights are small: when the caller's buffers are pinned, the routing kernel writes a second copy there
    long long* ids_alias = (long long*)mapped_alias(c->topk_ids);
    float* w_alias = (float*)mapped_alias(c->topk_weights);
    LayerExtras x;
    x.ids_mirror = ids_alias;
    x.weights_mirror = w_alias;
    int st = moe_layer_impl(&dev, stream, x);
    if (st != FK_OK) return st;
    if (!out_alias) FK_CUDA_OK(cudaMemcpyAsync(c->out, d_out, T * H * 4, cudaMemcpyDeviceToHost, s), "d2h out");
    if (c->layer_hidden && !layer_alias)
        FK_CUDA_OK(cudaMemcpyAsync(c->layer_hidden, d_layer, T * H * 4, cudaMemcpyDeviceToHost, s), "d2h layer");
    if (c->logits) FK_CUDA_OK(cudaMemcpyAsync(c->logits, d_logits, T * E * 4, cudaMemcpyDeviceToHost, s), "d2h logits");
    if (c->topk_ids && !ids_alias) FK_CUDA_OK(cudaMemcpyAsync(c->topk_ids, d_ids, T * k * 8, cudaMemcpyDeviceToHost, s), "d2h ids");
    if (c->topk_weights && !w_alias)
        FK_CUDA_OK(cudaMemcpyAsync(c->topk_weights, d_w, T * k * 4, cudaMemcpyDeviceToHost, s), "d2h weights");
    return FK_OK;
}

// ---------------------------------------------------------------------------------------------
// Expert parallel over peer memory
// ---------------------------------------------------------------------------------------------
size_t fk_ep_buffer_bytes(int world, int tokens_per_rank, int hidden, int top_k, int hidden_dtype) {
    if (world < 1 || world > FK_EP_MAX_RANKS || tokens_per_rank < 1 || hidden < 1 || hidden > FK_MAX_HIDDEN || top_k < 1 ||
        top_k > FK_MAX_TOP_K || !dtype_ok(hidden_dtype))
        return 0;
    return ep_layout(world, tokens_per_rank, hidden, top_k, hidden_dtype).total;
}

int fk_ep_buffer_create(size_t bytes, void** buffer, void* handle_out) {
    if (bytes < 256 || buffer == nullptr || handle_out == nullptr) return FK_ERR_ARG;
    static_assert(sizeof(cudaIpcMemHandle_t) <= FK_EP_HANDLE_BYTES, "IPC handle does not fit");
    void* ptr = nullptr;
    FK_CUDA_OK(cudaMalloc(&ptr, bytes), "ep buffer alloc");
    FK_CUDA_OK(cudaMemset(ptr, 0, bytes), "ep buffer clear");
    cudaIpcMemHandle_t h;
    FK_CUDA_OK(cudaIpcGetMemHandle(&h, ptr), "ep buffer handle");
    memset(handle_out, 0, FK_EP_HANDLE_BYTES);
    memcpy(handle_out, &h, sizeof(h));
    FK_CUDA_OK(cudaDeviceSynchronize(), "ep buffer sync");
    *buffer = ptr;
    return FK_OK;
}

int fk_ep_buffer_open(const void* handle, void** buffer) {
    if (handle == nullptr || buffer == nullptr) return FK_ERR_ARG;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* ptr = nullptr;
    FK_CUDA_OK(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess), "ep buffer open");
    *buffer = ptr;
    return FK_OK;
}

int fk_ep_buffer_close(void* buffer) {
    if (buffer == nullptr) return FK_OK;
    FK_CUDA_OK(cudaIpcCloseMemHandle(buffer), "ep buffer close");
    return FK_OK;
}

int fk_ep_buffer_destroy(void* buffer) {
    if (buffer == nullptr) return FK_OK;
    FK_CUDA_OK(cudaFree(buffer), "ep buffer free");
    return FK_OK;
}

int fk_ep_buffer_reset(void* buffer) {
    if (buffer == nullptr) return FK_ERR_ARG;
    FK_CUDA_OK(cudaDeviceSynchronize(), "ep buffer reset sync");
    FK_CUDA_OK(cudaMemset(buffer, 0, 256), "ep buffer reset");     // the header: epochs, tickets, error word
    FK_CUDA_OK(cudaDeviceSynchronize(), "ep buffer reset sync");
    return FK_OK;
}

int fk_ep_status(const fk_ep_comm* comm, int* error) {
    if (comm == nullptr || error == nullptr || comm->rank < 0 || comm->rank >= FK_EP_MAX_RANKS || !comm->base[comm->rank]) return FK_ERR_ARG;
    FK_CUDA_OK(cudaDeviceSynchronize(), "ep status sync");
    FK_CUDA_OK(cudaMemcpy(error, reinterpret_cast<const char*>(comm->base[comm->rank]) + 20 * 4, sizeof(int), cudaMemcpyDeviceToHost),
               "ep status read");
    return FK_OK;
}

int fk_moe_layer_ep(const fk_moe_call* c, const fk_ep_comm* comm, void* stream) {
    if (c == nullptr || comm == nullptr || !dims_ok(c->dims, true) || c->dims.top_k > c->dims.experts) return FK_ERR_ARG;
    if (!dtype_ok(c->hidden_dtype) || !dtype_ok(c->weight_dtype)) return FK_ERR_UNSUPPORTED;
    const int G = comm->world, rank = comm->rank, T = c->dims.tokens, H = c->dims.hidden, k = c->dims.top_k;
    if (G < 1 || G > FK_EP_MAX_RANKS || rank < 0 || rank >= G || T != comm->tokens_per_rank || T < 1) return FK_ERR_ARG;
    if (c->dims.experts % G != 0 || H % 8 != 0) return FK_ERR_ARG;
    if (!c->hidden || !c->norm_weight || !c->router_weight || !c->expert_gate_up || !c->expert_down || !c->out || !c->logits ||
        !c->topk_ids || !c->topk_weights)
        return FK_ERR_ARG;
    if ((c->shared_gate_up == nullptr) != (c->shared_down == nullptr)) return FK_ERR_ARG;
    const EpLayout lay = ep_layout(G, T, H, k, c->hidden_dtype);
    if (comm->bytes < lay.total) return FK_ERR_WORKSPACE;
    for (int r = 0; r < G; ++r)
        if (comm->base[r] == nullptr) return FK_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(c->hidden) | reinterpret_cast<uintptr_t>(c->out) | reinterpret_cast<uintptr_t>(c->layer_hidden)) & 15)
        return FK_ERR_ARG;
    const int e_local = c->dims.experts / G;
    // the gathered call: all ranks' tokens, this rank's experts
    fk_moe_call all = *c;
    all.dims.tokens = G * T;
    all.dims.experts = e_local;
    Workspace w_all;
    int st = check_workspace(&all, w_all);
    if (st != FK_OK) return st;
    Workspace w_own = workspace_layout(c->dims);
    if (c->workspace_bytes < w_own.total) return FK_ERR_WORKSPACE;
    cudaStream_t s = (cudaStream_t)stream;
    const bool gated = c->shared_gate_up && c->shared_gate;
    unsigned char* mine = reinterpret_cast<unsigned char*>(comm->base[rank]);

    // 1. router on the rank's own tokens; the shared gate lands where the gathered call looks for it
    RouterParams rp{};
    rp.hidden = c->hidden; rp.hidden_dtype = c->hidden_dtype;
    rp.norm_weight = c->norm_weight; rp.router_weight = c->router_weight; rp.router_bias = c->router_bias;
    rp.shared_gate_weight = gated ? c->shared_gate : nullptr;
    rp.shared_gate_out = gated ? at<float>(c->workspace, w_all.shared_gate) + (size_t)rank * T : nullptr;
    rp.logits = c->logits; rp.topk_ids = reinterpret_cast<long long*>(c->topk_ids); rp.topk_weights = c->topk_weights;
    rp.ids32 = nullptr;
    rp.tickets = at<unsigned>(c->workspace, w_all.tickets);
    rp.T = T; rp.H = H; rp.E = c->dims.experts; rp.top_k = k;
    rp.eps = c->eps; rp.norm_offset = c->norm_offset;
    stage_mark();   // start
    st = launch_router(rp, c->weight_dtype, s);
    if (st != FK_OK) return st;
    stage_mark();   // end of router

    // 2. dispatch: own rows into every rank's buffer, flags, wait for everyone's rows
    EpPeers peers{};
    for (int r = 0; r < G; ++r) peers.header[r] = reinterpret_cast<unsigned*>(comm->base[r]);
    peers.partial_offset = lay.partial;
    peers.world = G; peers.rank = rank; peers.tokens = T;
    peers.wait_cycles = wait_limit_cycles();
    EpDispatchParams dp{};
    dp.peers = peers; dp.layout = lay;
    dp.hidden = c->hidden; dp.ids = rp.topk_ids; dp.weights = c->topk_weights;
    dp.T = T; dp.H = H; dp.top_k = k; dp.elem_bytes = c->hidden_dtype == FK_F32 ? 4 : 2;
    st = launch_ep_dispatch(dp, s);
    if (st != FK_OK) return st;
    stage_mark();   // end of dispatch (stores, flags, wait for every rank's rows)

    // 3. local experts on the gathered tokens (+ shared expert on the own ones); rows go to the home ranks
    all.hidden = mine + lay.hidden;
    all.flags = c->flags | FK_FLAG_SKIP_FOREIGN;
    all.expert_base = rank * e_local;
    all.shared_token_base = rank * T;
    all.shared_token_count = T;
    all.out = reinterpret_cast<float*>(mine + lay.partial);     // not written: the combine stores to the peers
    all.layer_hidden = nullptr;
    st = run_experts(&all, w_all, nullptr, reinterpret_cast<const float*>(mine + lay.weights),
                     gated ? at<float>(c->workspace, w_all.shared_gate) : nullptr, s,
                     reinterpret_cast<const int*>(mine + lay.ids), &peers, (int)((long long)G * T * k / c->dims.experts));
    if (st != FK_OK) return st;

    // 4. fixed-order sum of the world partials for the own tokens
    st = launch_ep_reduce(reinterpret_cast<const float*>(mine + lay.partial), G, rank, T, H, rp.topk_ids, k, e_local,
                          c->shared_gate_up != nullptr ? 1 : 0, c->out, c->layer_hidden, c->hidden, c->hidden_dtype, s);
    stage_mark();   // end of reduce
    return st;
}

int fk_single_expert_mlp(const void* hidden, int hidden_dtype, const void* gate_up, const void* down, int weight_dtype,
                         float* out, int hidden_size, int intermediate, void* workspace, size_t workspace_bytes,
                         void* stream) {
    // one token through one expert == a layer with no routed experts whose "shared expert" is this expert
    fk_moe_call c{};
    c.dims = fk_moe_dims{1, hidden_size, 1, intermediate, 0};
    c.hidden_dtype = hidden_dtype;
    c.weight_dtype = weight_dtype;
    c.hidden = hidden;
    c.shared_gate_up = gate_up;
    c.shared_down = down;
    c.out = out;
    c.workspace = workspace;
    c.workspace_bytes = workspace_bytes;
    if (!gate_up || !down) return FK_ERR_ARG;
    return fk_moe_experts(&c, stream);
}

int fk_residual_rmsnorm(float* x, const float* update, void* normed, int out_dtype, int tokens, int hidden_size, float eps,
                        void* stream) {
    if (!dtype_ok(out_dtype)) return FK_ERR_UNSUPPORTED;
    if (tokens < 0 || hidden_size < 1) return FK_ERR_ARG;
    if (tokens > 0 && (!x || !normed)) return FK_ERR_ARG;
    return launch_residual_norm(x, update, normed, out_dtype, tokens, hidden_size, eps, (cudaStream_t)stream);
}

int fk_fused_swiglu(const void* gate_up, void* out, int dtype, int64_t rows, int intermediate, void* stream) {
    if (!dtype_ok(dtype)) return FK_ERR_UNSUPPORTED;
    if (rows > 0 && intermediate > 0 && (!gate_up || !out)) return FK_ERR_ARG;
    return launch_swiglu(gate_up, out, dtype, rows, intermediate, (cudaStream_t)stream);
}

int fk_expert_histogram(const void* ids, int ids_are_int64, int64_t count, int num_experts, int32_t* counts, void* stream) {
    if (!counts || (count > 0 && !ids)) return FK_ERR_ARG;
    return launch_histogram(ids, ids_are_int64, count, num_experts, counts, (cudaStream_t)stream);
}

int fk_moe_permute(const int64_t* topk_ids, int tokens, int top_k, int num_experts, int32_t* counts, int32_t* offsets,
                   int32_t* order, void* workspace, size_t workspace_bytes, void* stream) {
    (void)workspace; (void)workspace_bytes;
    if (!topk_ids || !counts || !offsets || !order || tokens < 0 || top_k < 1) return FK_ERR_ARG;
    PermuteParams pp{};
    pp.ids64 = reinterpret_cast<const long long*>(topk_ids);
    pp.routes = tokens * top_k;
    pp.E = num_experts;
    pp.skip_foreign = 1;
    pp.counts = counts; pp.offsets = offsets; pp.order = order;
    return launch_permute(pp, (cudaStream_t)stream);
}

}  // extern "C"
