"""GPU parity: every stage of the MoE decode layer against the CPU oracle, through the C ABI.

The stage list follows the reference's own CUDA tests (tests/test_triton_moe.py:57-681, :1112-1157):
swiglu, histogram, router (single/batched, fp32/bf16), single expert, routed, routed+shared, shared
gate, full MoE, layer residual, tiny fused block.  Inputs are seeded; real-shape cases use
H=2048, E=256, I=512, k=8 like the reference.
"""

from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import moe_oracle as O
from oracle.pin_against_reference import CASES, ROUTER_CASES
from fastkernels_b200 import _lib
from fastkernels_b200.kernels.triton import (
    triton_expert_histogram,
    triton_fused_swiglu,
    triton_qwen36_batched_moe_decode,
    triton_qwen36_batched_moe_layer_decode,
    triton_qwen36_batched_moe_router_decode,
    triton_qwen36_batched_routed_experts_decode,
    triton_qwen36_batched_routed_shared_experts_decode,
    triton_qwen36_moe_decode,
    triton_qwen36_moe_router_decode,
    triton_qwen36_routed_experts_decode,
    triton_qwen36_routed_shared_experts_decode,
    triton_qwen36_single_expert_mlp_decode,
    triton_synthetic_qwen36_moe_decode,
)
from fastkernels_b200.moe import expert_permutation
from fastkernels_b200.spec import MoESpec, MoEWeights
from fastkernels_b200.workloads import HOT_EXPERT_IDS, make_hidden, make_moe_weights
from tests.parity import check_output, check_output_where_ids_agree, check_routing, oracle_layer
from tests.tolerances import default_tolerance

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).parent / "golden"
REAL = MoESpec()
FIXED_IDS = list(HOT_EXPERT_IDS)


@pytest.fixture(scope="module")
def real_bf16():
    return make_moe_weights(0, REAL, dtype=torch.bfloat16, device="cuda")


@pytest.fixture(scope="module")
def real_bf16_biased():
    return make_moe_weights(1, REAL, dtype=torch.bfloat16, device="cuda", bias_std=0.5)


def _randn(*shape, dtype, seed=0, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (scale * torch.randn(*shape, generator=g, device="cuda", dtype=torch.float32)).to(dtype)


# ---------------------------------------------------------------- stand-alone ops
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
def test_fused_swiglu_matches_oracle(dtype):
    gate_up = _randn(128, 1024, dtype=dtype)
    cand = triton_fused_swiglu(gate_up)
    ref = O.fused_swiglu(gate_up.cpu().float()).to(dtype)
    assert cand.dtype == dtype and cand.shape == (128, 512)
    atol, rtol = default_tolerance(dtype)
    torch.testing.assert_close(cand.cpu(), ref, atol=atol, rtol=rtol)


@pytest.mark.parametrize("idtype", [torch.int32, torch.int64])
def test_expert_histogram_bit_exact(idtype):
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 256, (64, 8), generator=g, dtype=idtype)
    cand = triton_expert_histogram(ids.cuda(), 256)
    assert cand.dtype == torch.int32
    assert torch.equal(cand.cpu(), O.expert_histogram(ids, 256))


@pytest.mark.parametrize("tokens,experts", [(1, 256), (7, 5), (64, 256), (256, 256), (2048, 32), (300, 1024), (511, 256), (513, 64),
                                            (2048, 256), (5000, 1024)])
def test_expert_permutation_bit_exact(tokens, experts):
    g = torch.Generator().manual_seed(tokens)
    ids = torch.randint(0, experts, (tokens, 8), generator=g)
    if tokens == 256:
        ids[:200, 0] = 17          # one hot expert
    counts, offsets, order = expert_permutation(ids.cuda(), experts)
    rc, ro, rord = O.expert_permutation(ids, experts)
    assert torch.equal(counts.cpu(), rc) and torch.equal(offsets.cpu(), ro) and torch.equal(order.cpu(), rord)


# ---------------------------------------------------------------- router
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_router_single_token_real_shape(dtype):
    hidden = _randn(2048, dtype=dtype, seed=1)
    norm_w = _randn(2048, dtype=dtype, seed=2, scale=0.02)
    router_w = _randn(256, 2048, dtype=dtype, seed=3, scale=0.02)
    logits, ids, weights = triton_qwen36_moe_router_decode(hidden, norm_w, router_w, top_k=8)
    assert logits.shape == (256,) and ids.dtype == torch.int64 and weights.dtype == torch.float32
    rl, rid, rw = O.router(hidden.cpu().unsqueeze(0), norm_w.cpu(), router_w.cpu(), top_k=8)
    atol, rtol = default_tolerance(torch.float32)
    torch.testing.assert_close(logits.cpu(), rl[0], atol=atol, rtol=rtol)
    own_ids, own_w = O.route_from_logits(logits.cpu().unsqueeze(0), 8)
    assert torch.equal(ids.cpu(), own_ids[0])
    assert torch.equal(ids.cpu(), rid[0])
    torch.testing.assert_close(weights.cpu(), rw[0], atol=1e-5, rtol=1e-4)


@pytest.mark.parametrize("name", list(ROUTER_CASES))
def test_router_matches_reference_golden(name):
    tokens, dtype, seed = ROUTER_CASES[name]
    gold = np.load(GOLDEN / f"{name}.npz")
    g = torch.Generator().manual_seed(seed)
    hidden = torch.randn(tokens, 2048, generator=g).to(dtype)
    norm_w = (0.02 * torch.randn(2048, generator=g)).to(dtype)
    router_w = (0.02 * torch.randn(256, 2048, generator=g)).to(dtype)
    logits, ids, weights = triton_qwen36_batched_moe_router_decode(hidden.cuda(), norm_w.cuda(), router_w.cuda())
    np.testing.assert_allclose(logits.cpu().numpy(), gold["logits"], atol=1e-4, rtol=1e-4)
    clear = torch.from_numpy(gold["margin"]) > 2e-6
    assert torch.equal(ids.cpu()[clear], torch.from_numpy(gold["topk_ids"])[clear])
    np.testing.assert_allclose(weights.cpu().numpy()[clear.numpy()], gold["topk_weights"][clear.numpy()], atol=1e-5, rtol=1e-4)


@pytest.mark.parametrize("tokens", [4, 33, 256])
def test_router_batched_with_bias_and_offset(tokens):
    dtype = torch.bfloat16
    hidden = _randn(tokens, 2048, dtype=dtype, seed=4)
    norm_w = _randn(2048, dtype=dtype, seed=5, scale=0.02)
    router_w = _randn(256, 2048, dtype=dtype, seed=6, scale=0.02)
    bias = _randn(256, dtype=torch.float32, seed=7, scale=0.5)
    for off in (1.0, 0.0):
        nw = norm_w if off == 1.0 else (norm_w + 1).to(dtype)
        logits, ids, weights = triton_qwen36_batched_moe_router_decode(hidden, nw, router_w, norm_offset=off,
                                                                       router_bias=bias)
        rl, rid, rw = O.router(hidden.cpu(), nw.cpu(), router_w.cpu(), top_k=8, norm_offset=off, router_bias=bias.cpu())
        torch.testing.assert_close(logits.cpu(), rl, atol=1e-4, rtol=1e-4)
        own_ids, own_w = O.route_from_logits(logits.cpu(), 8)
        assert torch.equal(ids.cpu(), own_ids)
        torch.testing.assert_close(weights.cpu(), own_w, atol=1e-6, rtol=1e-5)


@pytest.mark.parametrize("top_k", [1, 2, 5, 8])
def test_router_exact_ties_go_to_lower_index(top_k):
    # identical router rows give bit-identical logits: groups {0,1,2,3} and {100..103} tie exactly
    dtype = torch.bfloat16
    hidden = _randn(3, 2048, dtype=dtype, seed=8)
    router_w = _randn(256, 2048, dtype=dtype, seed=9, scale=0.02)
    router_w[1:4] = router_w[0]
    router_w[101:104] = router_w[100]
    norm_w = torch.zeros(2048, device="cuda", dtype=dtype)
    bias = torch.zeros(256, device="cuda")
    bias[0:4] = 40.0
    bias[100:104] = 30.0
    logits, ids, weights = triton_qwen36_batched_moe_router_decode(hidden, norm_w, router_w, top_k=top_k, router_bias=bias)
    lc = logits.cpu()
    assert torch.equal(lc[:, 0], lc[:, 1]) and torch.equal(lc[:, 100], lc[:, 103])
    expect = [0, 1, 2, 3, 100, 101, 102, 103][:top_k]
    assert ids.cpu().tolist() == [expect] * 3
    own_ids, _ = O.route_from_logits(lc, top_k)
    assert torch.equal(ids.cpu(), own_ids)
    # all logits equal: the first k experts win
    z = torch.zeros(256, 2048, device="cuda", dtype=dtype)
    _, ids0, w0 = triton_qwen36_batched_moe_router_decode(hidden, norm_w, z, top_k=top_k)
    assert ids0.cpu().tolist() == [list(range(top_k))] * 3
    torch.testing.assert_close(w0.cpu(), torch.full((3, top_k), 1.0 / top_k))


def test_router_odd_shapes_and_many_experts():
    for (T, H, E, k, dtype) in [(3, 200, 24, 5, torch.float32), (2, 100, 1000, 8, torch.bfloat16), (5, 16, 4, 2, torch.float16)]:
        hidden = _randn(T, H, dtype=dtype, seed=10)
        norm_w = _randn(H, dtype=dtype, seed=11, scale=0.1)
        router_w = _randn(E, H, dtype=dtype, seed=12, scale=0.1)
        logits, ids, weights = triton_qwen36_batched_moe_router_decode(hidden, norm_w, router_w, top_k=k)
        rl, rid, rw = O.router(hidden.cpu(), norm_w.cpu(), router_w.cpu(), top_k=k)
        torch.testing.assert_close(logits.cpu(), rl, atol=1e-4, rtol=1e-4)
        own_ids, own_w = O.route_from_logits(logits.cpu(), k)
        assert torch.equal(ids.cpu(), own_ids)


@pytest.mark.parametrize("tokens", [1, 130, 300])
def test_router_widest_hidden_size(tokens):
    """H = 4096, the limit the header advertises: the bf16 fast path must pick a block size that fits its shared
    memory (32 tokens of 4096 columns do not)."""
    H, E = 4096, 256
    hidden = _randn(tokens, H, dtype=torch.bfloat16, seed=20)
    norm_w = _randn(H, dtype=torch.bfloat16, seed=21, scale=0.1)
    router_w = _randn(E, H, dtype=torch.bfloat16, seed=22, scale=0.02)
    logits, ids, weights = triton_qwen36_batched_moe_router_decode(hidden, norm_w, router_w, top_k=8)
    rl, rid, rw = O.router(hidden.cpu(), norm_w.cpu(), router_w.cpu(), top_k=8)
    torch.testing.assert_close(logits.cpu(), rl, atol=1e-4, rtol=1e-4)
    own_ids, own_w = O.route_from_logits(logits.cpu(), 8)
    assert torch.equal(ids.cpu(), own_ids)
    torch.testing.assert_close(weights.cpu(), own_w, atol=1e-6, rtol=1e-5)


def test_alternating_routings_on_one_workspace_never_see_a_stale_pass_list(real_bf16_biased):
    """Two batches with different routing alternate on one prepared call (one workspace, programmatic dependent
    launch on): the down kernel reads the pass list without waiting for the gate_up kernel, so a stale list or a
    y buffer overwritten too early would show up as a difference from the first results."""
    from fastkernels_b200.plan import MoEDecodePlan
    w = real_bf16_biased
    for tokens in (8, 32):
        plan = MoEDecodePlan(w, tokens)
        xs = [make_hidden(600 + i, tokens, REAL, dtype=torch.bfloat16, device="cuda") for i in range(2)]
        want = []
        for x in xs:
            out, _, ids, _ = plan.run(x)
            want.append((out.clone(), ids.clone()))
        assert not torch.equal(want[0][1], want[1][1])
        plan.capture()
        for rep in range(40):
            out, _, ids, _ = plan.run(xs[rep % 2])
            assert torch.equal(ids, want[rep % 2][1]) and torch.equal(out, want[rep % 2][0]), f"{tokens} tokens, repetition {rep}"


# ---------------------------------------------------------------- experts with fixed routing
def _fixed_routing(tokens):
    ids = torch.tensor([[(i + t) % 256 for i in FIXED_IDS] for t in range(tokens)], dtype=torch.int64)
    ids[:, -1] = torch.arange(255, 255 - tokens, -1)
    g = torch.Generator().manual_seed(3)
    w = torch.rand(tokens, 8, generator=g) + 0.1
    return ids.cuda(), (w / w.sum(-1, keepdim=True)).cuda()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_single_expert_mlp(dtype):
    hidden = _randn(2048, dtype=dtype, seed=1)
    gu = _randn(1024, 2048, dtype=dtype, seed=2, scale=0.02)
    dn = _randn(2048, 512, dtype=dtype, seed=3, scale=0.02)
    out = triton_qwen36_single_expert_mlp_decode(hidden, gu, dn)
    assert out.dtype == torch.float32 and out.shape == (2048,)
    ref = O.expert_mlp(hidden.cpu().unsqueeze(0), gu.cpu(), dn.cpu())[0]
    check_output(out, ref, dtype)


@pytest.mark.parametrize("shared,gated", [(False, False), (True, False), (True, True)])
def test_routed_experts_single_token_fixed_ids(real_bf16, shared, gated):
    w = real_bf16
    hidden = _randn(2048, dtype=torch.bfloat16, seed=5)
    ids, wts = _fixed_routing(1)
    if shared:
        out = triton_qwen36_routed_shared_experts_decode(hidden, ids[0], wts[0], w.expert_gate_up_weight, w.expert_down_weight,
                                                         w.shared_gate_up_weight, w.shared_down_weight,
                                                         w.shared_expert_gate_weight if gated else None)
    else:
        out = triton_qwen36_routed_experts_decode(hidden, ids[0], wts[0], w.expert_gate_up_weight, w.expert_down_weight)
    sel = ids[0].cpu()
    ref = O.routed_experts(hidden.cpu().unsqueeze(0), torch.arange(8).unsqueeze(0), wts.cpu(),
                           w.expert_gate_up_weight[sel.cuda()].cpu(), w.expert_down_weight[sel.cuda()].cpu())
    if shared:
        ref = ref + O.shared_expert(hidden.cpu().unsqueeze(0), w.shared_gate_up_weight.cpu(), w.shared_down_weight.cpu(),
                                    w.shared_expert_gate_weight.cpu() if gated else None)
    check_output(out, ref[0], torch.bfloat16)


@pytest.mark.parametrize("tokens", [2, 4, 19])
@pytest.mark.parametrize("shared,gated", [(False, False), (True, True)])
def test_routed_experts_batched_fixed_ids(real_bf16, tokens, shared, gated):
    w = real_bf16
    hidden = _randn(tokens, 2048, dtype=torch.bfloat16, seed=6)
    ids, wts = _fixed_routing(tokens)
    if shared:
        out = triton_qwen36_batched_routed_shared_experts_decode(hidden, ids, wts, w.expert_gate_up_weight, w.expert_down_weight,
                                                                 w.shared_gate_up_weight, w.shared_down_weight,
                                                                 w.shared_expert_gate_weight if gated else None)
    else:
        out = triton_qwen36_batched_routed_experts_decode(hidden, ids, wts, w.expert_gate_up_weight, w.expert_down_weight)
    uniq, local = torch.unique(ids.cpu(), return_inverse=True)
    ref = O.routed_experts(hidden.cpu(), local, wts.cpu(), w.expert_gate_up_weight[uniq.cuda()].cpu(),
                           w.expert_down_weight[uniq.cuda()].cpu())
    if shared:
        ref = ref + O.shared_expert(hidden.cpu(), w.shared_gate_up_weight.cpu(), w.shared_down_weight.cpu(),
                                    w.shared_expert_gate_weight.cpu() if gated else None)
    check_output(out, ref, torch.bfloat16)


def test_out_of_range_ids_are_clamped(real_bf16):
    w = real_bf16
    hidden = _randn(2, 2048, dtype=torch.bfloat16, seed=7)
    ids, wts = _fixed_routing(2)
    bad = ids.clone()
    bad[0, 0] = 999
    bad[1, 1] = -5
    fixed = ids.clone()
    fixed[0, 0] = 255
    fixed[1, 1] = 0
    a = triton_qwen36_batched_routed_experts_decode(hidden, bad, wts, w.expert_gate_up_weight, w.expert_down_weight)
    b = triton_qwen36_batched_routed_experts_decode(hidden, fixed, wts, w.expert_gate_up_weight, w.expert_down_weight)
    assert torch.equal(a, b)


# ---------------------------------------------------------------- whole layer
@pytest.mark.parametrize("tokens", [1, 4, 16, 32])
def test_full_layer_bf16_real_shape(real_bf16_biased, tokens):
    w = real_bf16_biased
    hidden = make_hidden(100 + tokens, tokens, REAL, dtype=torch.bfloat16, device="cuda")
    out, logits, ids, weights = triton_qwen36_batched_moe_decode(hidden, *w.tuple(), top_k=8, router_bias=w.router_bias)
    ref = oracle_layer(hidden, w, 8)
    check_routing(logits, ids, weights, ref, torch.bfloat16)
    check_output_where_ids_agree(out, ids, ref.topk_ids, ref.output, torch.bfloat16, what=f"layer, {tokens} tokens")
    hist = triton_expert_histogram(ids, 256)
    assert torch.equal(hist.cpu(), O.expert_histogram(ids.cpu(), 256))
    # bitwise run-to-run determinism
    out2, _, ids2, _ = triton_qwen36_batched_moe_decode(hidden, *w.tuple(), top_k=8, router_bias=w.router_bias)
    assert torch.equal(out, out2) and torch.equal(ids, ids2)


def test_full_layer_single_token_api(real_bf16):
    w = real_bf16
    hidden = make_hidden(7, 1, REAL, dtype=torch.bfloat16, device="cuda")[0]
    out, logits, ids, weights = triton_qwen36_moe_decode(hidden, *w.tuple())
    assert out.shape == (2048,) and logits.shape == (256,) and ids.shape == (8,)
    ref = oracle_layer(hidden.unsqueeze(0), w, 8)
    check_routing(logits.unsqueeze(0), ids.unsqueeze(0), weights.unsqueeze(0), ref, torch.bfloat16)
    check_output(out, ref.output[0], torch.bfloat16)
    # ungated shared expert
    out_u, _, _, _ = triton_qwen36_moe_decode(hidden, *w.tuple()[:6], None)
    w_u = MoEWeights(*w.tuple()[:6], None)
    check_output(out_u, oracle_layer(hidden.unsqueeze(0), w_u, 8).output[0], torch.bfloat16)


@pytest.mark.parametrize("flags", [_lib.FLAG_FORCE_GENERIC, _lib.FLAG_FORCE_GEMV | _lib.FLAG_NO_FUSED_DECODE])
def test_full_layer_generic_kernels_agree(real_bf16, flags):
    w = real_bf16
    hidden = make_hidden(9, 3, REAL, dtype=torch.bfloat16, device="cuda")
    fast, _, ids_f, _ = triton_qwen36_batched_moe_decode(hidden, *w.tuple(), flags=_lib.FLAG_NO_FUSED_DECODE)
    slow, _, ids_s, _ = triton_qwen36_batched_moe_decode(hidden, *w.tuple(), flags=flags)
    assert torch.equal(ids_f, ids_s)
    torch.testing.assert_close(fast, slow, atol=2e-5, rtol=1e-4)


@pytest.mark.parametrize("gated,bias", [(True, True), (False, False)])
def test_single_token_fused_kernel_matches_staged_path_and_oracle(real_bf16_biased, gated, bias):
    w = real_bf16_biased
    args = list(w.tuple())
    if not gated:
        args[6] = None
    rb = w.router_bias if bias else None
    for seed in range(4):
        hidden = make_hidden(300 + seed, 1, REAL, dtype=torch.bfloat16, device="cuda")
        fused = triton_qwen36_batched_moe_layer_decode(hidden, *args, router_bias=rb)
        staged = triton_qwen36_batched_moe_layer_decode(hidden, *args, router_bias=rb, flags=_lib.FLAG_NO_FUSED_DECODE)
        assert torch.equal(fused[3], staged[3])                       # ids
        torch.testing.assert_close(fused[2], staged[2], atol=1e-5, rtol=1e-5)   # logits
        torch.testing.assert_close(fused[4], staged[4], atol=1e-6, rtol=1e-5)   # weights
        torch.testing.assert_close(fused[1], staged[1], atol=2e-5, rtol=1e-4)   # update
        torch.testing.assert_close(fused[0], hidden.float() + fused[1], atol=0, rtol=0)
        ref = oracle_layer(hidden, MoEWeights(*args, rb), 8)
        check_routing(fused[2], fused[3], fused[4], ref, torch.bfloat16)
        check_output(fused[1], ref.output, torch.bfloat16)
        again = triton_qwen36_batched_moe_layer_decode(hidden, *args, router_bias=rb)
        assert torch.equal(again[1], fused[1])                        # bitwise repeatable


@pytest.mark.parametrize("tokens", [2, 3, 4])
@pytest.mark.parametrize("gated,bias", [(True, True), (False, False)])
def test_few_token_fused_kernel_matches_staged_path_and_oracle(real_bf16_biased, tokens, gated, bias):
    """Two to four tokens take one launch (decode_few.cu): routing bit-exact against the staged kernels, the update
    within the bf16-activation tolerance of both the staged path and the oracle, bitwise repeatable."""
    w = real_bf16_biased
    args = list(w.tuple())
    if not gated:
        args[6] = None
    rb = w.router_bias if bias else None
    for seed in range(3):
        hidden = make_hidden(700 + 10 * tokens + seed, tokens, REAL, dtype=torch.bfloat16, device="cuda")
        fused = triton_qwen36_batched_moe_layer_decode(hidden, *args, router_bias=rb)
        staged = triton_qwen36_batched_moe_layer_decode(hidden, *args, router_bias=rb, flags=_lib.FLAG_NO_FUSED_DECODE)
        assert torch.equal(fused[3], staged[3])                       # ids
        torch.testing.assert_close(fused[2], staged[2], atol=1e-5, rtol=1e-5)   # logits
        torch.testing.assert_close(fused[4], staged[4], atol=1e-6, rtol=1e-5)   # weights
        assert O.max_abs(fused[1].cpu(), staged[1].cpu()) <= 2e-2 and O.rel_l2(fused[1].cpu(), staged[1].cpu()) <= 5e-3
        torch.testing.assert_close(fused[0], hidden.float() + fused[1], atol=0, rtol=0)
        ref = oracle_layer(hidden, MoEWeights(*args, rb), 8)
        check_routing(fused[2], fused[3], fused[4], ref, torch.bfloat16)
        check_output_where_ids_agree(fused[1], fused[3], ref.topk_ids, ref.output, torch.bfloat16, what=f"few-token kernel, {tokens} tokens")
        again = triton_qwen36_batched_moe_layer_decode(hidden, *args, router_bias=rb)
        assert torch.equal(again[1], fused[1]) and torch.equal(again[3], fused[3])      # bitwise repeatable


@pytest.mark.parametrize("tokens,top_k", [(2, 1), (3, 2), (4, 5), (2, 8)])
def test_few_token_fused_kernel_other_top_k_and_few_experts(tokens, top_k):
    """Fewer than eight experts per token, and a router with fewer experts than the GPU has blocks (16: most blocks own
    no router row): the single-launch kernel against the staged kernels and the oracle."""
    spec = MoESpec(hidden_size=2048, num_experts=16, num_routed_experts=top_k, expert_intermediate_size=512)
    w = make_moe_weights(60 + top_k, spec, dtype=torch.bfloat16, device="cuda", bias_std=0.5)
    for seed in range(2):
        hidden = make_hidden(800 + 10 * tokens + seed, tokens, spec, dtype=torch.bfloat16, device="cuda")
        fused = triton_qwen36_batched_moe_layer_decode(hidden, *w.tuple(), top_k=top_k, router_bias=w.router_bias)
        staged = triton_qwen36_batched_moe_layer_decode(hidden, *w.tuple(), top_k=top_k, router_bias=w.router_bias,
                                                        flags=_lib.FLAG_NO_FUSED_DECODE)
        assert torch.equal(fused[3], staged[3])
        torch.testing.assert_close(fused[4], staged[4], atol=1e-6, rtol=1e-5)
        assert O.max_abs(fused[1].cpu(), staged[1].cpu()) <= 2e-2 and O.rel_l2(fused[1].cpu(), staged[1].cpu()) <= 5e-3
        ref = oracle_layer(hidden, w, top_k)
        check_routing(fused[2], fused[3], fused[4], ref, torch.bfloat16)
        check_output_where_ids_agree(fused[1], fused[3], ref.topk_ids, ref.output, torch.bfloat16,
                                     what=f"few-token kernel, {tokens} tokens, top-{top_k}")


def test_few_token_fused_kernel_tokens_sharing_experts():
    """Experts chosen by several tokens are streamed once and multiplied for all of them: identical tokens share all
    eight experts, hot experts are shared by most tokens, and a token's result must not depend on its neighbours."""
    w = make_moe_weights(55, REAL, dtype=torch.bfloat16, device="cuda", bias_std=0.5, hot_experts=HOT_EXPERT_IDS)
    x = make_hidden(56, 4, REAL, dtype=torch.bfloat16, device="cuda")
    same = x[:1].repeat(4, 1).contiguous()
    out, _, ids, _ = triton_qwen36_batched_moe_decode(same, *w.tuple(), router_bias=w.router_bias)
    assert all(torch.equal(ids[0], ids[t]) for t in range(1, 4))
    assert all(torch.equal(out[0], out[t]) for t in range(1, 4)), "identical tokens must give identical rows"
    out, logits, ids, weights = triton_qwen36_batched_moe_decode(x, *w.tuple(), router_bias=w.router_bias)
    assert len(set(ids.flatten().tolist())) < 32, "the case needs experts shared between tokens"
    ref = oracle_layer(x, w, 8)
    check_routing(logits, ids, weights, ref, torch.bfloat16)
    check_output_where_ids_agree(out, ids, ref.topk_ids, ref.output, torch.bfloat16, what="few-token kernel, shared experts")
    # a token's row does not depend on which tokens travel with it
    pair, _, ids2, _ = triton_qwen36_batched_moe_decode(x[1:3].contiguous(), *w.tuple(), router_bias=w.router_bias)
    assert torch.equal(ids2, ids[1:3])
    assert O.max_abs(pair.cpu(), out[1:3].cpu()) <= 1e-4


def test_few_token_fused_kernel_sees_fresh_data_every_call(real_bf16_biased):
    """Alternating two batches on one workspace: a stale logit or activation word of the previous call (same address,
    older tag) would show up as a mismatch."""
    from fastkernels_b200.plan import MoEDecodePlan
    w = real_bf16_biased
    plan = MoEDecodePlan(w, 4)
    xa = make_hidden(911, 4, REAL, dtype=torch.bfloat16, device="cuda")
    xb = (xa.flip(0) * -1.3).to(torch.bfloat16)
    refs = []
    for x in (xa, xb):
        out, logits, ids, weights = plan.run(x)
        torch.cuda.synchronize()
        refs.append((out.clone(), ids.clone()))
    assert not torch.equal(refs[0][1], refs[1][1])
    for i in range(300):
        out, _, ids, _ = plan.run(xa if i % 2 == 0 else xb)
        if i % 20 >= 18:
            torch.cuda.synchronize()
            assert torch.equal(out, refs[i % 2][0]) and torch.equal(ids, refs[i % 2][1]), f"call {i}"
    # and interleaved with the single-token kernel on the same weights (the two share nothing but the GPU)
    one = MoEDecodePlan(w, 1)
    o1 = one.run(xa[:1].contiguous())[0].clone()
    for i in range(20):
        plan.run(xb)
        o = one.run(xa[:1].contiguous())[0]
    torch.cuda.synchronize()
    assert torch.equal(o, o1)


_COOPERATIVE_CHILD = """
import sys, torch
from fastkernels_b200 import _lib
from fastkernels_b200.plan import MoEDecodePlan
from fastkernels_b200.spec import MoESpec
from fastkernels_b200.workloads import make_hidden, make_moe_weights
spec = MoESpec()
w = make_moe_weights(1, spec, dtype=torch.bfloat16, device="cuda", bias_std=0.5)
for tokens in (1, 4):
    x = make_hidden(40 + tokens, tokens, spec, dtype=torch.bfloat16, device="cuda")
    fused, staged = MoEDecodePlan(w, tokens), MoEDecodePlan(w, tokens, flags=_lib.FLAG_NO_FUSED_DECODE)
    lib = _lib.load()
    for _ in range(5):
        before = lib.fk_launch_count()
        out, _, ids, _ = fused.run(x)
        assert lib.fk_launch_count() - before == 1       # the single-launch kernel took the call
    ref, _, ref_ids, _ = staged.run(x)
    torch.cuda.synchronize()
    assert torch.equal(ids, ref_ids)
    err = float((out - ref).abs().max())
    assert err <= 2e-2, err
    print("tokens", tokens, "max_abs", err)
print("cooperative ok")
"""


def test_single_launch_kernels_as_cooperative_launches():
    """FKMOE_D1_COOPERATIVE=1 (read once per process, hence the child): both single-launch kernels as cooperative
    launches, which guarantee that all blocks are resident together, against the staged kernels."""
    import os
    import subprocess
    import sys
    env = dict(os.environ, FKMOE_D1_COOPERATIVE="1")
    root = str(Path(__file__).resolve().parents[1])
    env["PYTHONPATH"] = root + os.pathsep + env.get("PYTHONPATH", "")
    r = subprocess.run([sys.executable, "-c", _COOPERATIVE_CHILD], env=env, cwd=root, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "cooperative ok" in r.stdout, (r.stdout[-2000:], r.stderr[-2000:])


def test_single_token_fused_kernel_fp32_hidden_and_many_calls(real_bf16):
    w = real_bf16
    hidden = make_hidden(5, 1, REAL, dtype=torch.float32, device="cuda")
    out = None
    for _ in range(50):                                               # the barrier words re-arm themselves
        out, logits, ids, weights = triton_qwen36_batched_moe_decode(hidden, *w.tuple())
    ref = oracle_layer(hidden, w, 8)
    check_routing(logits, ids, weights, ref, torch.bfloat16)
    check_output(out, ref.output, torch.bfloat16)


@pytest.mark.parametrize("tokens", [1, 5, 17, 64, 130])
def test_tensor_core_grouped_gemm_matches_gemv_path_and_oracle(real_bf16_biased, tokens):
    """tcgen05 grouped GEMM (forced at any batch) against the CUDA-core GEMV path and the oracle.
    The tensor path rounds the SwiGLU activations to bf16 before the down projection, so it is
    compared with the bf16 output bounds, not bitwise."""
    w = real_bf16_biased
    hidden = make_hidden(400 + tokens, tokens, REAL, dtype=torch.bfloat16, device="cuda")
    gemv = triton_qwen36_batched_moe_decode(hidden, *w.tuple(), router_bias=w.router_bias,
                                            flags=_lib.FLAG_FORCE_GEMV | _lib.FLAG_NO_FUSED_DECODE)
    tc = triton_qwen36_batched_moe_decode(hidden, *w.tuple(), router_bias=w.router_bias,
                                          flags=_lib.FLAG_FORCE_TENSOR | _lib.FLAG_NO_FUSED_DECODE)
    tc2 = triton_qwen36_batched_moe_decode(hidden, *w.tuple(), router_bias=w.router_bias,
                                           flags=_lib.FLAG_FORCE_TENSOR | _lib.FLAG_NO_FUSED_DECODE)
    assert torch.equal(tc[2], gemv[2]) and torch.equal(tc[0], tc2[0])
    check_output(tc[0], gemv[0].cpu(), torch.bfloat16)
    sample = torch.arange(0, tokens, max(1, tokens // 6))
    ref = oracle_layer(hidden[sample.cuda()], w, 8)
    check_output_where_ids_agree(tc[0][sample.cuda()], tc[2][sample.cuda()], ref.topk_ids, ref.output, torch.bfloat16,
                                 what=f"tensor-core path, {tokens} tokens")


def test_tensor_core_path_hot_experts_and_fp32_hidden():
    """Groups taller than one 64-row pass (hot experts), and fp32 activations converted on the way in."""
    w = make_moe_weights(2, REAL, dtype=torch.bfloat16, device="cuda", hot_experts=HOT_EXPERT_IDS, hot_boost=6.0)
    hidden = make_hidden(77, 192, REAL, dtype=torch.float32, device="cuda")
    out, logits, ids, weights = triton_qwen36_batched_moe_decode(hidden, *w.tuple(), router_bias=w.router_bias)
    hist = triton_expert_histogram(ids, 256).cpu()
    assert int(hist.max()) > 64                       # at least one group needs several passes
    sample = torch.arange(0, 192, 24)
    ref = oracle_layer(hidden[sample.cuda()], w, 8)
    assert torch.equal(ids.cpu()[sample][ref.margin > 2e-6], ref.topk_ids[ref.margin > 2e-6])
    check_output_where_ids_agree(out[sample.cuda()], ids[sample.cuda()], ref.topk_ids, ref.output, torch.bfloat16,
                                 what="hot experts, fp32 hidden")


def test_full_layer_fp32_hidden_with_bf16_weights(real_bf16):
    w = real_bf16
    hidden = make_hidden(11, 4, REAL, dtype=torch.float32, device="cuda")
    out, logits, ids, weights = triton_qwen36_batched_moe_decode(hidden, *w.tuple())
    ref = oracle_layer(hidden, w, 8)
    check_routing(logits, ids, weights, ref, torch.bfloat16)
    check_output(out, ref.output, torch.bfloat16)


def test_layer_residual(real_bf16):
    w = real_bf16
    hidden = make_hidden(13, 4, REAL, dtype=torch.bfloat16, device="cuda")
    layer, update, logits, ids, weights = triton_qwen36_batched_moe_layer_decode(hidden, *w.tuple())
    assert layer.dtype == torch.float32
    torch.testing.assert_close(layer, hidden.float() + update, atol=0, rtol=0)
    ref = oracle_layer(hidden, w, 8)
    check_output(update, ref.output, torch.bfloat16)


@pytest.mark.parametrize("name", list(CASES))
def test_full_layer_matches_reference_golden(name):
    spec, tokens, dtype, seed, bias_std = CASES[name]
    gold = np.load(GOLDEN / f"moe_{name}.npz")
    w = make_moe_weights(seed, spec, dtype=dtype, bias_std=bias_std).to("cuda")
    hidden = make_hidden(seed, tokens, spec, dtype=dtype).cuda()
    out, logits, ids, weights = triton_qwen36_batched_moe_decode(hidden, *w.tuple(), top_k=spec.num_routed_experts,
                                                                 router_bias=w.router_bias)
    np.testing.assert_allclose(logits.cpu().numpy(), gold["logits"], atol=1e-4, rtol=1e-4)
    clear = torch.from_numpy(gold["margin"]) > 2e-6
    assert torch.equal(ids.cpu()[clear], torch.from_numpy(gold["topk_ids"])[clear])
    gold_ids = torch.from_numpy(gold["topk_ids"])
    hist = triton_expert_histogram(ids, spec.num_experts).cpu()
    assert torch.equal(hist, O.expert_histogram(ids.cpu(), spec.num_experts))
    agree = (ids.cpu() == gold_ids).all(dim=-1)
    assert int((~agree).sum()) <= max(1, tokens // 64)
    assert bool(agree.all()) is False or torch.equal(hist, torch.from_numpy(gold["histogram"]))
    check_output_where_ids_agree(out, ids, gold_ids, torch.from_numpy(gold["output"]), dtype, what=f"golden {name}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("top_k", [1, 2, 4, 8])
def test_synthetic_tiny_block(dtype, top_k):
    spec = MoESpec(hidden_size=16, num_experts=8 if top_k > 4 else 4, num_routed_experts=top_k, expert_intermediate_size=8)
    w = make_moe_weights(20 + top_k, spec, dtype=dtype, device="cuda", shared_gate=False, scale=0.2)
    norm_w = torch.ones(16, device="cuda", dtype=dtype)
    hidden = make_hidden(21, 1, spec, dtype=dtype, device="cuda")[0]
    out = triton_synthetic_qwen36_moe_decode(hidden, norm_w, w.router_weight, w.expert_gate_up_weight, w.expert_down_weight,
                                             w.shared_gate_up_weight, w.shared_down_weight, top_k=top_k)
    assert out.dtype == dtype and out.shape == hidden.shape
    ref = O.synthetic_moe_decode(hidden.cpu(), norm_w.cpu(), w.router_weight.cpu(), w.expert_gate_up_weight.cpu(),
                                 w.expert_down_weight.cpu(), w.shared_gate_up_weight.cpu(), w.shared_down_weight.cpu(), top_k=top_k)
    atol, rtol = default_tolerance(dtype)
    torch.testing.assert_close(out.float().cpu(), ref, atol=atol, rtol=rtol)


def test_synthetic_tiny_block_golden_and_256_experts():
    g = np.load(GOLDEN / "synthetic_tiny.npz")
    t = {k: torch.from_numpy(g[k]).cuda() for k in g.files}
    out = triton_synthetic_qwen36_moe_decode(t["hidden"], t["norm_weight"], t["router_weight"], t["expert_gate_up_weight"],
                                             t["expert_down_weight"], t["shared_gate_up_weight"], t["shared_down_weight"], top_k=2)
    torch.testing.assert_close(out.cpu(), t["output"].cpu(), atol=1e-5, rtol=1e-4)
    spec = MoESpec(hidden_size=16, num_experts=256, num_routed_experts=8, expert_intermediate_size=8)
    w = make_moe_weights(30, spec, dtype=torch.float32, device="cuda", shared_gate=False, scale=0.2)
    hidden = make_hidden(31, 1, spec, dtype=torch.float32, device="cuda")[0]
    norm_w = torch.ones(16, device="cuda")
    out = triton_synthetic_qwen36_moe_decode(hidden, norm_w, w.router_weight, w.expert_gate_up_weight, w.expert_down_weight,
                                             w.shared_gate_up_weight, w.shared_down_weight, top_k=8)
    ref = O.synthetic_moe_decode(hidden.cpu(), norm_w.cpu(), w.router_weight.cpu(), w.expert_gate_up_weight.cpu(),
                                 w.expert_down_weight.cpu(), w.shared_gate_up_weight.cpu(), w.shared_down_weight.cpu(), top_k=8)
    torch.testing.assert_close(out.cpu(), ref, atol=1e-4, rtol=1e-4)


# ---------------------------------------------------------------- edge cases and full-size properties
def test_empty_batch(real_bf16):
    w = real_bf16
    hidden = torch.empty(0, 2048, device="cuda", dtype=torch.bfloat16)
    out, logits, ids, weights = triton_qwen36_batched_moe_decode(hidden, *w.tuple())
    assert out.shape == (0, 2048) and logits.shape == (0, 256) and ids.shape == (0, 8)
    assert triton_expert_histogram(ids, 256).sum().item() == 0


def test_all_tokens_on_the_same_experts(real_bf16):
    # ragged extreme: every token routes to the same 8 experts (one group of 24 rows each)
    w = real_bf16
    tokens = 24
    hidden = _randn(tokens, 2048, dtype=torch.bfloat16, seed=40)
    ids = torch.tensor([FIXED_IDS] * tokens, device="cuda")
    wts = torch.full((tokens, 8), 0.125, device="cuda")
    out = triton_qwen36_batched_routed_experts_decode(hidden, ids, wts, w.expert_gate_up_weight, w.expert_down_weight)
    sel = torch.tensor(FIXED_IDS)
    ref = O.routed_experts(hidden.cpu(), torch.arange(8).repeat(tokens, 1), wts.cpu(),
                           w.expert_gate_up_weight[sel.cuda()].cpu(), w.expert_down_weight[sel.cuda()].cpu())
    check_output(out, ref, torch.bfloat16)


@pytest.mark.parametrize("tokens,hot", [(64, False), (256, False), (256, True)])
def test_full_size_batches_properties(tokens, hot):
    """Largest single-GPU batches: routing bit-exact on the kernel's own logits, histogram sums,
    linearity in the routing weights, token-order independence, and oracle parity on a token sample."""
    w = make_moe_weights(2, REAL, dtype=torch.bfloat16, device="cuda", hot_experts=HOT_EXPERT_IDS if hot else None)
    hidden = make_hidden(200 + tokens, tokens, REAL, dtype=torch.bfloat16, device="cuda")
    out, logits, ids, weights = triton_qwen36_batched_moe_decode(hidden, *w.tuple(), router_bias=w.router_bias)
    own_ids, own_w = O.route_from_logits(logits.cpu(), 8)
    assert torch.equal(ids.cpu(), own_ids)
    hist = triton_expert_histogram(ids, 256)
    assert int(hist.sum()) == tokens * 8
    assert torch.equal(hist.cpu(), O.expert_histogram(ids.cpu(), 256))
    if hot:
        assert int(hist.cpu()[list(HOT_EXPERT_IDS)].sum()) > tokens * 8 // 4
    # permuting the tokens permutes the outputs (bitwise: per-token math does not depend on batch order)
    perm = torch.randperm(tokens, generator=torch.Generator().manual_seed(1)).cuda()
    out_p, _, ids_p, _ = triton_qwen36_batched_moe_decode(hidden[perm], *w.tuple(), router_bias=w.router_bias)
    assert torch.equal(ids_p, ids[perm])
    torch.testing.assert_close(out_p, out[perm], atol=1e-5, rtol=1e-4)
    # linearity of the routed part in the routing weights
    r1 = triton_qwen36_batched_routed_experts_decode(hidden, ids, weights, w.expert_gate_up_weight, w.expert_down_weight)
    r2 = triton_qwen36_batched_routed_experts_decode(hidden, ids, 2 * weights, w.expert_gate_up_weight, w.expert_down_weight)
    torch.testing.assert_close(r2, 2 * r1, atol=1e-6, rtol=1e-5)
    # oracle parity on a sample of tokens (the oracle needs only the experts those tokens use)
    sample = torch.arange(0, tokens, max(1, tokens // 8))
    ref = oracle_layer(hidden[sample.cuda()], w, 8)
    clear = ref.margin > 2e-6
    assert torch.equal(ids.cpu()[sample][clear], ref.topk_ids[clear])
    check_output_where_ids_agree(out[sample.cuda()], ids[sample.cuda()], ref.topk_ids, ref.output, torch.bfloat16,
                                 what=f"{tokens} tokens, hot={hot}")


@pytest.mark.parametrize("hot", [False, True])
def test_full_256_token_batch_every_token_against_the_token_loop_oracle(hot):
    """The largest single-GPU batch, all 256 tokens (not a sample), against the oracle with the reference's own loop
    structure (token by token, route by route)."""
    w = make_moe_weights(3, REAL, dtype=torch.bfloat16, device="cuda", bias_std=0.0 if hot else 0.5,
                         hot_experts=HOT_EXPERT_IDS if hot else None)
    tokens = 256
    hidden = make_hidden(900 + int(hot), tokens, REAL, dtype=torch.bfloat16, device="cuda")
    out, logits, ids, weights = triton_qwen36_batched_moe_decode(hidden, *w.tuple(), router_bias=w.router_bias)
    wc = w.to("cpu")
    ref_out = O.moe_update_token_loop(hidden.cpu(), *wc.tuple(), top_k=8, router_bias=wc.router_bias)
    ref_logits, ref_ids, ref_w = O.router(hidden.cpu(), wc.norm_weight, wc.router_weight, top_k=8, router_bias=wc.router_bias)
    torch.testing.assert_close(logits.cpu(), ref_logits, atol=1e-4, rtol=1e-4)
    own_ids, _ = O.route_from_logits(logits.cpu(), 8)
    assert torch.equal(ids.cpu(), own_ids)
    assert torch.equal(triton_expert_histogram(ids, 256).cpu(), O.expert_histogram(ids.cpu(), 256))
    if hot:
        assert int(triton_expert_histogram(ids, 256).cpu()[list(HOT_EXPERT_IDS)].sum()) > tokens * 8 // 4
    check_output_where_ids_agree(out, ids, ref_ids, ref_out, torch.bfloat16, what=f"256 tokens, hot={hot}")


# ---------------------------------------------------------------- layer stack
@pytest.mark.parametrize("tokens", [1, 3])
def test_layer_stack_matches_oracle(tokens):
    """x <- x + MoE_l(RMSNorm(x)) over three real-shape layers, one CUDA graph, against the oracle."""
    from fastkernels_b200.stack import MoEStackPlan
    layers = [make_moe_weights(50 + l, REAL, dtype=torch.bfloat16, device="cuda") for l in range(3)]
    x0 = make_hidden(60, tokens, REAL, dtype=torch.float32, device="cuda")
    plan = MoEStackPlan(layers, tokens)
    out = plan.run(x0).clone()
    out2 = plan.run(x0).clone()
    assert torch.equal(out, out2)
    ref, ref_ids = O.moe_stack(x0.cpu(), [[None if t is None else t.cpu() for t in w.tuple()] for w in layers],
                               act_dtype=torch.bfloat16, return_ids=True)
    same = all(torch.equal(a.cpu(), b) for a, b in zip(plan.topk_ids, ref_ids))
    if same:
        delta, ref_delta = (out - x0).cpu(), ref - x0.cpu()
        assert O.max_abs(delta, ref_delta) <= 2e-2 and O.rel_l2(delta, ref_delta) <= 5e-3


@pytest.mark.parametrize("tokens,lo,n", [(10, 3, 4), (96, 32, 32)])
def test_shared_expert_on_a_token_sub_range(real_bf16, tokens, lo, n):
    """The shared expert restricted to tokens [lo, lo+n) (what an expert-parallel rank asks for its own
    tokens among the gathered ones) on the GEMV path (10 tokens) and the tensor-core path (96 tokens)."""
    from fastkernels_b200.moe import _experts
    w = real_bf16
    hidden = make_hidden(500 + tokens, tokens, REAL, dtype=torch.bfloat16, device="cuda")
    _, ids, wts = triton_qwen36_batched_moe_router_decode(hidden, w.norm_weight, w.router_weight)
    routed = triton_qwen36_batched_routed_experts_decode(hidden, ids, wts, w.expert_gate_up_weight, w.expert_down_weight)
    both = triton_qwen36_batched_routed_shared_experts_decode(hidden, ids, wts, w.expert_gate_up_weight, w.expert_down_weight,
                                                              w.shared_gate_up_weight, w.shared_down_weight,
                                                              w.shared_expert_gate_weight)
    sub = _experts(hidden, ids, wts, w.expert_gate_up_weight, w.expert_down_weight, w.shared_gate_up_weight,
                   w.shared_down_weight, w.shared_expert_gate_weight, shared_token_range=(lo, n))
    inside = torch.zeros(tokens, dtype=torch.bool, device="cuda")
    inside[lo:lo + n] = True
    torch.testing.assert_close(sub[inside], both[inside], atol=1e-6, rtol=1e-5)
    torch.testing.assert_close(sub[~inside], routed[~inside], atol=1e-6, rtol=1e-5)


def test_single_token_fused_kernel_sees_fresh_data_every_call(real_bf16_biased):
    """The fused kernel exchanges logits and activations between its blocks through global memory.
    Alternating two different tokens on the same workspace makes any read of the previous call's
    values (a grid barrier that opens early) show up as a mismatch."""
    from fastkernels_b200.plan import MoEDecodePlan
    w = real_bf16_biased
    plan = MoEDecodePlan(w, 1)
    xa = make_hidden(901, 1, REAL, dtype=torch.bfloat16, device="cuda")
    xb = (xa * -1.7).to(torch.bfloat16)
    refs = []
    for x in (xa, xb):
        out, logits, ids, weights = plan.run(x)
        torch.cuda.synchronize()
        refs.append((out.clone(), ids.clone()))
    assert not torch.equal(refs[0][0], refs[1][0])
    for i in range(400):
        out, _, ids, _ = plan.run(xa if i % 2 == 0 else xb)
        if i % 20 >= 18:
            torch.cuda.synchronize()
            assert torch.equal(out, refs[i % 2][0]) and torch.equal(ids, refs[i % 2][1]), f"call {i}"


def test_single_token_fused_kernel_first_run_on_fresh_weights():
    """Freshly allocated weights are read through cold pages, so the bulk copies of a block complete far
    out of order.  The first call after a warm-up on a different token must already equal the later calls
    (a consumer that took a ring slot one lap early would have used stale data on exactly this call)."""
    from fastkernels_b200.plan import MoEDecodePlan
    x = make_hidden(77, 1, REAL, dtype=torch.bfloat16, device="cuda")
    for rep in range(3):
        w = make_moe_weights(300 + rep, REAL, dtype=torch.bfloat16, device="cuda", bias_std=0.5)
        plan = MoEDecodePlan(w, 1)
        plan.run(torch.zeros_like(x))                      # warm-up on other data: leaves different values behind
        outs = []
        for _ in range(3):
            out, _, ids, _ = plan.run(x)
            outs.append((out.clone(), ids.clone()))
        torch.cuda.synchronize()
        assert torch.equal(outs[0][0], outs[2][0]) and torch.equal(outs[1][0], outs[2][0]), f"weights {rep}"
        assert torch.equal(outs[0][1], outs[2][1])
        ref = oracle_layer(x, w, 8)
        assert float(ref.margin.min()) > 2e-6, "pick another seed: this token's cut is a near-tie"
        assert torch.equal(outs[0][1].cpu(), ref.topk_ids)
        check_output(outs[0][0], ref.output, torch.bfloat16)
        del plan, w


def test_resident_layers_from_checkpoint_mapping_match_function_api():
    """Checkpoint-style mapping -> packed bf16 layers on the GPU -> per-layer calls, against the drop-in
    function on the same packed tensors (the caller of the reference's decode loop, MoE sublayer only)."""
    from fastkernels_b200.stack import ResidentMoELayers
    from fastkernels_b200.weights import pack_qwen36_moe_weights_from_state_dict, state_dict_from_moe_weights
    spec = MoESpec(hidden_size=256, num_experts=16, num_routed_experts=4, expert_intermediate_size=256, num_layers=2)
    ckpt = {}
    for layer in (0, 1):
        ckpt.update(state_dict_from_moe_weights(make_moe_weights(400 + layer, spec, dtype=torch.float32), layer,
                                                grouped=(layer == 0)))
    tokens = 5
    resident = ResidentMoELayers.from_state_dict(ckpt, [0, 1], tokens, spec=spec, top_k=4)
    hidden = make_hidden(41, tokens, spec, dtype=torch.bfloat16, device="cuda")
    for layer in (0, 1):
        w = pack_qwen36_moe_weights_from_state_dict(ckpt, layer, spec=spec, device="cuda", dtype=torch.bfloat16).weights
        want = triton_qwen36_batched_moe_layer_decode(hidden, *w.tuple(), top_k=4)[0]
        got = resident.layer(layer, hidden)
        assert torch.equal(got, want)
        ref = oracle_layer(hidden, w, 4)
        check_output(got - hidden.float(), ref.output, torch.bfloat16)


def test_host_buffer_call_eager_and_graph(real_bf16_biased):
    """Host buffers in, host buffers out: the captured variant equals the eager one and the device-resident call."""
    from fastkernels_b200.plan import MoEDecodePlan
    w = real_bf16_biased
    tokens = 7
    plan = MoEDecodePlan(w, tokens)
    x = make_hidden(55, tokens, REAL, dtype=torch.bfloat16)
    out_d, _, ids_d, w_d = plan.run(x.cuda())
    out_d, ids_d, w_d = out_d.cpu(), ids_d.cpu(), w_d.cpu()
    out_e = torch.empty(tokens, REAL.hidden_size).pin_memory()
    ids_e = torch.empty(tokens, 8, dtype=torch.int64).pin_memory()
    w_e = torch.empty(tokens, 8).pin_memory()
    plan.run_host(x.pin_memory(), out_e, ids_e, w_e)
    torch.cuda.synchronize()
    assert torch.equal(out_e, out_d) and torch.equal(ids_e, ids_d) and torch.equal(w_e, w_d)
    for _ in range(2):
        out_g, ids_g, w_g = plan.run_host_graph(x)
        torch.cuda.synchronize()
        assert torch.equal(out_g, out_d) and torch.equal(ids_g, ids_d) and torch.equal(w_g, w_d)


def test_peer_memory_layer_with_one_rank_equals_the_plain_layer(real_bf16_biased, tmp_path):
    """World size 1 runs the dispatch, home-rank combine and reduce kernels of the expert-parallel call against the
    rank's own buffer: same bits as the single-GPU layer."""
    import torch.distributed as dist
    from fastkernels_b200.ep import PeerEPLayer, PeerExchange, shard_weights
    w = real_bf16_biased
    created = not dist.is_initialized()
    if created:
        dist.init_process_group("gloo", init_method=f"file://{tmp_path}/pg", rank=0, world_size=1)
    try:
        for tokens in (1, 9, 70):
            exchange = PeerExchange(tokens, REAL.hidden_size, 8, torch.bfloat16)
            layer = PeerEPLayer(shard_weights(w, 0, 1), exchange, tokens)
            for seed in (5, 6):
                hidden = make_hidden(seed, tokens, REAL, dtype=torch.bfloat16, device="cuda")
                out, logits, ids, weights = layer.run(hidden)
                want, want_logits, want_ids, want_w = triton_qwen36_batched_moe_decode(
                    hidden, *w.tuple(), router_bias=w.router_bias, flags=_lib.FLAG_NO_FUSED_DECODE)
                assert torch.equal(ids, want_ids) and torch.equal(weights, want_w) and torch.equal(logits, want_logits)
                assert torch.equal(out, want)
            assert exchange.error() == 0
            exchange.close()
        # many tokens per expert (32 experts, 600 tokens: 150 each) through the tcgen05 kernels, and the same with
        # 128-token passes: the rows must not depend on how an expert's tokens are split into passes
        spec32 = MoESpec(num_experts=32)
        w32 = make_moe_weights(9, spec32, dtype=torch.bfloat16, device="cuda", bias_std=0.5)
        tokens = 600
        exchange = PeerExchange(tokens, spec32.hidden_size, 8, torch.bfloat16)
        layer = PeerEPLayer(shard_weights(w32, 0, 1), exchange, tokens)
        hidden = make_hidden(12, tokens, spec32, dtype=torch.bfloat16, device="cuda")
        out, logits, ids, weights = layer.run(hidden)
        want, _, want_ids, _ = triton_qwen36_batched_moe_decode(hidden, *w32.tuple(), router_bias=w32.router_bias)
        assert torch.equal(ids, want_ids) and torch.equal(out, want)
        wide, _, wide_ids, _ = triton_qwen36_batched_moe_decode(hidden, *w32.tuple(), router_bias=w32.router_bias,
                                                                flags=_lib.FLAG_WIDE_PASSES)
        assert torch.equal(wide_ids, want_ids) and torch.equal(wide, want)
        sample = torch.arange(0, tokens, 75)
        ref = oracle_layer(hidden[sample.cuda()], w32, 8)
        clear = ref.margin > 2e-6
        assert torch.equal(ids.cpu()[sample][clear], ref.topk_ids[clear])
        check_output_where_ids_agree(out[sample.cuda()], ids[sample.cuda()], ref.topk_ids, ref.output, torch.bfloat16,
                                     what="32 experts, 600 tokens")
        assert exchange.error() == 0
        exchange.close()
    finally:
        if created:
            dist.destroy_process_group()
