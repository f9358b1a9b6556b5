"""CPU: the oracle replays the golden vectors written from the reference's own functions
(oracle/pin_against_reference.py), plus the reference's RMSNorm known answer."""

import hashlib
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import moe_oracle as O
from oracle.pin_against_reference import CASES, ROUTER_CASES, checksum
from fastkernels_b200.spec import MoESpec
from fastkernels_b200.workloads import make_hidden, make_moe_weights

GOLDEN = Path(__file__).parent / "golden"


def test_rms_norm_known_answer():
    # tests/test_qwen36_spec.py:368-377 of the reference
    hidden = torch.tensor([[3.0, 4.0]])
    expected = hidden * torch.rsqrt(torch.mean(hidden * hidden, dim=-1, keepdim=True) + 1e-6)
    torch.testing.assert_close(O.rms_norm(hidden, torch.zeros(2)), expected)
    torch.testing.assert_close(O.rms_norm(hidden, torch.ones(2)), 2.0 * expected)


@pytest.mark.parametrize("name", list(CASES))
def test_moe_update_matches_reference_golden(name):
    spec, tokens, dtype, seed, bias_std = CASES[name]
    gold = np.load(GOLDEN / f"moe_{name}.npz")
    wts = make_moe_weights(seed, spec, dtype=dtype, bias_std=bias_std)
    hidden = make_hidden(seed, tokens, spec, dtype=dtype)
    assert checksum(hidden, *wts.tuple(), wts.router_bias) == str(gold["inputs_sha256"]), "input generator drifted"
    res = O.moe_update(hidden, *wts.tuple(), top_k=spec.num_routed_experts, router_bias=wts.router_bias)
    assert np.array_equal(res.topk_ids.numpy(), gold["topk_ids"])
    assert np.array_equal(res.histogram.numpy(), gold["histogram"])
    assert np.array_equal(res.logits.numpy(), gold["logits"])
    np.testing.assert_allclose(res.topk_weights.numpy(), gold["topk_weights"], rtol=0, atol=1e-7)
    scale = max(1.0, float(np.abs(gold["output"]).max()))
    assert float(np.abs(res.output.numpy() - gold["output"]).max()) <= 2e-6 * scale


@pytest.mark.parametrize("name", list(ROUTER_CASES))
def test_router_matches_reference_golden(name):
    tokens, dtype, seed = ROUTER_CASES[name]
    gold = np.load(GOLDEN / f"{name}.npz")
    real = MoESpec()
    g = torch.Generator().manual_seed(seed)
    hidden = torch.randn(tokens, real.hidden_size, generator=g).to(dtype)
    norm_w = (0.02 * torch.randn(real.hidden_size, generator=g)).to(dtype)
    router_w = (0.02 * torch.randn(real.num_experts, real.hidden_size, generator=g)).to(dtype)
    assert checksum(hidden, norm_w, router_w) == str(gold["inputs_sha256"])
    logits, ids, weights = O.router(hidden, norm_w, router_w, top_k=8)
    assert np.array_equal(ids.numpy(), gold["topk_ids"])
    assert np.array_equal(logits.numpy(), gold["logits"])
    np.testing.assert_allclose(weights.numpy(), gold["topk_weights"], rtol=0, atol=1e-7)


def test_synthetic_block_matches_reference_golden():
    g = np.load(GOLDEN / "synthetic_tiny.npz")
    t = {k: torch.from_numpy(g[k]) for k in g.files}
    out = O.synthetic_moe_decode(t["hidden"], t["norm_weight"], t["router_weight"], t["expert_gate_up_weight"],
                                 t["expert_down_weight"], t["shared_gate_up_weight"], t["shared_down_weight"], top_k=2)
    assert O.max_abs(out, t["output"]) < 1e-6


def test_tie_goes_to_lower_index():
    probs = torch.tensor([[0.1, 0.3, 0.3, 0.3, 0.0], [0.2, 0.2, 0.2, 0.2, 0.2]])
    _, ids = O.topk_lower_index(probs, 2)
    assert ids.tolist() == [[1, 2], [0, 1]]
    logits = torch.zeros(1, 16)
    ids, w = O.route_from_logits(logits, 8)
    assert ids.tolist() == [list(range(8))]
    torch.testing.assert_close(w, torch.full((1, 8), 0.125))


def test_permutation_definition():
    ids = torch.tensor([[3, 1], [1, 0], [3, 3]])
    counts, offsets, order = O.expert_permutation(ids, 4)
    assert counts.tolist() == [1, 2, 0, 3]
    assert offsets.tolist() == [0, 1, 3, 3, 6]
    assert order.tolist() == [3, 1, 2, 0, 4, 5]


def test_slot_loop_equals_reference_style_token_loop():
    # the oracle batches rows inside a slot; the reference loops token by token: same numbers
    spec = MoESpec(hidden_size=64, num_experts=8, num_routed_experts=3, expert_intermediate_size=32)
    w = make_moe_weights(3, spec, dtype=torch.float32)
    x = make_hidden(3, 6, spec, dtype=torch.float32)
    res = O.moe_update(x, *w.tuple(), top_k=3)
    out = torch.zeros_like(x)
    for t in range(6):
        for r in range(3):
            e = int(res.topk_ids[t, r])
            gu = w.expert_gate_up_weight[e] @ x[t]
            g, u = gu.chunk(2)
            out[t] += res.topk_weights[t, r] * (w.expert_down_weight[e] @ (torch.nn.functional.silu(g) * u))
        gu = w.shared_gate_up_weight @ x[t]
        g, u = gu.chunk(2)
        sh = w.shared_down_weight @ (torch.nn.functional.silu(g) * u)
        out[t] += sh * torch.sigmoid(w.shared_expert_gate_weight @ x[t])
    assert O.max_abs(res.output, out) < 1e-6
