"""CPU oracle for the Qwen3.6 MoE decode layer.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain PyTorch fp32 on the CPU, the algorithm of the
reference project's MoE path.  It exists so that the CUDA kernels can be
checked against it; it is never imported by the product package.  Only the
test-suite, the smoke check and the CPU-baseline leg of the benchmark use it.

Parity status: PINNED.  `oracle/pin_against_reference.py` imports the
reference's own functions (`fastkernels.reference.qwen36_real_moe_update`,
`reference_routed_moe`, `reference_expert_histogram`, `reference_fused_swiglu`,
`reference_qwen36_moe_decode`, `qwen36_real_rms_norm`) and checks every
function below against them; it also writes the golden vectors under
`tests/golden/` that `tests/test_oracle_golden.py` replays without the
reference tree.  The reference ships no golden vectors of its own for this
path (its pins are formula-equivalence tests in tests/test_triton_moe.py and
the RMSNorm known answer in tests/test_qwen36_spec.py:368-377, replayed in
`tests/test_oracle_golden.py`).

Every function cites the reference lines it follows (paths are relative to the
reference project's root).

One rule is stated more tightly than the reference does: ties between equal
router probabilities go to the LOWER expert index.  `torch.topk` leaves tie
order unspecified, so the reference's result is only defined when the selected
probabilities are distinct; for distinct probabilities the two agree exactly.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------- #
# Router                                                                      #
# --------------------------------------------------------------------------- #

def rms_norm(hidden: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6,
             norm_offset: float = 1.0) -> torch.Tensor:
    """`x * rsqrt(mean(x^2) + eps) * (norm_offset + w)` in fp32.

    Follows src/fastkernels/reference/qwen36_real.py:23-28 (offset 1.0) and the
    `norm_offset` knob of src/fastkernels/kernels/triton/qwen36_router.py:130-133.
    With `norm_offset=0` it is the plain-weight norm of
    src/fastkernels/reference/qwen36_decode.py:27-29.
    """
    x = hidden.float()
    inv = torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return (x * inv) * (norm_offset + weight.float())


def topk_lower_index(probs: torch.Tensor, k: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Top-k of each row, descending, ties to the lower column index.

    Equal to `torch.topk(probs, k)` (src/fastkernels/reference/qwen36_real.py:336,
    src/fastkernels/reference/moe.py:78) whenever the values are distinct.
    """
    order = torch.sort(probs, dim=-1, descending=True, stable=True).indices[..., :k]
    return torch.gather(probs, -1, order), order


def route_from_logits(logits: torch.Tensor, top_k: int,
                      normalize: bool = True) -> tuple[torch.Tensor, torch.Tensor]:
    """softmax -> top-k -> renormalise (qwen36_real.py:335-337, moe.py:77-80).

    Returns `(ids int64 [T,k], weights fp32 [T,k])`.
    """
    probs = torch.softmax(logits.float(), dim=-1)
    vals, ids = topk_lower_index(probs, top_k)
    if normalize:
        vals = vals / vals.sum(dim=-1, keepdim=True)
    return ids, vals


def router(hidden: torch.Tensor, norm_weight: torch.Tensor, router_weight: torch.Tensor, *,
           top_k: int = 8, eps: float = 1e-6, norm_offset: float = 1.0,
           router_bias: Optional[torch.Tensor] = None):
    """Router logits, ids and weights (qwen36_real.py:333-337).

    `router_bias` (fp32 `[E]`, added to the logits) is the load-skew knob of the
    benchmark configurations; the reference takes ready-made logits for that
    case (`reference_routed_moe`, moe.py:33-41).
    """
    normed = rms_norm(hidden, norm_weight, eps, norm_offset)
    logits = normed @ router_weight.float().t()
    if router_bias is not None:
        logits = logits + router_bias.float()
    ids, weights = route_from_logits(logits, top_k)
    return logits, ids, weights


# --------------------------------------------------------------------------- #
# Histogram / permutation                                                     #
# --------------------------------------------------------------------------- #

def expert_histogram(topk_ids: torch.Tensor, num_experts: int) -> torch.Tensor:
    """Routes per expert, int32 `[E]` (src/fastkernels/reference/moe.py:24-30)."""
    if topk_ids.ndim != 2:
        raise ValueError("topk_ids must have shape [tokens, top_k]")
    return torch.bincount(topk_ids.reshape(-1).long(), minlength=num_experts).to(torch.int32)


def expert_permutation(topk_ids: torch.Tensor, num_experts: int):
    """Histogram, exclusive offsets and the stable expert-major route order.

    The reference has no packing function (it is a TODO in
    docs/QWEN36_MEGAKERNEL_PLAN.md:142-149); the definition used here is
    `order = argsort(ids.flatten(), stable=True)`: `order[j] // k` is the token
    and `order[j] % k` the slot of the j-th packed row.
    Returns `(counts int32 [E], offsets int32 [E+1], order int32 [T*k])`.
    """
    counts = expert_histogram(topk_ids, num_experts)
    offsets = torch.zeros(num_experts + 1, dtype=torch.int32)
    offsets[1:] = torch.cumsum(counts, 0)
    order = torch.sort(topk_ids.reshape(-1).long(), stable=True).indices.to(torch.int32)
    return counts, offsets, order


# --------------------------------------------------------------------------- #
# Expert math                                                                 #
# --------------------------------------------------------------------------- #

def fused_swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """`silu(gate) * up` for `[N, 2I]` (src/fastkernels/reference/moe.py:16-21)."""
    gate, up = gate_up.chunk(2, dim=-1)
    return F.silu(gate) * up


def expert_mlp(x: torch.Tensor, gate_up_weight: torch.Tensor, down_weight: torch.Tensor) -> torch.Tensor:
    """`Wd (silu(Wg x) * (Wu x))` for rows `x [n,H]`, fp32 (qwen36_real.py:343-347)."""
    gu = x.float() @ gate_up_weight.float().t()
    return fused_swiglu(gu) @ down_weight.float().t()


def routed_experts(hidden, topk_ids, topk_weights, expert_gate_up_weight, expert_down_weight):
    """Weighted sum of the selected experts, slot by slot (qwen36_real.py:339-347).

    The token x route loop of the reference is kept (slot order fixes the fp32
    summation order); rows that share an expert are batched inside one slot.
    """
    x = hidden.float()
    out = torch.zeros_like(x)
    tokens, top_k = topk_ids.shape
    for slot in range(top_k):
        ids = topk_ids[:, slot].long()
        contrib = torch.zeros_like(x)
        for e in torch.unique(ids).tolist():
            rows = torch.nonzero(ids == e).flatten()
            contrib[rows] = expert_mlp(x[rows], expert_gate_up_weight[e], expert_down_weight[e])
        out += topk_weights[:, slot].float().unsqueeze(1) * contrib
    return out


def shared_expert(hidden, shared_gate_up_weight, shared_down_weight, shared_expert_gate_weight=None):
    """Shared expert on the un-normed token, optionally sigmoid-gated (qwen36_real.py:348-352)."""
    x = hidden.float()
    y = expert_mlp(x, shared_gate_up_weight, shared_down_weight)
    if shared_expert_gate_weight is not None:
        g = x @ shared_expert_gate_weight.float().reshape(-1, x.shape[-1])[0]
        y = y * torch.sigmoid(g).unsqueeze(1)
    return y


def routed_shared_experts(hidden, topk_ids, topk_weights, expert_gate_up_weight, expert_down_weight,
                          shared_gate_up_weight, shared_down_weight, shared_expert_gate_weight=None):
    """Routed experts plus the (gated) shared expert (qwen36_real.py:339-353)."""
    return routed_experts(hidden, topk_ids, topk_weights, expert_gate_up_weight, expert_down_weight) + \
        shared_expert(hidden, shared_gate_up_weight, shared_down_weight, shared_expert_gate_weight)


@dataclass
class MoEResult:
    output: torch.Tensor          # fp32 [T,H]  (the MoE update, no residual)
    logits: torch.Tensor          # fp32 [T,E]
    topk_ids: torch.Tensor        # int64 [T,k], descending probability
    topk_weights: torch.Tensor    # fp32 [T,k], sums to one
    histogram: torch.Tensor       # int32 [E]
    margin: torch.Tensor          # fp32 [T]: p(k-th) - p((k+1)-th), how close the cut is to a tie


def moe_update(hidden, norm_weight, router_weight, expert_gate_up_weight, expert_down_weight,
               shared_gate_up_weight, shared_down_weight, shared_expert_gate_weight=None, *,
               top_k: int = 8, eps: float = 1e-6, norm_offset: float = 1.0,
               router_bias=None) -> MoEResult:
    """The whole MoE block: the oracle for the layer (qwen36_real.py:329-354)."""
    logits, ids, weights = router(hidden, norm_weight, router_weight, top_k=top_k, eps=eps,
                                  norm_offset=norm_offset, router_bias=router_bias)
    out = routed_shared_experts(hidden, ids, weights, expert_gate_up_weight, expert_down_weight,
                                shared_gate_up_weight, shared_down_weight, shared_expert_gate_weight)
    probs = torch.softmax(logits, dim=-1)
    srt = torch.sort(probs, dim=-1, descending=True, stable=True).values
    num_experts = router_weight.shape[0]
    margin = srt[:, top_k - 1] - srt[:, top_k] if top_k < num_experts else srt[:, top_k - 1]
    return MoEResult(out, logits, ids, weights, expert_histogram(ids, num_experts), margin)


def moe_update_token_loop(hidden, norm_weight, router_weight, expert_gate_up_weight, expert_down_weight,
                          shared_gate_up_weight, shared_down_weight, shared_expert_gate_weight=None, *,
                          top_k: int = 8, eps: float = 1e-6, router_bias=None) -> torch.Tensor:
    """The same block with the reference's exact loop structure: token by token, route by route, one
    matrix-vector product at a time with the weights upcast per use (qwen36_real.py:339-353).

    Numerically it equals `moe_update`; it exists so that the CPU baseline is timed on the
    reference's own control flow, not on a batched rewrite of it.
    """
    x = hidden.float()
    logits = rms_norm(x, norm_weight, eps) @ router_weight.float().t()
    if router_bias is not None:
        logits = logits + router_bias.float()
    ids, weights = route_from_logits(logits, top_k)
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        token = x[t]
        for r in range(top_k):
            e = int(ids[t, r].item())
            gate, up = torch.chunk(expert_gate_up_weight[e].float() @ token, 2, dim=0)
            out[t] += weights[t, r] * (expert_down_weight[e].float() @ (F.silu(gate) * up))
        gate, up = torch.chunk(shared_gate_up_weight.float() @ token, 2, dim=0)
        shared = shared_down_weight.float() @ (F.silu(gate) * up)
        if shared_expert_gate_weight is not None:
            shared = shared * torch.sigmoid((shared_expert_gate_weight.float().reshape(-1, x.shape[-1]) @ token)[0])
        out[t] += shared
    return out


def moe_layer(hidden, *args, **kwargs):
    """`hidden + moe_update(hidden)` in fp32 (src/fastkernels/kernels/triton/qwen36_layer.py:94-105)."""
    res = moe_update(hidden, *args, **kwargs)
    return hidden.float() + res.output, res


def routed_moe_from_logits(hidden_states, router_logits, expert_gate_up_weight, expert_down_weight, *,
                           top_k: int, normalize_topk: bool = True):
    """`reference_routed_moe` (src/fastkernels/reference/moe.py:33-93): logits given, routed experts only."""
    ids, weights = route_from_logits(router_logits, top_k, normalize_topk)
    return routed_experts(hidden_states, ids, weights, expert_gate_up_weight, expert_down_weight)


def synthetic_moe_decode(hidden, norm_weight, router_weight, expert_gate_up_weight, expert_down_weight,
                         shared_gate_up_weight, shared_down_weight, *, top_k: int, eps: float = 1e-6):
    """Tiny-spec block: plain-weight norm for the router, ungated shared expert, residual included.

    Follows src/fastkernels/reference/qwen36_decode.py:212-224 for one token `hidden [H]`.
    """
    x = hidden.float().unsqueeze(0)
    res = moe_update(x, norm_weight, router_weight, expert_gate_up_weight, expert_down_weight,
                     shared_gate_up_weight, shared_down_weight, None,
                     top_k=top_k, eps=eps, norm_offset=0.0)
    return (x + res.output)[0]


def moe_stack(hidden, layers, *, top_k: int = 8, eps: float = 1e-6, act_dtype=None, return_ids: bool = False):
    """`x <- x + MoE_l(RMSNorm(x))` over a list of layer weight tuples (unit-gain norm, eps 1e-6).

    The outer norm output is the layer's input: router, experts, shared expert
    and shared gate all read it (benchmark configuration "stack of 40 layers").
    Each element of `layers` is the positional weight tuple of `moe_update`.  The residual stream stays fp32.
    """
    x = hidden.float()
    unit = torch.zeros(x.shape[-1])
    all_ids = []
    for lw in layers:
        xin = rms_norm(x, unit, eps, 1.0)
        if act_dtype is not None:
            xin = xin.to(act_dtype)          # activations between layers are stored in this dtype
        res = moe_update(xin, *lw, top_k=top_k, eps=eps)
        all_ids.append(res.topk_ids)
        x = x + res.output
    return (x, all_ids) if return_ids else x


# --------------------------------------------------------------------------- #
# Parity metrics                                                              #
# --------------------------------------------------------------------------- #

def max_abs(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.double() - b.double()).abs().max()) if a.numel() else 0.0


def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    """`||a-b||_2 / ||b||_2` (b is the reference)."""
    den = float(b.double().norm())
    return float((a.double() - b.double()).norm()) / den if den > 0 else 0.0
