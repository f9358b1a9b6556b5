"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

The reference measures this path only on random tensors (for example
bench/qwen36_batched_real_moe_microbench.py:44-72: fp32 normal draws scaled by
0.02, then cast to the run's dtype); no public dataset is involved.  Draw order
is fixed: hidden, router, router bias, gate_up, down, shared gate_up, shared
down, shared gate.  Values are drawn in fp32 and then cast.
"""

from __future__ import annotations

from typing import Optional, Sequence

import torch

from .spec import MoESpec, MoEWeights

HOT_EXPERT_IDS = (3, 17, 42, 89, 127, 199, 231, 255)   # the reference tests' fixed routing ids
                                                      # (tests/test_triton_moe.py:192)


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return g


def make_hidden(seed: int, tokens: int, spec: MoESpec, *, dtype=torch.bfloat16, device="cpu",
                scale: float = 1.0) -> torch.Tensor:
    """`x ~ N(0, scale^2)` per token, `[tokens, H]`."""
    g = _gen(seed * 7919 + 1, device)
    x = torch.randn(tokens, spec.hidden_size, generator=g, device=device, dtype=torch.float32) * scale
    return x.to(dtype)


def make_moe_weights(seed: int, spec: MoESpec, *, dtype=torch.bfloat16, device="cpu", scale: float = 0.02,
                     bias_std: float = 0.0, hot_experts: Optional[Sequence[int]] = None,
                     hot_boost: float = 3.0, shared_gate: bool = True,
                     expert_range: Optional[tuple[int, int]] = None) -> MoEWeights:
    """All weights `~ N(0, scale^2)`, `norm_weight = 0` (unit gain under the `(1 + w)` rule).

    bias_std > 0 adds a per-expert router-logit bias `~ N(0, bias_std^2)` (mild load skew);
    hot_experts adds `hot_boost` to those experts' logits (hot-expert variant).
    expert_range=(lo, hi) keeps only that slice of the routed-expert tensors (an
    expert-parallel shard); every rank still draws the same full sequence, so the values
    of an expert do not depend on how many ranks there are.
    """
    g = _gen(seed, device)
    H, E, I = spec.hidden_size, spec.num_experts, spec.expert_intermediate_size

    def randn(*shape):
        return torch.randn(*shape, generator=g, device=device, dtype=torch.float32) * scale

    router = randn(E, H).to(dtype)
    bias = torch.randn(E, generator=g, device=device, dtype=torch.float32) * bias_std
    lo, hi = expert_range if expert_range is not None else (0, E)

    def experts(rows, cols):
        # drawn expert by expert so that a shard never holds more than its own slice
        out = torch.empty(hi - lo, rows, cols, device=device, dtype=dtype)
        for e in range(E):
            w = randn(rows, cols)
            if lo <= e < hi:
                out[e - lo] = w.to(dtype)
        return out

    gate_up = experts(2 * I, H)
    down = experts(H, I)
    shared_gate_up = randn(2 * I, H).to(dtype)
    shared_down = randn(H, I).to(dtype)
    sgate = randn(H).to(dtype) if shared_gate else None
    if hot_experts is not None:
        bias = bias.clone()
        bias[list(hot_experts)] += hot_boost
    use_bias = bias_std > 0 or hot_experts is not None
    return MoEWeights(torch.zeros(H, device=device, dtype=dtype), router, gate_up, down,
                      shared_gate_up, shared_down, sgate, bias if use_bias else None)


def make_expert_subset(seed: int, spec: MoESpec, expert_ids: Sequence[int], *, dtype=torch.bfloat16, device="cpu",
                       scale: float = 0.02) -> dict:
    """`{expert id: (gate_up [2I,H], down [H,I])}` with exactly the values `make_moe_weights(seed, ...)` gives those
    experts: the whole layer's sequence is drawn again (same calls, same shapes, same order) and only the asked-for
    experts are kept.  Lets a rank that holds a shard check a few tokens against the oracle without the full layer."""
    g = _gen(seed, device)
    H, E, I = spec.hidden_size, spec.num_experts, spec.expert_intermediate_size
    keep = set(int(e) for e in expert_ids)

    def randn(*shape):
        return torch.randn(*shape, generator=g, device=device, dtype=torch.float32) * scale

    randn(E, H)                                                                  # router
    torch.randn(E, generator=g, device=device, dtype=torch.float32)              # router bias
    gate_up, down = {}, {}
    for e in range(E):
        w = randn(2 * I, H)
        if e in keep:
            gate_up[e] = w.to(dtype)
    for e in range(E):
        w = randn(H, I)
        if e in keep:
            down[e] = w.to(dtype)
    return {e: (gate_up[e], down[e]) for e in sorted(keep)}


def algorithmic_bytes(spec: MoESpec, tokens: int, distinct_experts: int, *, weight_bytes: int = 2,
                      hidden_bytes: int = 2, shared_gate: bool = True) -> int:
    """Bytes one layer call must move: each touched expert once, shared expert, router, gate, norm,
    hidden in, and the fp32 output, fp32 logits, int64 ids and fp32 weights out."""
    H, E, I, k = spec.hidden_size, spec.num_experts, spec.expert_intermediate_size, spec.num_routed_experts
    per_expert = 3 * H * I
    w = weight_bytes * (distinct_experts * per_expert + per_expert + E * H + (H if shared_gate else 0) + H)
    io = tokens * H * hidden_bytes + tokens * H * 4 + tokens * E * 4 + tokens * k * 12
    return w + io
