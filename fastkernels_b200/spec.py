"""Shape spec and weight container for one Qwen3.6 MoE layer.

Mirrors the MoE-relevant fields of the reference's `Qwen36A3BSpec`
(src/fastkernels/models/qwen36.py:11-32, real spec :170-191, tiny spec :194-214)
and of `Qwen36MoEWeights` (src/fastkernels/models/qwen36_weights.py:26-37).
Field names are the reference's so that objects of either kind can be passed
to `moe_weights_tuple`.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional


@dataclass(frozen=True)
class MoESpec:
    hidden_size: int = 2048
    num_experts: int = 256
    num_routed_experts: int = 8          # top-k
    num_shared_experts: int = 1
    expert_intermediate_size: int = 512
    num_layers: int = 40
    name: str = "Qwen3.6-35B-A3B"

    @property
    def gated_up_features(self) -> int:
        return 2 * self.expert_intermediate_size

    @property
    def expert_bytes_bf16(self) -> int:
        """bf16 bytes of one expert (gate_up + down)."""
        return 2 * 3 * self.hidden_size * self.expert_intermediate_size


def qwen36_35b_a3b_spec() -> MoESpec:
    """H=2048, E=256, k=8, I=512, one shared expert, 40 layers."""
    return MoESpec()


def synthetic_qwen36_spec() -> MoESpec:
    """The reference's tiny test spec: H=16, E=4, k=2, I=8."""
    return MoESpec(hidden_size=16, num_experts=4, num_routed_experts=2, num_shared_experts=1,
                   expert_intermediate_size=8, num_layers=4, name="synthetic-qwen3.6-a3b")


@dataclass(frozen=True)
class MoEWeights:
    """Kernel-facing tensors of one layer, all row-major contiguous.

    norm_weight [H]; router_weight [E,H]; expert_gate_up_weight [E,2I,H] (gate
    rows 0..I-1, up rows I..2I-1); expert_down_weight [E,H,I];
    shared_gate_up_weight [2I,H]; shared_down_weight [H,I];
    shared_expert_gate_weight [H] or [1,H] or None; router_bias fp32 [E] or None
    (benchmark-only load skew, not part of the reference container).
    """

    norm_weight: Any
    router_weight: Any
    expert_gate_up_weight: Any
    expert_down_weight: Any
    shared_gate_up_weight: Any
    shared_down_weight: Any
    shared_expert_gate_weight: Optional[Any] = None
    router_bias: Optional[Any] = None

    def tuple(self):
        return moe_weights_tuple(self)

    def to(self, *args, **kwargs) -> "MoEWeights":
        def mv(t):
            return None if t is None else t.to(*args, **kwargs)
        bias = self.router_bias
        if bias is not None:
            dev_kwargs = {k: v for k, v in kwargs.items() if k == "device"}
            dev_args = [a for a in args if not _is_dtype(a)]
            bias = bias.to(*dev_args, **dev_kwargs)
        return MoEWeights(mv(self.norm_weight), mv(self.router_weight), mv(self.expert_gate_up_weight),
                          mv(self.expert_down_weight), mv(self.shared_gate_up_weight),
                          mv(self.shared_down_weight), mv(self.shared_expert_gate_weight), bias)


def _is_dtype(obj) -> bool:
    import torch
    return isinstance(obj, torch.dtype)


def moe_weights_tuple(w) -> tuple:
    """Positional weight tuple in the order every MoE entry point takes them."""
    return (w.norm_weight, w.router_weight, w.expert_gate_up_weight, w.expert_down_weight,
            w.shared_gate_up_weight, w.shared_down_weight, w.shared_expert_gate_weight)
