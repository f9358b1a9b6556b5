"""B200-native Qwen3.6 MoE decode layer: hand-written sm_100a CUDA behind the reference's MoE signatures."""

from .spec import MoESpec, MoEWeights, moe_weights_tuple, qwen36_35b_a3b_spec, synthetic_qwen36_spec
from .moe import (
    expert_histogram,
    expert_permutation,
    fused_swiglu,
    qwen36_batched_moe_decode,
    qwen36_batched_moe_layer_decode,
    qwen36_batched_moe_router_decode,
    qwen36_batched_routed_experts_decode,
    qwen36_batched_routed_shared_experts_decode,
    qwen36_moe_decode,
    qwen36_moe_router_decode,
    qwen36_routed_experts_decode,
    qwen36_routed_shared_experts_decode,
    qwen36_single_expert_mlp_decode,
    synthetic_qwen36_moe_decode,
)

__all__ = [
    "MoESpec", "MoEWeights", "moe_weights_tuple", "qwen36_35b_a3b_spec", "synthetic_qwen36_spec",
    "expert_histogram", "expert_permutation", "fused_swiglu",
    "qwen36_batched_moe_decode", "qwen36_batched_moe_layer_decode", "qwen36_batched_moe_router_decode",
    "qwen36_batched_routed_experts_decode", "qwen36_batched_routed_shared_experts_decode",
    "qwen36_moe_decode", "qwen36_moe_router_decode", "qwen36_routed_experts_decode",
    "qwen36_routed_shared_experts_decode", "qwen36_single_expert_mlp_decode", "synthetic_qwen36_moe_decode",
]
