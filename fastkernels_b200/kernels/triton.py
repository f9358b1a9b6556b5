"""Drop-in names: `from fastkernels_b200.kernels.triton import triton_qwen36_batched_moe_decode`.

The reference exports its MoE functions from `fastkernels.kernels.triton` with a
`triton_` prefix (src/fastkernels/kernels/triton/__init__.py:34-59).  The same names are
bound here to the CUDA implementations so that a caller only changes the import.
Nothing in this package uses Triton.
"""

from .. import moe as _moe

triton_fused_swiglu = _moe.fused_swiglu
triton_expert_histogram = _moe.expert_histogram
triton_qwen36_moe_router_decode = _moe.qwen36_moe_router_decode
triton_qwen36_batched_moe_router_decode = _moe.qwen36_batched_moe_router_decode
triton_qwen36_single_expert_mlp_decode = _moe.qwen36_single_expert_mlp_decode
triton_qwen36_routed_experts_decode = _moe.qwen36_routed_experts_decode
triton_qwen36_routed_shared_experts_decode = _moe.qwen36_routed_shared_experts_decode
triton_qwen36_batched_routed_experts_decode = _moe.qwen36_batched_routed_experts_decode
triton_qwen36_batched_routed_shared_experts_decode = _moe.qwen36_batched_routed_shared_experts_decode
triton_qwen36_moe_decode = _moe.qwen36_moe_decode
triton_qwen36_batched_moe_decode = _moe.qwen36_batched_moe_decode
triton_qwen36_batched_moe_layer_decode = _moe.qwen36_batched_moe_layer_decode
triton_synthetic_qwen36_moe_decode = _moe.synthetic_qwen36_moe_decode

__all__ = [n for n in dir() if n.startswith("triton_")]
