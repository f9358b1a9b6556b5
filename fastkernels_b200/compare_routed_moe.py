"""Matched-operator comparison at the routed-experts-only boundary (the boundary of a fused-MoE operator).

    python -m fastkernels_b200.compare_routed_moe --tokens 2 [--iters 50] [--checkpoint DIR --layer 0] [--require-vllm]

Mirrors the reference's harness bench/qwen36_vllm_moe_compare.py: a random case drawn as it draws it (:179-206:
hidden, router logits, gate_up and down from one CPU generator, scaled by --hidden-scale), routing from the logits
(softmax, top-k, renormalise, :127-131), this library's `triton_qwen36_batched_routed_experts_decode` timed at
that boundary (:281-314), and the same printed keys (`fastkernels_routed_max_abs_diff`, `fastkernels_routed_moe_ms`,
`..._ms_per_token`, `..._tokens_per_second`, then the vLLM block when vLLM imports).  Differences: times are CUDA
events, not a host clock; the comparison values come from a token x route loop in fp32 PyTorch on the same device
(the arithmetic of the reference's `_reference_routed`, :100-124) that belongs to this script, not to the library.
"""

from __future__ import annotations

import argparse
import inspect

import torch
import torch.nn.functional as F

from .spec import MoESpec


def torch_routed(hidden, topk_ids, topk_weights, gate_up, down):
    x = hidden.float()
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for r in range(topk_ids.shape[1]):
            e = int(topk_ids[t, r])
            g, u = torch.chunk(gate_up[e].float() @ x[t], 2)
            out[t] += topk_weights[t, r] * (down[e].float() @ (F.silu(g) * u))
    return out


def topk_from_logits(router_logits, top_k: int):
    probs = torch.softmax(router_logits.float(), dim=-1)
    ids = torch.sort(probs, dim=-1, descending=True, stable=True).indices[:, :top_k]
    vals = torch.gather(probs, -1, ids)
    return ids.to(torch.int64), vals / vals.sum(dim=-1, keepdim=True)


def load_vllm(require: bool):
    """The other operator: vLLM's fused MoE.  Newer releases export `fused_experts` (routing given, exactly this
    boundary); older ones `fused_moe` (routing from the logits inside), which is what the reference's harness calls."""
    try:
        import vllm
        import vllm.model_executor.layers.fused_moe as fm
        op = getattr(fm, "fused_experts", None)
        if not callable(op):
            op = getattr(fm, "fused_moe", None)
        if not callable(op):
            raise ImportError("neither fused_experts nor fused_moe is a callable of vllm.model_executor.layers.fused_moe")
    except Exception as exc:  # optional package
        if require:
            raise RuntimeError("vLLM is required for this comparison but could not be imported") from exc
        return None, None, repr(exc)
    return op, getattr(vllm, "__version__", "unknown"), None


def call_vllm(op, hidden, gate_up, down, router_logits, top_k, ids, weights):
    params = inspect.signature(op).parameters
    if "topk_ids" in params and "topk_weights" in params:
        return op(hidden, gate_up, down, topk_weights=weights.float(), topk_ids=ids.to(torch.int32))
    kwargs = {}
    if "renormalize" in params:
        kwargs["renormalize"] = True
    if "inplace" in params:
        kwargs["inplace"] = False
    if "gating_output" in params and "topk" in params:
        return op(hidden, gate_up, down, gating_output=router_logits, topk=top_k, **kwargs)
    return op(hidden, gate_up, down, router_logits, top_k, **kwargs)


def time_ms(fn, iters: int, warmup: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=1)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--hidden-scale", type=float, default=0.02)
    ap.add_argument("--checkpoint", default=None, help="safetensors file or directory: use that layer's real expert tensors")
    ap.add_argument("--layer", type=int, default=0)
    ap.add_argument("--require-vllm", action="store_true")
    args = ap.parse_args(argv)
    from .kernels.triton import triton_qwen36_batched_routed_experts_decode          # fails loudly without the CUDA library
    dtype = getattr(torch, args.dtype)
    spec = MoESpec()
    H, E, I, k = spec.hidden_size, spec.num_experts, spec.expert_intermediate_size, spec.num_routed_experts
    g = torch.Generator(device="cpu").manual_seed(args.seed)
    s = args.hidden_scale
    hidden = (s * torch.randn(args.tokens, H, generator=g, dtype=dtype)).cuda()
    router_logits = torch.randn(args.tokens, E, generator=g, dtype=torch.float32).cuda()
    if args.checkpoint:
        from .weights import load_qwen36_moe_weights_from_safetensors
        w = load_qwen36_moe_weights_from_safetensors(args.checkpoint, args.layer, spec=spec, device="cuda", dtype=dtype).weights
        gate_up, down = w.expert_gate_up_weight, w.expert_down_weight
    else:
        gate_up = torch.empty(E, 2 * I, H, dtype=dtype, device="cuda")
        down = torch.empty(E, H, I, dtype=dtype, device="cuda")
        for e in range(E):                                           # expert by expert: no fp32 copy of the layer
            gate_up[e] = (s * torch.randn(2 * I, H, generator=g, dtype=dtype)).cuda()
        for e in range(E):
            down[e] = (s * torch.randn(H, I, generator=g, dtype=dtype)).cuda()
    ids, weights = topk_from_logits(router_logits, k)
    want = torch_routed(hidden, ids, weights, gate_up, down)
    run = lambda: triton_qwen36_batched_routed_experts_decode(hidden, ids, weights, gate_up, down)
    ms = time_ms(run, args.iters, args.warmup)
    diff = float((run().float() - want).abs().max())
    result = {"fastkernels_routed_max_abs_diff": diff, "fastkernels_routed_moe_ms": ms}
    print(f"model: {spec.name}")
    print(f"weights: {'real' if args.checkpoint else 'random'}")
    print("device: cuda")
    print(f"dtype: {dtype}")
    print(f"tokens: {args.tokens}")
    print(f"hidden_size: {H}")
    print(f"experts: {E}")
    print(f"top_k: {k}")
    print(f"intermediate: {I}")
    print("comparison_scope: routed_experts_only")
    print(f"iters: {args.iters}")
    print(f"fastkernels_routed_max_abs_diff: {diff:.6f}")
    print(f"fastkernels_routed_moe_ms: {ms:.4f}")
    print(f"fastkernels_routed_moe_ms_per_token: {ms / args.tokens:.4f}")
    print(f"fastkernels_routed_moe_tokens_per_second: {args.tokens * 1000 / ms:.2f}")
    fused_moe, version, why = load_vllm(args.require_vllm)
    if fused_moe is None:
        print("vllm_available: False")
        print(f"vllm_import_error: {why}")
        return result
    try:
        vrun = lambda: call_vllm(fused_moe, hidden, gate_up, down, router_logits, k, ids, weights)
        vms = time_ms(vrun, args.iters, args.warmup)
        vdiff = float((vrun().float() - want).abs().max())
    except Exception as exc:  # noqa: BLE001 - the other operator's failure must not hide this library's numbers
        if args.require_vllm:
            raise
        print("vllm_available: True")
        print(f"vllm_version: {version}")
        print(f"vllm_call_failed: {exc!r}")
        return result
    print("vllm_available: True")
    print(f"vllm_version: {version}")
    print(f"vllm_routed_max_abs_diff: {vdiff:.6f}")
    print(f"vllm_routed_moe_ms: {vms:.4f}")
    print(f"vllm_routed_moe_ms_per_token: {vms / args.tokens:.4f}")
    print(f"vllm_routed_moe_tokens_per_second: {args.tokens * 1000 / vms:.2f}")
    print(f"fastkernels_to_vllm_ms_ratio: {ms / vms:.4f}")
    result.update({"vllm_routed_moe_ms": vms, "vllm_routed_max_abs_diff": vdiff})
    return result


if __name__ == "__main__":
    main()
