"""Decode loop over a stack of MoE sublayers with a switchable MoE implementation.

    python -m fastkernels_b200.decode_runner --moe-impl b200 [--layers 40] [--prompt-token-ids 0,5] [--max-new-tokens 4]

The reference's streaming runner (bench/qwen36_full_decode.py:132-545) walks the 40 layers of the real
checkpoint per position, reloading each layer's tensors from disk, and selects the MoE sublayer with
`--moe-impl {reference,triton}` (:562; call sites :407-419, :508-520).  This runner has the same loop shape
and prints the same timing keys (`elapsed_ms_per_position`, `elapsed_ms_per_layer_position`,
`layer_positions_per_second`), with what this library changes: all layers stay resident in HBM, packed once
(`ResidentMoELayers`), and `--moe-impl b200` runs the sublayer on the CUDA kernels.

Outside this library's scope and therefore stand-ins here: the sequence mixers (attention, DeltaNet) are the
identity, and without `--checkpoint` the embedding, head and layer weights are drawn from seeds (the real
checkpoint is 72 GB and not bundled).  With `--checkpoint DIR` the MoE tensors of each layer are read from
safetensors shards through `load_qwen36_moe_weights_from_safetensors`.

`--moe-impl reference` is this script's comparison arm: the layer update written with plain PyTorch ops on the
same device (the arithmetic of src/fastkernels/reference/qwen36_real.py:329-354, top-k by a stable descending
sort, ties to the lower index).  It is not part of the library's API and nothing else imports it.
"""

from __future__ import annotations

import argparse
import time
from typing import Optional, Sequence

import torch
import torch.nn.functional as F

from .spec import MoESpec, MoEWeights, synthetic_qwen36_spec
from .workloads import make_moe_weights


def torch_moe_update(hidden: torch.Tensor, w: MoEWeights, top_k: int, eps: float = 1e-6) -> torch.Tensor:
    """fp32 PyTorch form of one layer's MoE update for `hidden [T,H]` (the comparison arm of this runner)."""
    x = hidden.float()
    normed = x * torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps) * (1.0 + w.norm_weight.float())
    logits = normed @ w.router_weight.float().t()
    if w.router_bias is not None:
        logits = logits + w.router_bias.float()
    probs = torch.softmax(logits, dim=-1)
    ids = torch.sort(probs, dim=-1, descending=True, stable=True).indices[:, :top_k]
    vals = torch.gather(probs, -1, ids)
    vals = vals / vals.sum(dim=-1, keepdim=True)
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for r in range(top_k):
            e = int(ids[t, r])
            gate, up = torch.chunk(w.expert_gate_up_weight[e].float() @ x[t], 2)
            out[t] += vals[t, r] * (w.expert_down_weight[e].float() @ (F.silu(gate) * up))
        if w.shared_gate_up_weight is not None:
            gate, up = torch.chunk(w.shared_gate_up_weight.float() @ x[t], 2)
            shared = w.shared_down_weight.float() @ (F.silu(gate) * up)
            if w.shared_expert_gate_weight is not None:
                shared = shared * torch.sigmoid(w.shared_expert_gate_weight.float().reshape(-1) @ x[t])
            out[t] += shared
    return out


class DecodeRunner:
    """Embedding -> L x (mixer stand-in, hidden + MoE(hidden)) -> final norm -> head, one position at a time."""

    def __init__(self, layers: Sequence[MoEWeights], spec: MoESpec, *, moe_impl: str = "b200", vocab: int = 1024,
                 dtype: torch.dtype = torch.bfloat16, seed: int = 0, device: str = "cuda"):
        if moe_impl not in ("reference", "b200"):
            raise ValueError("moe_impl must be 'reference' or 'b200'")
        self.spec, self.moe_impl, self.dtype, self.device = spec, moe_impl, dtype, device
        self.layers = list(layers)
        g = torch.Generator(device="cpu").manual_seed(seed)
        H = spec.hidden_size
        self.embedding = torch.randn(vocab, H, generator=g).to(device=device, dtype=dtype)
        self.lm_head = (0.02 * torch.randn(vocab, H, generator=g)).to(device=device, dtype=dtype)
        self.output_norm = torch.zeros(H, device=device, dtype=dtype)
        self.resident = None
        if moe_impl == "b200":
            from .stack import ResidentMoELayers          # the CUDA library; raises if it is not built
            self.resident = ResidentMoELayers(self.layers, 1, hidden_dtype=dtype, top_k=spec.num_routed_experts)
        self.position = 0

    def step(self, token_id: int) -> torch.Tensor:
        """One position through all layers; returns the logits `[vocab]` (fp32)."""
        hidden = self.embedding[token_id].float().unsqueeze(0)
        for i, w in enumerate(self.layers):
            # the attention / DeltaNet mixer of the layer would run here (out of this library's scope: identity)
            if self.moe_impl == "reference":
                hidden = hidden + torch_moe_update(hidden.to(self.dtype), w, self.spec.num_routed_experts)
            else:
                hidden = self.resident.layer(i, hidden.to(self.dtype)).clone()
        self.position += 1
        x = hidden[0]
        normed = x * torch.rsqrt((x * x).mean() + 1e-6) * (1.0 + self.output_norm.float())
        return normed @ self.lm_head.float().t()

    def generate(self, prompt_ids: Sequence[int], max_new_tokens: int):
        logits = None
        for t in prompt_ids:
            logits = self.step(int(t))
        generated = []
        for _ in range(max_new_tokens):
            nxt = int(torch.argmax(logits).item())
            generated.append(nxt)
            logits = self.step(nxt)
        return generated, logits


def build_layers(spec: MoESpec, layers: int, dtype: torch.dtype, device: str, checkpoint: Optional[str] = None,
                 bias_std: float = 0.0):
    if checkpoint:
        from .weights import load_qwen36_moe_weights_from_safetensors
        return [load_qwen36_moe_weights_from_safetensors(checkpoint, i, spec=spec, device=device, dtype=dtype).weights
                for i in range(layers)]
    return [make_moe_weights(i, spec, dtype=dtype, device=device, bias_std=bias_std) for i in range(layers)]


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--spec", default="real", choices=["real", "tiny"])
    ap.add_argument("--layers", type=int, default=None, help="MoE layers to run (default: all of the spec)")
    ap.add_argument("--checkpoint", default=None, help="safetensors file or directory with the layers' MoE tensors")
    ap.add_argument("--prompt-token-ids", default="0")
    ap.add_argument("--max-new-tokens", type=int, default=1)
    ap.add_argument("--moe-impl", default="b200", choices=["reference", "b200"])
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args(argv)
    dtype = getattr(torch, args.dtype)
    spec = MoESpec() if args.spec == "real" else synthetic_qwen36_spec()
    n_layers = args.layers or spec.num_layers
    prompt = [int(t) for t in args.prompt_token_ids.split(",") if t.strip()]
    if not prompt:
        raise ValueError("prompt must contain at least one token")
    layers = build_layers(spec, n_layers, dtype, args.device, args.checkpoint)
    runner = DecodeRunner(layers, spec, moe_impl=args.moe_impl, dtype=dtype, seed=args.seed, device=args.device)
    runner.step(prompt[0])                 # warm-up position (kernel attributes, tensor maps); not timed
    runner.position = 0
    if args.device == "cuda":
        torch.cuda.synchronize()
    start = time.perf_counter()
    generated, _ = runner.generate(prompt, args.max_new_tokens)
    if args.device == "cuda":
        torch.cuda.synchronize()
    elapsed = time.perf_counter() - start
    positions = runner.position
    layer_positions = n_layers * positions
    print(f"model: {spec.name}")
    print(f"weights: {'checkpoint ' + args.checkpoint if args.checkpoint else 'seeded synthetic (layer index = seed)'}")
    print(f"device: {args.device}")
    print(f"dtype: {dtype}")
    print(f"layers_total: {spec.num_layers}")
    print(f"layers_executed: {n_layers}")
    print(f"prompt_tokens: {len(prompt)}")
    print(f"generated_tokens: {len(generated)}")
    print(f"generated_token_ids: {','.join(str(t) for t in generated)}")
    print(f"final_position: {positions}")
    print(f"elapsed_seconds: {elapsed:.4f}")
    print(f"elapsed_ms_per_position: {elapsed * 1000 / max(positions, 1):.4f}")
    print(f"elapsed_ms_per_layer_position: {elapsed * 1000 / max(layer_positions, 1):.4f}")
    print(f"layer_positions_per_second: {layer_positions / elapsed:.4f}")
    print("attention_impl: identity (out of scope)")
    print("deltanet_impl: identity (out of scope)")
    print(f"moe_impl: {args.moe_impl}")
    print("serving_scope: MoE sublayers of the decode loop with resident weights; sequence mixers are stand-ins")


if __name__ == "__main__":
    main()
