"""Pin `oracle/moe_oracle.py` against the reference's own Python functions and write golden vectors.

TEST INFRASTRUCTURE.  Run in a container that has the reference checkout:

    python oracle/pin_against_reference.py --reference /path/to/fastkernels [--write]

It imports `fastkernels.reference` from `<reference>/src`, runs reference and
oracle on the same seeded inputs, asserts agreement, and (with --write) stores
the REFERENCE's outputs under tests/golden/*.npz.  Inputs are regenerated from
seeds by `fastkernels_b200.workloads`; each file carries a checksum of the inputs so
a drift of the random generator is detected instead of silently mis-compared.
The golden files are replayed by tests/test_oracle_golden.py (CPU) and by the
GPU parity tests, neither of which needs the reference tree.
"""

from __future__ import annotations

import argparse
import hashlib
import os
import sys
from dataclasses import replace
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

from oracle import moe_oracle as O                      # noqa: E402
from fastkernels_b200.spec import MoESpec                  # noqa: E402
from fastkernels_b200.workloads import make_hidden, make_moe_weights  # noqa: E402

GOLDEN = ROOT / "tests" / "golden"

CASES = {
    # name: (spec, tokens, dtype, seed, bias_std)
    "tiny_fp32": (MoESpec(hidden_size=16, num_experts=4, num_routed_experts=2, expert_intermediate_size=8), 3,
                  torch.float32, 11, 0.0),
    "medium_bf16": (MoESpec(hidden_size=256, num_experts=32, num_routed_experts=8, expert_intermediate_size=64), 8,
                    torch.bfloat16, 12, 0.5),
    "odd_fp32": (MoESpec(hidden_size=200, num_experts=24, num_routed_experts=5, expert_intermediate_size=72), 5,
                 torch.float32, 13, 0.0),
    "real16_bf16": (MoESpec(hidden_size=2048, num_experts=16, num_routed_experts=8, expert_intermediate_size=512), 4,
                    torch.bfloat16, 14, 0.0),
    # the full layer shape (H 2048, E 256, I 512, top-8); outputs come from qwen36_real_moe_update itself
    "real_full_fp32_1tok": (MoESpec(), 1, torch.float32, 31, 0.0),       # benchmark configuration 1: fp32, one token
    "real_full_bf16_4tok": (MoESpec(), 4, torch.bfloat16, 32, 0.0),
    # one case per kernel family of the CUDA library at the full shape: single-token launch, few-token launch,
    # streaming kernels (the default benchmark batch), grouped tensor-core GEMM
    "real_full_bf16_1tok": (MoESpec(), 1, torch.bfloat16, 33, 0.0),
    "real_full_bf16_2tok": (MoESpec(), 2, torch.bfloat16, 34, 0.0),
    "real_full_bf16_32tok": (MoESpec(), 32, torch.bfloat16, 35, 0.0),
    "real_full_bf16_64tok": (MoESpec(), 64, torch.bfloat16, 36, 0.0),
}
ROUTER_CASES = {
    # full-shape router (E=256, H=2048), several tokens
    "router_real_bf16": (16, torch.bfloat16, 21),
    "router_real_fp32": (4, torch.float32, 22),
}


def checksum(*tensors) -> str:
    h = hashlib.sha256()
    for t in tensors:
        if t is None:
            h.update(b"none")
        else:
            h.update(t.detach().contiguous().view(torch.uint8).numpy().tobytes())
    return h.hexdigest()


def load_reference(path: str):
    sys.path.insert(0, os.path.join(path, "src"))
    sys.dont_write_bytecode = True
    import fastkernels.reference as R
    from fastkernels.reference.qwen36_real import qwen36_real_rms_norm
    from fastkernels.models import Qwen36MoEWeights, qwen36_35b_a3b_spec, synthetic_qwen36_spec
    from fastkernels.reference import make_synthetic_qwen36_decode_weights
    return R, qwen36_real_rms_norm, Qwen36MoEWeights, qwen36_35b_a3b_spec, synthetic_qwen36_spec, \
        make_synthetic_qwen36_decode_weights


def pin_weight_packer(reference_path: str) -> None:
    """`fastkernels_b200.weights` against the reference's packer on synthetic checkpoints: same keys chosen,
    same tensors out, for the split, per-expert packed and grouped (both orientations) layouts."""
    import importlib
    rw = importlib.import_module("fastkernels.models.qwen36_weights")
    rq = importlib.import_module("fastkernels.models.qwen36")
    from fastkernels_b200.weights import (pack_qwen36_moe_weights_from_state_dict, resolve_qwen36_moe_weight_keys,
                                          state_dict_from_moe_weights)
    rspec = rq.synthetic_qwen36_spec()
    spec = MoESpec(hidden_size=rspec.hidden_size, num_experts=rspec.num_experts, num_routed_experts=rspec.num_routed_experts,
                   expert_intermediate_size=rspec.expert_intermediate_size)
    full = make_moe_weights(21, spec, dtype=torch.float32)
    variants = {"grouped": state_dict_from_moe_weights(full, 3, grouped=True),
                "split": state_dict_from_moe_weights(full, 3, grouped=False, prefix="model.layers")}
    flipped = dict(variants["grouped"])
    k = "model.language_model.layers.3.mlp.experts.down_proj"
    flipped[k] = flipped[k].transpose(1, 2).contiguous()
    variants["grouped, down stored [E,I,H]"] = flipped
    packed = {kk: v for kk, v in variants["split"].items() if ".experts." not in kk}
    for e in range(spec.num_experts):
        packed[f"model.layers.3.mlp.experts.{e}.gate_up_proj.weight"] = full.expert_gate_up_weight[e]
        packed[f"model.layers.3.mlp.experts.{e}.down_proj.weight"] = full.expert_down_weight[e]
    variants["per-expert packed"] = packed
    fields = ("norm_weight", "router_weight", "expert_gate_up_weight", "expert_down_weight",
              "shared_gate_up_weight", "shared_down_weight", "shared_expert_gate_weight")
    for name, ckpt in variants.items():
        ref_keys = rw.resolve_qwen36_moe_weight_keys(ckpt, 3, spec=rspec)
        ours_keys = resolve_qwen36_moe_weight_keys(ckpt, 3, spec=spec)
        for field in fields:
            assert getattr(ref_keys, field) == getattr(ours_keys, field), (name, field)
        ref = rw.pack_qwen36_moe_weights_from_state_dict(ckpt, 3, spec=rspec)
        ours = pack_qwen36_moe_weights_from_state_dict(ckpt, 3, spec=spec).weights
        for field in fields:
            a, b = getattr(ref, field), getattr(ours, field)
            assert (a is None) == (b is None) and (a is None or torch.equal(a, b)), (name, field)
        print(f"pinned: weight packer [{name}] keys and tensors equal the reference packer's")

    # the safetensors loader on a two-shard checkpoint with an index (the reference's own loader test layout,
    # tests/test_qwen36_spec.py:544-606) and on the same directory without the index
    import json
    import tempfile
    from safetensors.torch import save_file
    from fastkernels_b200.weights import load_qwen36_moe_weights_from_safetensors
    ckpt = variants["split"]
    names = sorted(ckpt)
    with tempfile.TemporaryDirectory() as tmp:
        halves = {"model-00001-of-00002.safetensors": names[: len(names) // 2], "model-00002-of-00002.safetensors": names[len(names) // 2:]}
        for fname, ks in halves.items():
            save_file({k: ckpt[k].contiguous() for k in ks}, os.path.join(tmp, fname))
        index = os.path.join(tmp, "model.safetensors.index.json")
        with open(index, "w", encoding="utf-8") as f:
            json.dump({"metadata": {}, "weight_map": {k: fname for fname, ks in halves.items() for k in ks}}, f)
        for how in ("with index", "without index"):
            if how == "without index":
                os.remove(index)
            ref = rw.load_qwen36_moe_weights_from_safetensors(tmp, 3, spec=rspec)
            ours = load_qwen36_moe_weights_from_safetensors(tmp, 3, spec=spec).weights
            for field in fields:
                a, b = getattr(ref, field), getattr(ours, field)
                assert (a is None) == (b is None) and (a is None or torch.equal(a, b)), (how, field)
            print(f"pinned: safetensors loader [{how}] tensors equal the reference loader's")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout")
    ap.add_argument("--write", action="store_true")
    args = ap.parse_args()
    R, ref_rms, RefWeights, ref_real_spec, ref_tiny_spec, ref_make_tiny = load_reference(args.reference)
    torch.set_num_threads(os.cpu_count() or 1)
    GOLDEN.mkdir(parents=True, exist_ok=True)

    # 1. RMSNorm, swiglu, histogram: oracle == reference on random inputs.
    g = torch.Generator().manual_seed(1)
    x = torch.randn(5, 64, generator=g)
    w = 0.1 * torch.randn(64, generator=g)
    assert torch.equal(O.rms_norm(x, w), ref_rms(x, w))
    gu = torch.randn(7, 32, generator=g)
    assert torch.equal(O.fused_swiglu(gu), R.reference_fused_swiglu(gu))
    ids = torch.randint(0, 256, (64, 8), generator=g)
    assert torch.equal(O.expert_histogram(ids, 256), R.reference_expert_histogram(ids, 256))
    cnt, off, order = O.expert_permutation(ids, 256)
    flat = ids.flatten()
    assert torch.equal(flat[order.long()], torch.sort(flat).values) and int(off[-1]) == flat.numel()
    print("pinned: rms_norm, fused_swiglu, expert_histogram (bit-exact)")

    # 2. whole MoE update on each case: oracle vs qwen36_real_moe_update (no bias: the reference
    #    function has no bias argument) and vs reference_routed_moe + shared path (bias cases).
    for name, (spec, tokens, dtype, seed, bias_std) in CASES.items():
        wts = make_moe_weights(seed, spec, dtype=dtype, bias_std=bias_std)
        hidden = make_hidden(seed, tokens, spec, dtype=dtype)
        ref_spec = replace(ref_real_spec(), hidden_size=spec.hidden_size, num_experts=spec.num_experts,
                           num_routed_experts=spec.num_routed_experts,
                           expert_intermediate_size=spec.expert_intermediate_size)
        rw = RefWeights(wts.norm_weight, wts.router_weight, wts.expert_gate_up_weight, wts.expert_down_weight,
                        wts.shared_gate_up_weight, wts.shared_down_weight, keys=None,
                        shared_expert_gate_weight=wts.shared_expert_gate_weight)
        res = O.moe_update(hidden, *wts.tuple(), top_k=spec.num_routed_experts, router_bias=wts.router_bias)
        if wts.router_bias is None:
            ref_out = R.qwen36_real_moe_update(hidden, rw, ref_spec)
        else:
            logits = ref_rms(hidden.float(), wts.norm_weight) @ wts.router_weight.float().t() + wts.router_bias
            routed = R.reference_routed_moe(hidden.float(), logits, wts.expert_gate_up_weight.float(),
                                            wts.expert_down_weight.float(), top_k=spec.num_routed_experts)
            ref_out = routed + O.shared_expert(hidden, wts.shared_gate_up_weight, wts.shared_down_weight,
                                               wts.shared_expert_gate_weight)
        # reference ids via torch.topk on the same logits (distinct probabilities => same as the oracle)
        ref_logits = ref_rms(hidden.float(), wts.norm_weight) @ wts.router_weight.float().t()
        if wts.router_bias is not None:
            ref_logits = ref_logits + wts.router_bias
        pv, pi = torch.topk(torch.softmax(ref_logits, -1), k=spec.num_routed_experts, dim=-1)
        assert torch.equal(pi, res.topk_ids), name
        assert torch.equal(res.logits, ref_logits), name
        torch.testing.assert_close(res.topk_weights, pv / pv.sum(-1, keepdim=True), atol=0, rtol=0)
        err = O.max_abs(res.output, ref_out)
        assert err <= 2e-6 * max(1.0, float(ref_out.abs().max())), (name, err)
        print(f"pinned: moe_update[{name}] max_abs vs reference {err:.3e}; ids/logits/weights bit-exact")
        if args.write:
            np.savez_compressed(
                GOLDEN / f"moe_{name}.npz",
                inputs_sha256=checksum(hidden, *wts.tuple(), wts.router_bias),
                output=ref_out.numpy(), logits=ref_logits.numpy(), topk_ids=pi.numpy(),
                topk_weights=(pv / pv.sum(-1, keepdim=True)).numpy(),
                histogram=R.reference_expert_histogram(pi, spec.num_experts).numpy(),
                margin=res.margin.numpy())

    # 3. full-shape router: logits / ids / weights.
    real = MoESpec()
    for name, (tokens, dtype, seed) in ROUTER_CASES.items():
        g = torch.Generator().manual_seed(seed)
        hidden = torch.randn(tokens, real.hidden_size, generator=g).to(dtype)
        norm_w = (0.02 * torch.randn(real.hidden_size, generator=g)).to(dtype)
        router_w = (0.02 * torch.randn(real.num_experts, real.hidden_size, generator=g)).to(dtype)
        ref_logits = ref_rms(hidden.float(), norm_w) @ router_w.float().t()
        pv, pi = torch.topk(torch.softmax(ref_logits, -1), k=8, dim=-1)
        lg, ids_o, w_o = O.router(hidden, norm_w, router_w, top_k=8)
        assert torch.equal(lg, ref_logits) and torch.equal(ids_o, pi)
        print(f"pinned: router[{name}] bit-exact")
        if args.write:
            srt = torch.sort(torch.softmax(ref_logits, -1), dim=-1, descending=True).values
            np.savez_compressed(GOLDEN / f"{name}.npz", inputs_sha256=checksum(hidden, norm_w, router_w),
                                logits=ref_logits.numpy(), topk_ids=pi.numpy(),
                                topk_weights=(pv / pv.sum(-1, keepdim=True)).numpy(),
                                margin=(srt[:, 7] - srt[:, 8]).numpy())

    # 4. tiny synthetic block with residual (reference_qwen36_moe_decode), weights from the
    #    reference's own seeded generator; inputs are stored inline (they are tiny).
    tiny = ref_tiny_spec()
    layers = ref_make_tiny(tiny, seed=0)
    layer = next(l for l in layers["layers"] if "router_weight" in l) if isinstance(layers, dict) else layers[0]
    g = torch.Generator().manual_seed(5)
    hidden = torch.randn(tiny.hidden_size, generator=g)
    ref = R.reference_qwen36_moe_decode(hidden, layer, tiny)
    mine = O.synthetic_moe_decode(hidden, layer["norm_weight"], layer["router_weight"],
                                  layer["expert_gate_up_weight"], layer["expert_down_weight"],
                                  layer["shared_gate_up_weight"], layer["shared_down_weight"],
                                  top_k=tiny.num_routed_experts)
    assert O.max_abs(mine, ref) < 1e-6
    print(f"pinned: synthetic_moe_decode max_abs {O.max_abs(mine, ref):.2e}")
    if args.write:
        np.savez_compressed(GOLDEN / "synthetic_tiny.npz", hidden=hidden.numpy(), output=ref.numpy(),
                            **{k: layer[k].numpy() for k in ("norm_weight", "router_weight", "expert_gate_up_weight",
                                                             "expert_down_weight", "shared_gate_up_weight",
                                                             "shared_down_weight")})
    pin_weight_packer(args.reference)
    print("all pins hold" + ("; golden vectors written" if args.write else ""))


if __name__ == "__main__":
    main()
