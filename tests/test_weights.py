"""Checkpoint -> kernel layout packing (host logic, CPU).

Cases follow the reference's packing tests (tests/test_qwen36_spec.py:195-307: split per-expert
projections, the released grouped layout with a [1,H] shared gate) and add the transposed grouped
orientation, per-expert packed gate_up, shard packing, conversion while packing and the error paths.
"""

import pytest
import torch

from fastkernels_b200.spec import MoESpec, synthetic_qwen36_spec
from fastkernels_b200.weights import (pack_qwen36_moe_weights_from_state_dict, resolve_qwen36_moe_weight_keys,
                                      state_dict_from_moe_weights)
from fastkernels_b200.workloads import make_moe_weights

SPEC = synthetic_qwen36_spec()
H, E, I = SPEC.hidden_size, SPEC.num_experts, SPEC.expert_intermediate_size


def split_checkpoint(layer=0, prefix="model.layers", gate=False):
    t = {f"{prefix}.{layer}.post_attention_layernorm.weight": torch.arange(H, dtype=torch.float32),
         f"{prefix}.{layer}.mlp.gate.weight": torch.arange(E * H, dtype=torch.float32).reshape(E, H),
         f"{prefix}.{layer}.mlp.shared_expert.gate_proj.weight": torch.full((I, H), 3.0),
         f"{prefix}.{layer}.mlp.shared_expert.up_proj.weight": torch.full((I, H), 4.0),
         f"{prefix}.{layer}.mlp.shared_expert.down_proj.weight": torch.full((H, I), 5.0)}
    for e in range(E):
        t[f"{prefix}.{layer}.mlp.experts.{e}.gate_proj.weight"] = torch.full((I, H), float(e + 1))
        t[f"{prefix}.{layer}.mlp.experts.{e}.up_proj.weight"] = torch.full((I, H), float(e + 11))
        t[f"{prefix}.{layer}.mlp.experts.{e}.down_proj.weight"] = torch.full((H, I), float(e + 21))
    if gate:
        t[f"{prefix}.{layer}.mlp.shared_expert_gate.weight"] = torch.full((1, H), 0.5)
    return t


def test_split_layout_gate_rows_then_up_rows():
    t = split_checkpoint()
    packed = pack_qwen36_moe_weights_from_state_dict(t, 0, spec=SPEC)
    w = packed.weights
    assert w.norm_weight.shape == (H,) and w.router_weight.shape == (E, H)
    assert w.expert_gate_up_weight.shape == (E, 2 * I, H) and w.expert_down_weight.shape == (E, H, I)
    for e in range(E):
        assert torch.equal(w.expert_gate_up_weight[e, :I], torch.full((I, H), float(e + 1)))
        assert torch.equal(w.expert_gate_up_weight[e, I:], torch.full((I, H), float(e + 11)))
        assert torch.equal(w.expert_down_weight[e], torch.full((H, I), float(e + 21)))
    assert torch.equal(w.shared_gate_up_weight[:I], torch.full((I, H), 3.0))
    assert torch.equal(w.shared_gate_up_weight[I:], torch.full((I, H), 4.0))
    assert w.shared_expert_gate_weight is None
    assert packed.expert_range == (0, E)
    for x in (w.norm_weight, w.router_weight, w.expert_gate_up_weight, w.expert_down_weight, w.shared_gate_up_weight,
              w.shared_down_weight):
        assert x.is_contiguous()


@pytest.mark.parametrize("transposed", [False, True])
def test_grouped_layout_either_orientation(transposed):
    # 2I != H here, so that the two orientations of gate_up can be told apart by shape (when they cannot, the
    # tensor is taken as stored, like the reference does)
    spec = MoESpec(hidden_size=24, num_experts=4, num_routed_experts=2, expert_intermediate_size=8, num_layers=4)
    h, e_, i = spec.hidden_size, spec.num_experts, spec.expert_intermediate_size
    base = "model.language_model.layers.2"
    gu = torch.arange(e_ * 2 * i * h, dtype=torch.float32).reshape(e_, 2 * i, h)
    dn = torch.arange(e_ * h * i, dtype=torch.float32).reshape(e_, h, i)
    t = {f"{base}.post_attention_layernorm.weight": torch.arange(h, dtype=torch.float32),
         f"{base}.mlp.gate.weight": torch.zeros(e_, h),
         f"{base}.mlp.experts.gate_up_proj": gu.transpose(1, 2).contiguous() if transposed else gu,
         f"{base}.mlp.experts.down_proj": dn.transpose(1, 2).contiguous() if transposed else dn,
         f"{base}.mlp.shared_expert.gate_proj.weight": torch.full((i, h), 3.0),
         f"{base}.mlp.shared_expert.up_proj.weight": torch.full((i, h), 4.0),
         f"{base}.mlp.shared_expert.down_proj.weight": torch.full((h, i), 5.0),
         f"{base}.mlp.shared_expert_gate.weight": torch.full((1, h), 0.5)}
    keys = resolve_qwen36_moe_weight_keys(t, 2, spec=spec)
    assert keys.expert_gate_up_weight == f"{base}.mlp.experts.gate_up_proj"
    assert keys.expert_down_weight == f"{base}.mlp.experts.down_proj"
    assert keys.shared_expert_gate_weight == f"{base}.mlp.shared_expert_gate.weight"
    w = pack_qwen36_moe_weights_from_state_dict(t, 2, spec=spec).weights
    assert torch.equal(w.expert_gate_up_weight, gu) and torch.equal(w.expert_down_weight, dn)
    assert w.expert_gate_up_weight.is_contiguous() and w.expert_down_weight.is_contiguous()
    assert w.shared_expert_gate_weight.shape == (1, h)


def test_per_expert_packed_gate_up_and_alternative_names():
    t = split_checkpoint(layer=1, prefix="layers")
    for e in range(E):
        g = t.pop(f"layers.1.mlp.experts.{e}.gate_proj.weight")
        u = t.pop(f"layers.1.mlp.experts.{e}.up_proj.weight")
        t[f"layers.1.mlp.experts.{e}.w1.weight"] = torch.cat((g, u), dim=0)
        t[f"layers.1.mlp.experts.{e}.w2.weight"] = t.pop(f"layers.1.mlp.experts.{e}.down_proj.weight")
    t["layers.1.mlp.router.weight"] = t.pop("layers.1.mlp.gate.weight")
    w = pack_qwen36_moe_weights_from_state_dict(t, 1, spec=SPEC).weights
    ref = pack_qwen36_moe_weights_from_state_dict(split_checkpoint(), 0, spec=SPEC).weights
    for a, b in zip(w.tuple()[:6], ref.tuple()[:6]):
        assert torch.equal(a, b)


@pytest.mark.parametrize("grouped", [True, False])
def test_round_trip_shard_and_conversion(grouped):
    full = make_moe_weights(3, SPEC, dtype=torch.float32)
    ckpt = state_dict_from_moe_weights(full, 5, grouped=grouped)
    back = pack_qwen36_moe_weights_from_state_dict(ckpt, 5, spec=SPEC).weights
    for a, b in zip(back.tuple(), full.tuple()):
        assert torch.equal(a, b)
    # a shard holds its block only, and is what slicing the full layer gives
    shard = pack_qwen36_moe_weights_from_state_dict(ckpt, 5, spec=SPEC, expert_range=(1, 3), dtype=torch.bfloat16)
    assert shard.expert_range == (1, 3)
    assert shard.weights.expert_gate_up_weight.shape == (2, 2 * I, H)
    assert shard.weights.expert_gate_up_weight.dtype == torch.bfloat16
    assert torch.equal(shard.weights.expert_gate_up_weight, full.expert_gate_up_weight[1:3].to(torch.bfloat16))
    assert torch.equal(shard.weights.expert_down_weight, full.expert_down_weight[1:3].to(torch.bfloat16))
    assert torch.equal(shard.weights.router_weight, full.router_weight.to(torch.bfloat16))


def test_shard_never_reads_foreign_experts():
    class Recording(dict):
        def __init__(self, *a):
            super().__init__(*a)
            self.read = []

        def __getitem__(self, k):
            self.read.append(k)
            return super().__getitem__(k)

    t = Recording(split_checkpoint())
    pack_qwen36_moe_weights_from_state_dict(t, 0, spec=SPEC, expert_range=(2, 4))
    touched = {k for k in t.read if ".experts." in k}
    assert touched and all(".experts.2." in k or ".experts.3." in k for k in touched)


def test_errors():
    t = split_checkpoint()
    del t["model.layers.0.mlp.experts.2.up_proj.weight"]
    with pytest.raises(KeyError, match="expert 2 up projection"):
        pack_qwen36_moe_weights_from_state_dict(t, 0, spec=SPEC)
    t = split_checkpoint()
    t["model.layers.0.mlp.experts.1.down_proj.weight"] = torch.zeros(H, I + 1)
    with pytest.raises(ValueError, match="expected"):
        pack_qwen36_moe_weights_from_state_dict(t, 0, spec=SPEC)
    t = split_checkpoint(gate=True)
    t["model.layers.0.mlp.shared_expert_gate.weight"] = torch.zeros(2, H)
    with pytest.raises(ValueError, match="expected"):
        pack_qwen36_moe_weights_from_state_dict(t, 0, spec=SPEC)
    with pytest.raises(KeyError, match="MoE input norm weight"):
        pack_qwen36_moe_weights_from_state_dict(split_checkpoint(), 7, spec=SPEC)
    with pytest.raises(ValueError, match="expert_range"):
        pack_qwen36_moe_weights_from_state_dict(split_checkpoint(), 0, spec=SPEC, expert_range=(3, 9))


def _two_shard_checkpoint(tmp_path, spec, layer=0):
    """The fake checkpoint of the reference's loader test (tests/test_qwen36_spec.py:544-606): norm and router in
    the first shard, split per-expert and shared-expert projections in the second, an index that maps the names."""
    import json
    safetensors = pytest.importorskip("safetensors.torch")
    H, E, I = spec.hidden_size, spec.num_experts, spec.expert_intermediate_size
    shard_a = {f"model.layers.{layer}.post_attention_layernorm.weight": torch.arange(H, dtype=torch.float32),
               f"model.layers.{layer}.mlp.gate.weight": torch.arange(E * H, dtype=torch.float32).reshape(E, H)}
    shard_b = {f"model.layers.{layer}.mlp.shared_expert.gate_proj.weight": torch.full((I, H), 3.0),
               f"model.layers.{layer}.mlp.shared_expert.up_proj.weight": torch.full((I, H), 4.0),
               f"model.layers.{layer}.mlp.shared_expert.down_proj.weight": torch.full((H, I), 5.0)}
    for e in range(E):
        shard_b[f"model.layers.{layer}.mlp.experts.{e}.gate_proj.weight"] = torch.full((I, H), float(e + 1))
        shard_b[f"model.layers.{layer}.mlp.experts.{e}.up_proj.weight"] = torch.full((I, H), float(e + 11))
        shard_b[f"model.layers.{layer}.mlp.experts.{e}.down_proj.weight"] = torch.full((H, I), float(e + 21))
    safetensors.save_file(shard_a, str(tmp_path / "model-00001-of-00002.safetensors"))
    safetensors.save_file(shard_b, str(tmp_path / "model-00002-of-00002.safetensors"))
    weight_map = {key: "model-00001-of-00002.safetensors" for key in shard_a}
    weight_map.update({key: "model-00002-of-00002.safetensors" for key in shard_b})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": weight_map}), encoding="utf-8")
    return shard_a, shard_b


def test_loader_uses_the_safetensors_index(tmp_path):
    from fastkernels_b200.weights import load_qwen36_moe_weights_from_safetensors
    spec = synthetic_qwen36_spec()
    H, E, I = spec.hidden_size, spec.num_experts, spec.expert_intermediate_size
    shard_a, shard_b = _two_shard_checkpoint(tmp_path, spec)
    packed = load_qwen36_moe_weights_from_safetensors(tmp_path, 0, spec=spec).weights
    assert packed.expert_gate_up_weight.shape == (E, 2 * I, H)
    torch.testing.assert_close(packed.expert_gate_up_weight[1, :I], shard_b["model.layers.0.mlp.experts.1.gate_proj.weight"])
    torch.testing.assert_close(packed.expert_gate_up_weight[1, I:], shard_b["model.layers.0.mlp.experts.1.up_proj.weight"])
    torch.testing.assert_close(packed.shared_gate_up_weight[I:], shard_b["model.layers.0.mlp.shared_expert.up_proj.weight"])
    torch.testing.assert_close(packed.expert_down_weight[2], shard_b["model.layers.0.mlp.experts.2.down_proj.weight"])
    torch.testing.assert_close(packed.router_weight, shard_a["model.layers.0.mlp.gate.weight"])
    assert packed.shared_expert_gate_weight is None
    # a rank's shard and a compute dtype, without touching the other experts
    part = load_qwen36_moe_weights_from_safetensors(tmp_path, 0, spec=spec, expert_range=(1, 3), dtype=torch.bfloat16)
    assert part.expert_range == (1, 3) and part.weights.expert_down_weight.shape == (2, H, I)
    assert part.weights.expert_down_weight.dtype == torch.bfloat16
    torch.testing.assert_close(part.weights.expert_down_weight[0].float(), torch.full((H, I), 22.0))


def test_loader_without_an_index_and_its_errors(tmp_path):
    import json
    from fastkernels_b200.weights import load_qwen36_moe_weights_from_safetensors
    spec = synthetic_qwen36_spec()
    with pytest.raises(FileNotFoundError):
        load_qwen36_moe_weights_from_safetensors(tmp_path, 0, spec=spec)
    _two_shard_checkpoint(tmp_path, spec)
    index = tmp_path / "model.safetensors.index.json"
    kept = json.loads(index.read_text())
    # every *.safetensors file of the directory when there is no index
    index.unlink()
    packed = load_qwen36_moe_weights_from_safetensors(tmp_path, 0, spec=spec).weights
    assert packed.expert_down_weight.shape[0] == spec.num_experts
    # an index whose weight map is not a mapping
    index.write_text(json.dumps({"weight_map": []}), encoding="utf-8")
    with pytest.raises(ValueError, match="weight_map"):
        load_qwen36_moe_weights_from_safetensors(tmp_path, 0, spec=spec)
    # an index that lacks a tensor of the layer
    del kept["weight_map"]["model.layers.0.mlp.experts.3.down_proj.weight"]
    index.write_text(json.dumps(kept), encoding="utf-8")
    with pytest.raises(KeyError):
        load_qwen36_moe_weights_from_safetensors(tmp_path, 0, spec=spec)
