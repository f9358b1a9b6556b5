"""Checkpoint tensors -> the kernel-facing layout of one MoE layer.

Host-side counterpart of the reference's `resolve_qwen36_moe_weight_keys` and
`pack_qwen36_moe_weights_from_state_dict` (src/fastkernels/models/qwen36_weights.py:161-357,
:416-527): the same tensor names are recognised (per-expert split projections, per-expert
packed gate_up, grouped `[E, ...]` tensors in either orientation, shared expert split or
packed, optional shared gate), the same shapes are enforced with `ValueError`, a missing
tensor is a `KeyError` that lists what was tried, and the result has the layout the kernels
stream: `gate_up [E, 2I, H]` with an expert's gate rows first and its up rows after them,
`down [E, H, I]`, every tensor row-major contiguous.

Two things go beyond the reference, both for memory laid out per GPU:
* `expert_range=(lo, hi)` packs only that block of routed experts (an expert-parallel shard);
  the other experts' tensors are never read, so a rank never holds more than its slice;
* `dtype` / `device` convert while packing, expert by expert, so a bf16 layer (1.6 GB) is built
  on the GPU without an fp32 or host copy of the whole layer.

The function takes any mapping of names to tensors (a `state_dict`, or a lazily loading
safetensors view): tensors are fetched one at a time with `tensors[key]`.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Sequence, Union

import torch

from .spec import MoESpec, MoEWeights, qwen36_35b_a3b_spec

DEFAULT_LAYER_PREFIXES = (
    "model.layers",
    "model.language_model.layers",
    "language_model.model.layers",
    "transformer.layers",
    "layers",
)

# suffixes in the order they are tried (first hit wins), below "<prefix>.<layer>."
_NORM = ("post_attention_layernorm.weight", "pre_feedforward_layernorm.weight", "mlp_norm.weight",
         "input_layernorm.weight")
_ROUTER = ("mlp.gate.weight", "mlp.router.weight", "mlp.router.linear.weight")
_GROUPED_GATE_UP = ("gate_up_proj", "gate_up_proj.weight", "gate_up", "gate_up.weight", "w1", "w1.weight")
_GROUPED_DOWN = ("down_proj", "down_proj.weight", "down", "down.weight", "w2", "w2.weight")
_PACKED_GATE_UP = ("gate_up_proj.weight", "gate_up.weight", "w1.weight")
_GATE = ("gate_proj.weight", "gate.weight", "w1_gate.weight")
_UP = ("up_proj.weight", "up.weight", "w1_up.weight")
_DOWN = ("down_proj.weight", "down.weight", "w2.weight")
_SHARED = ("shared_expert", "shared_experts.0")

GateUpKey = Union[str, tuple]          # one packed tensor, or (gate, up)


@dataclass(frozen=True)
class MoEWeightKeys:
    """Names of the tensors one layer is packed from.

    `expert_gate_up_weight` is a single name when the checkpoint stores all experts in one
    grouped tensor, else one entry per expert: a name (packed gate_up) or a (gate, up) pair.
    `expert_down_weight` is a single name or one name per expert.
    """

    norm_weight: str
    router_weight: str
    expert_gate_up_weight: Union[str, tuple]
    expert_down_weight: Union[str, tuple]
    shared_gate_up_weight: GateUpKey
    shared_down_weight: str
    shared_expert_gate_weight: Optional[str] = None


def _bases(layer_idx: int, prefixes: Sequence[str]) -> list:
    return [f"{p}.{layer_idx}" if p else str(layer_idx) for p in prefixes]


def _find(tensors: Mapping[str, Any], candidates: Sequence[str]) -> Optional[str]:
    for key in candidates:
        if key in tensors:
            return key
    return None


def _need(tensors: Mapping[str, Any], candidates: Sequence[str], what: str) -> str:
    key = _find(tensors, candidates)
    if key is None:
        shown = "\n  ".join(list(candidates)[:16])
        raise KeyError(f"missing {what}; tried:\n  {shown}")
    return key


def resolve_qwen36_moe_weight_keys(tensors: Mapping[str, Any], layer_idx: int, *, spec: Optional[MoESpec] = None,
                                   layer_prefixes: Sequence[str] = DEFAULT_LAYER_PREFIXES) -> MoEWeightKeys:
    """Find the tensor names of one MoE layer (reference: qwen36_weights.py:161-357)."""
    spec = spec or qwen36_35b_a3b_spec()
    bases = _bases(layer_idx, layer_prefixes)

    def under(middle: str, suffixes: Sequence[str]) -> list:
        return [f"{b}.{middle}{s}" for b in bases for s in suffixes]

    norm = _need(tensors, under("", _NORM), "MoE input norm weight")
    router = _need(tensors, under("", _ROUTER), "router weight")

    grouped_gu = _find(tensors, under("mlp.experts.", _GROUPED_GATE_UP))
    grouped_dn = _find(tensors, under("mlp.experts.", _GROUPED_DOWN))
    if grouped_gu is not None and grouped_dn is not None:
        gate_up: Union[str, tuple] = grouped_gu
        down: Union[str, tuple] = grouped_dn
    else:
        gu_list, dn_list = [], []
        for e in range(spec.num_experts):
            mid = f"mlp.experts.{e}."
            packed = _find(tensors, under(mid, _PACKED_GATE_UP))
            if packed is not None:
                gu_list.append(packed)
            else:
                gu_list.append((_need(tensors, under(mid, _GATE), f"expert {e} gate projection"),
                                _need(tensors, under(mid, _UP), f"expert {e} up projection")))
            dn_list.append(_need(tensors, under(mid, _DOWN), f"expert {e} down projection"))
        gate_up, down = tuple(gu_list), tuple(dn_list)

    def shared(suffixes: Sequence[str]) -> list:
        return [f"{b}.mlp.{name}.{s}" for b in bases for name in _SHARED for s in suffixes]

    shared_packed = _find(tensors, shared(_PACKED_GATE_UP))
    if shared_packed is not None:
        shared_gu: GateUpKey = shared_packed
    else:
        shared_gu = (_need(tensors, shared(_GATE), "shared expert gate projection"),
                     _need(tensors, shared(_UP), "shared expert up projection"))
    shared_dn = _need(tensors, shared(_DOWN), "shared expert down projection")
    shared_gate = _find(tensors, [f"{b}.mlp.shared_expert_gate.weight" for b in bases])
    return MoEWeightKeys(norm, router, gate_up, down, shared_gu, shared_dn, shared_gate)


def _shape(t) -> tuple:
    return tuple(int(d) for d in t.shape)


def _expect(name: str, t, shape: tuple) -> None:
    if _shape(t) != tuple(shape):
        raise ValueError(f"{name} has shape {_shape(t)}, expected {tuple(shape)}")


@dataclass(frozen=True)
class PackedMoELayer:
    """`weights` in kernel layout plus where they came from.  `expert_range` is the block of routed experts
    held in `weights.expert_*` (all of them unless a shard was asked for)."""

    weights: MoEWeights
    keys: MoEWeightKeys
    expert_range: tuple


def pack_qwen36_moe_weights_from_state_dict(tensors: Mapping[str, Any], layer_idx: int, *, spec: Optional[MoESpec] = None,
                                            layer_prefixes: Sequence[str] = DEFAULT_LAYER_PREFIXES,
                                            device: Optional[Union[str, torch.device]] = None,
                                            dtype: Optional[torch.dtype] = None,
                                            expert_range: Optional[tuple] = None) -> PackedMoELayer:
    """Pack one MoE layer (reference: qwen36_weights.py:416-527; `dtype` and `expert_range` are extensions)."""
    spec = spec or qwen36_35b_a3b_spec()
    keys = resolve_qwen36_moe_weight_keys(tensors, layer_idx, spec=spec, layer_prefixes=layer_prefixes)
    H, E, I = spec.hidden_size, spec.num_experts, spec.expert_intermediate_size
    lo, hi = expert_range if expert_range is not None else (0, E)
    if not (0 <= lo <= hi <= E):
        raise ValueError(f"expert_range {expert_range} outside [0, {E}]")

    def fetch(key: str):
        t = tensors[key]
        if device is not None or dtype is not None:
            t = t.to(device=device, dtype=dtype)
        return t

    norm = fetch(keys.norm_weight)
    router = fetch(keys.router_weight)
    _expect(keys.norm_weight, norm, (H,))
    _expect(keys.router_weight, router, (E, H))

    def grouped(key: str, canonical: tuple):
        """A grouped [E, rows, cols] tensor, stored either way round; only the local block is converted."""
        raw = tensors[key]
        flipped = (canonical[0], canonical[2], canonical[1])
        if _shape(raw) != canonical and _shape(raw) == flipped:
            raw = raw.transpose(1, 2)
        _expect(key, raw, canonical)
        block = raw[lo:hi]
        if device is not None or dtype is not None:
            block = block.to(device=device, dtype=dtype)
        return block.contiguous()

    def empty_like_first(first, rows: int, cols: int):
        return torch.empty((hi - lo, rows, cols), dtype=first.dtype, device=first.device)

    if isinstance(keys.expert_gate_up_weight, str):
        gate_up = grouped(keys.expert_gate_up_weight, (E, 2 * I, H))
    else:
        gate_up = None
        for e in range(lo, hi):
            item = keys.expert_gate_up_weight[e]
            if isinstance(item, str):
                rows = fetch(item)
                _expect(item, rows, (2 * I, H))
                if gate_up is None:
                    gate_up = empty_like_first(rows, 2 * I, H)
                gate_up[e - lo] = rows
            else:
                g, u = fetch(item[0]), fetch(item[1])
                _expect(item[0], g, (I, H))
                _expect(item[1], u, (I, H))
                if gate_up is None:
                    gate_up = empty_like_first(g, 2 * I, H)
                gate_up[e - lo, :I] = g
                gate_up[e - lo, I:] = u
        if gate_up is None:
            gate_up = torch.empty((0, 2 * I, H), dtype=router.dtype, device=router.device)

    if isinstance(keys.expert_down_weight, str):
        down = grouped(keys.expert_down_weight, (E, H, I))
    else:
        down = None
        for e in range(lo, hi):
            key = keys.expert_down_weight[e]
            rows = fetch(key)
            _expect(key, rows, (H, I))
            if down is None:
                down = empty_like_first(rows, H, I)
            down[e - lo] = rows
        if down is None:
            down = torch.empty((0, H, I), dtype=router.dtype, device=router.device)

    if isinstance(keys.shared_gate_up_weight, str):
        shared_gu = fetch(keys.shared_gate_up_weight)
        _expect(keys.shared_gate_up_weight, shared_gu, (2 * I, H))
    else:
        sg, su = fetch(keys.shared_gate_up_weight[0]), fetch(keys.shared_gate_up_weight[1])
        _expect(keys.shared_gate_up_weight[0], sg, (I, H))
        _expect(keys.shared_gate_up_weight[1], su, (I, H))
        shared_gu = torch.cat((sg, su), dim=0)
    shared_dn = fetch(keys.shared_down_weight)
    _expect(keys.shared_down_weight, shared_dn, (H, I))

    shared_gate = None
    if keys.shared_expert_gate_weight is not None:
        shared_gate = fetch(keys.shared_expert_gate_weight).contiguous()
        if _shape(shared_gate) not in ((H,), (1, H)):
            raise ValueError(f"{keys.shared_expert_gate_weight} has shape {_shape(shared_gate)}, expected ({H},) or (1, {H})")

    weights = MoEWeights(norm.contiguous(), router.contiguous(), gate_up, down, shared_gu.contiguous(),
                         shared_dn.contiguous(), shared_gate)
    return PackedMoELayer(weights, keys, (lo, hi))


class LazySafetensors(Mapping):
    """Name -> tensor view of a safetensors checkpoint (one file, or a directory of shards with or without an
    index), fetched tensor by tensor.  Only the shards that hold a requested name are opened, and a tensor is
    read when it is asked for (the files are memory-mapped), so packing one layer, or one rank's block of
    experts, never loads the rest of the checkpoint."""

    def __init__(self, path):
        try:
            from safetensors import safe_open
        except ImportError as exc:  # pragma: no cover - optional dependency
            raise RuntimeError("safetensors is required to load Qwen3.6 MoE weights") from exc
        import json
        from pathlib import Path
        self._open = safe_open
        self._handles = {}
        source = Path(path)
        self._where = {}
        if source.is_dir():
            index_files = sorted(source.glob("*.safetensors.index.json"))
            if index_files:
                with index_files[0].open("r", encoding="utf-8") as handle:
                    index = json.load(handle)
                weight_map = index.get("weight_map", {})
                if not isinstance(weight_map, dict):
                    raise ValueError(f"{index_files[0]} does not contain a valid weight_map")
                self._where = {key: source / str(name) for key, name in weight_map.items()}
                self.indexed = True
                return
            files = sorted(source.glob("*.safetensors"))
        else:
            files = [source] if source.exists() else []
        if not files:
            raise FileNotFoundError(f"no safetensors files found at {source}")
        self.indexed = False
        for f in files:
            for key in self._handle(f).keys():
                self._where[key] = f

    def _handle(self, file):
        h = self._handles.get(file)
        if h is None:
            if not file.exists():
                raise FileNotFoundError(f"{file} is named by the safetensors index but does not exist")
            h = self._open(str(file), framework="pt", device="cpu")
            self._handles[file] = h
        return h

    def __getitem__(self, key):
        return self._handle(self._where[key]).get_tensor(key)

    def __contains__(self, key):
        return key in self._where

    def __iter__(self):
        return iter(self._where)

    def __len__(self):
        return len(self._where)

    def files_for(self, keys) -> list:
        return sorted({self._where[k] for k in keys})


def _flatten_keys(keys: MoEWeightKeys) -> list:
    out = []
    for item in (keys.norm_weight, keys.router_weight, keys.expert_gate_up_weight, keys.expert_down_weight,
                 keys.shared_gate_up_weight, keys.shared_down_weight, keys.shared_expert_gate_weight):
        stack = [item]
        while stack:
            cur = stack.pop()
            if cur is None:
                continue
            if isinstance(cur, str):
                out.append(cur)
            else:
                stack.extend(cur)
    return out


def load_qwen36_moe_weights_from_safetensors(path, layer_idx: int, *, spec: Optional[MoESpec] = None,
                                             layer_prefixes: Sequence[str] = DEFAULT_LAYER_PREFIXES,
                                             device: Optional[Union[str, torch.device]] = None,
                                             dtype: Optional[torch.dtype] = None,
                                             expert_range: Optional[tuple] = None) -> PackedMoELayer:
    """Load and pack one MoE layer from a safetensors file or directory (reference:
    src/fastkernels/models/qwen36_weights.py:656-716, same lookup order: an index file's weight map if the directory
    has one, else every `*.safetensors` file in it; same errors: `ValueError` for an index without a weight map,
    `KeyError` when the index lacks a resolved name, `FileNotFoundError` when nothing is there).

    Where the reference reads every shard that holds one of the layer's tensors completely into host memory and then
    packs, this goes through `LazySafetensors`: tensors are fetched one at a time from memory-mapped shards and
    converted to `dtype` on `device` as they are packed, and with `expert_range` a rank touches only its own
    experts' tensors."""
    spec = spec or qwen36_35b_a3b_spec()
    view = LazySafetensors(path)
    if view.indexed:
        keys = resolve_qwen36_moe_weight_keys(view, layer_idx, spec=spec, layer_prefixes=layer_prefixes)
        missing = sorted(k for k in set(_flatten_keys(keys)) if k not in view)
        if missing:
            raise KeyError(f"safetensors index is missing resolved keys: {missing[:8]}")
    return pack_qwen36_moe_weights_from_state_dict(view, layer_idx, spec=spec, layer_prefixes=layer_prefixes, device=device,
                                                   dtype=dtype, expert_range=expert_range)


def state_dict_from_moe_weights(w: MoEWeights, layer_idx: int, *, prefix: str = "model.language_model.layers",
                                grouped: bool = True) -> dict:
    """The inverse, for tests and synthetic checkpoints: a checkpoint-style mapping (grouped tensors as in the
    released Qwen3.6 files, or one gate/up/down tensor per expert) that packs back to `w`."""
    base = f"{prefix}.{layer_idx}"
    I = w.expert_gate_up_weight.shape[1] // 2
    out = {f"{base}.post_attention_layernorm.weight": w.norm_weight, f"{base}.mlp.gate.weight": w.router_weight,
           f"{base}.mlp.shared_expert.gate_proj.weight": w.shared_gate_up_weight[:I],
           f"{base}.mlp.shared_expert.up_proj.weight": w.shared_gate_up_weight[I:],
           f"{base}.mlp.shared_expert.down_proj.weight": w.shared_down_weight}
    if w.shared_expert_gate_weight is not None:
        out[f"{base}.mlp.shared_expert_gate.weight"] = w.shared_expert_gate_weight
    if grouped:
        out[f"{base}.mlp.experts.gate_up_proj"] = w.expert_gate_up_weight
        out[f"{base}.mlp.experts.down_proj"] = w.expert_down_weight
    else:
        for e in range(w.expert_gate_up_weight.shape[0]):
            out[f"{base}.mlp.experts.{e}.gate_proj.weight"] = w.expert_gate_up_weight[e, :I]
            out[f"{base}.mlp.experts.{e}.up_proj.weight"] = w.expert_gate_up_weight[e, I:]
            out[f"{base}.mlp.experts.{e}.down_proj.weight"] = w.expert_down_weight[e]
    return out
