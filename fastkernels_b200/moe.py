"""Host side of the B200 MoE decode layer: the reference's MoE functions over libfkmoe.so.

Every function keeps the name (minus the `triton_` prefix; `fastkernels_b200.kernels.triton`
re-exports them with it), positional order, keyword defaults, return types and
ValueError conditions of its counterpart in the reference's
`fastkernels.kernels.triton` package:

  qwen36_moe_router_decode / qwen36_batched_moe_router_decode
      src/fastkernels/kernels/triton/qwen36_router.py:193, :260
  qwen36_single_expert_mlp_decode, qwen36_routed_experts_decode,
  qwen36_routed_shared_experts_decode, qwen36_batched_routed_experts_decode,
  qwen36_batched_routed_shared_experts_decode, qwen36_moe_decode, qwen36_batched_moe_decode
      src/fastkernels/kernels/triton/qwen36_expert.py:817, :889, :969, :1096, :1181, :1312, :1353
  qwen36_batched_moe_layer_decode   src/fastkernels/kernels/triton/qwen36_layer.py:55
  fused_swiglu, expert_histogram    src/fastkernels/kernels/triton/moe.py:67, :87
  synthetic_qwen36_moe_decode       src/fastkernels/kernels/triton/qwen36_moe.py:362

Outputs are freshly allocated on the input's device with the reference's dtypes
(logits/weights/outputs fp32, ids int64, histogram int32); inputs are never
modified.  All work is enqueued on torch's current CUDA stream; nothing
synchronises.  Extensions that the reference lacks are keyword-only and default
to the reference's behaviour (`router_bias`, `flags`).
"""

from __future__ import annotations

import ctypes as C
from typing import Any, Optional

import torch

from . import _lib
from ._lib import Call, Dims

_DTYPES = {torch.float32: _lib.FK_F32, torch.bfloat16: _lib.FK_BF16, torch.float16: _lib.FK_F16}
_workspaces: dict[tuple[int, int], torch.Tensor] = {}


def _dtype_code(t: torch.Tensor, what: str) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise ValueError(f"{what} must be float32, bfloat16 or float16, got {t.dtype}") from None


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def workspace_for(device: torch.device, dims: Dims) -> torch.Tensor:
    """Cached, zero-initialised scratch tensor for `dims` on `device` and the current stream."""
    lib = _lib.load()
    need = lib.fk_moe_workspace_bytes(C.byref(dims))
    if need == 0:
        raise ValueError("MoE dims outside the supported limits "
                         "(hidden<=4096, experts<=1024, intermediate<=1024, top_k<=8)")
    key = (device.index if device.index is not None else torch.cuda.current_device(), _stream())
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=device)
        _lib.check(lib.fk_moe_workspace_init(ws.data_ptr(), ws.numel(), _stream()), "fk_moe_workspace_init")
        _workspaces[key] = ws
    return ws


def _as_weight(t: Optional[torch.Tensor], dtype: torch.dtype) -> Optional[torch.Tensor]:
    if t is None:
        return None
    if t.dtype != dtype:
        t = t.to(dtype)
    return t.contiguous()


def _make_call(hidden: torch.Tensor, tokens: int, hidden_size: int, experts: int, intermediate: int, top_k: int,
               weight_dtype: torch.dtype, *, eps: float = 1e-6, norm_offset: float = 1.0, flags: int = 0,
               expert_base: int = 0) -> tuple[Call, torch.Tensor]:
    call = Call()
    call.dims = Dims(tokens, hidden_size, experts, intermediate, top_k)
    call.hidden_dtype = _dtype_code(hidden, "hidden")
    call.weight_dtype = _DTYPES.get(weight_dtype, -1)
    if call.weight_dtype < 0:
        raise ValueError(f"weights must be float32, bfloat16 or float16, got {weight_dtype}")
    call.eps = eps
    call.norm_offset = norm_offset
    call.flags = flags
    call.expert_base = expert_base
    ws = workspace_for(hidden.device, call.dims)
    call.workspace = ws.data_ptr()
    call.workspace_bytes = ws.numel()
    return call, ws


# --------------------------------------------------------------------------- #
# Router                                                                      #
# --------------------------------------------------------------------------- #

def _router(hidden2d, norm_weight, router_weight, top_k, eps, norm_offset, router_bias, flags=0):
    tokens, hidden_size = hidden2d.shape
    num_experts = router_weight.shape[0]
    if top_k < 1 or top_k > 8:
        raise ValueError("router kernel supports 1 <= top_k <= 8")
    if hidden_size > 4096 or num_experts > 1024:
        raise ValueError("router kernel currently supports hidden_size<=4096 and num_experts<=1024")
    if top_k > num_experts:
        raise ValueError("top_k must be <= number of experts")
    lib = _lib.load()
    dev = hidden2d.device
    wdt = router_weight.dtype
    hidden2d = hidden2d.contiguous()
    router_weight = router_weight.contiguous()
    norm_weight = _as_weight(norm_weight, wdt)
    bias = None if router_bias is None else router_bias.to(device=dev, dtype=torch.float32).contiguous()
    logits = torch.empty((tokens, num_experts), device=dev, dtype=torch.float32)
    topk_ids = torch.empty((tokens, top_k), device=dev, dtype=torch.int64)
    topk_weights = torch.empty((tokens, top_k), device=dev, dtype=torch.float32)
    call, ws = _make_call(hidden2d, tokens, hidden_size, num_experts, 1, top_k, wdt, eps=eps,
                          norm_offset=norm_offset, flags=flags)
    call.hidden = _ptr(hidden2d)
    call.norm_weight = _ptr(norm_weight)
    call.router_weight = _ptr(router_weight)
    call.router_bias = _ptr(bias)
    call.logits = _ptr(logits)
    call.topk_ids = _ptr(topk_ids)
    call.topk_weights = _ptr(topk_weights)
    with torch.cuda.device(dev):
        _lib.check(lib.fk_moe_router(C.byref(call), _stream()), "fk_moe_router")
    return logits, topk_ids, topk_weights


def qwen36_moe_router_decode(hidden: Any, norm_weight: Any, router_weight: Any, *, top_k: int = 8,
                             eps: float = 1e-6, norm_offset: float = 1.0, router_bias: Any = None):
    """One token: `(logits [E] f32, topk_ids [k] i64, topk_weights [k] f32)`."""
    if hidden.ndim != 1:
        raise ValueError("hidden must have shape [hidden_size]")
    if norm_weight.shape != hidden.shape:
        raise ValueError("norm_weight must have the same shape as hidden")
    if router_weight.ndim != 2 or router_weight.shape[1] != hidden.shape[0]:
        raise ValueError("router_weight must have shape [num_experts, hidden_size]")
    if not hidden.is_cuda or not norm_weight.is_cuda or not router_weight.is_cuda:
        raise ValueError("hidden, norm_weight, and router_weight must be CUDA tensors")
    logits, ids, weights = _router(hidden.unsqueeze(0), norm_weight, router_weight, top_k, eps, norm_offset,
                                   router_bias)
    return logits[0], ids[0], weights[0]


def qwen36_batched_moe_router_decode(hidden: Any, norm_weight: Any, router_weight: Any, *, top_k: int = 8,
                                     eps: float = 1e-6, norm_offset: float = 1.0, router_bias: Any = None):
    """Batched tokens: `(logits [T,E] f32, topk_ids [T,k] i64, topk_weights [T,k] f32)`."""
    if hidden.ndim != 2:
        raise ValueError("hidden must have shape [tokens, hidden_size]")
    if norm_weight.ndim != 1 or norm_weight.shape[0] != hidden.shape[1]:
        raise ValueError("norm_weight must have shape [hidden_size]")
    if router_weight.ndim != 2 or router_weight.shape[1] != hidden.shape[1]:
        raise ValueError("router_weight must have shape [num_experts, hidden_size]")
    if not hidden.is_cuda or not norm_weight.is_cuda or not router_weight.is_cuda:
        raise ValueError("hidden, norm_weight, and router_weight must be CUDA tensors")
    return _router(hidden, norm_weight, router_weight, top_k, eps, norm_offset, router_bias)


# --------------------------------------------------------------------------- #
# Experts                                                                     #
# --------------------------------------------------------------------------- #

def _check_expert_weights(hidden_size, expert_gate_up_weight, expert_down_weight):
    if expert_gate_up_weight.ndim != 3:
        raise ValueError("expert_gate_up_weight must have shape [experts, 2 * intermediate, hidden_size]")
    if expert_down_weight.ndim != 3:
        raise ValueError("expert_down_weight must have shape [experts, hidden_size, intermediate]")
    num_experts = expert_gate_up_weight.shape[0]
    if expert_down_weight.shape[0] != num_experts:
        raise ValueError("expert gate/up and down weights must have the same number of experts")
    if expert_gate_up_weight.shape[2] != hidden_size or expert_down_weight.shape[1] != hidden_size:
        raise ValueError("expert weight hidden dimensions must match hidden")
    if expert_gate_up_weight.shape[1] % 2:
        raise ValueError("expert_gate_up_weight second dimension must be even")
    intermediate = expert_gate_up_weight.shape[1] // 2
    if expert_down_weight.shape[2] != intermediate:
        raise ValueError("expert_down_weight intermediate dimension must match gate/up weight")
    if hidden_size > 4096 or intermediate > 1024 or num_experts > 1024:
        raise ValueError("expert kernels support hidden_size<=4096, intermediate<=1024 and experts<=1024")
    return num_experts, intermediate


def _experts(hidden2d, topk_ids, topk_weights, expert_gate_up_weight, expert_down_weight, shared_gate_up_weight,
             shared_down_weight, shared_expert_gate_weight, *, flags=0, expert_base=0, residual=False,
             shared_token_range=None):
    lib = _lib.load()
    tokens, hidden_size = hidden2d.shape
    num_experts, intermediate = _check_expert_weights(hidden_size, expert_gate_up_weight, expert_down_weight)
    top_k = topk_ids.shape[1]
    dev = hidden2d.device
    wdt = expert_gate_up_weight.dtype
    hidden2d = hidden2d.contiguous()
    ids = topk_ids.to(torch.int64).contiguous()
    wts = topk_weights.to(torch.float32).contiguous()
    gate_up = expert_gate_up_weight.contiguous()
    down = _as_weight(expert_down_weight, wdt)
    sgu = _as_weight(shared_gate_up_weight, wdt)
    sdn = _as_weight(shared_down_weight, wdt)
    sg = _as_weight(shared_expert_gate_weight, wdt)
    out = torch.empty((tokens, hidden_size), device=dev, dtype=torch.float32)
    layer = torch.empty_like(out) if residual else None
    call, ws = _make_call(hidden2d, tokens, hidden_size, num_experts, intermediate, top_k, wdt, flags=flags,
                          expert_base=expert_base)
    call.hidden = _ptr(hidden2d)
    call.expert_gate_up = _ptr(gate_up)
    call.expert_down = _ptr(down)
    call.shared_gate_up = _ptr(sgu)
    call.shared_down = _ptr(sdn)
    call.shared_gate = _ptr(sg)
    call.topk_ids_in = _ptr(ids)
    call.topk_weights_in = _ptr(wts)
    call.out = _ptr(out)
    call.layer_hidden = _ptr(layer)
    if shared_token_range is not None:
        call.shared_token_base, call.shared_token_count = shared_token_range
    with torch.cuda.device(dev):
        _lib.check(lib.fk_moe_experts(C.byref(call), _stream()), "fk_moe_experts")
    return (out, layer) if residual else out


def qwen36_single_expert_mlp_decode(hidden: Any, expert_gate_up_weight: Any, expert_down_weight: Any, *,
                                    block_intermediate: int = 16, block_hidden: int = 16):
    """One expert MLP for one token, fp32 `[H]`.  The block_* knobs of the reference are accepted and ignored."""
    if hidden.ndim != 1:
        raise ValueError("hidden must have shape [hidden_size]")
    if expert_gate_up_weight.ndim != 2:
        raise ValueError("expert_gate_up_weight must have shape [2 * intermediate, hidden_size]")
    if expert_down_weight.ndim != 2:
        raise ValueError("expert_down_weight must have shape [hidden_size, intermediate]")
    if not hidden.is_cuda or not expert_gate_up_weight.is_cuda or not expert_down_weight.is_cuda:
        raise ValueError("hidden and expert weights must be CUDA tensors")
    hidden_size = hidden.shape[0]
    if expert_gate_up_weight.shape[1] != hidden_size or expert_down_weight.shape[0] != hidden_size:
        raise ValueError("expert weight hidden dimensions must match hidden")
    if expert_gate_up_weight.shape[0] % 2:
        raise ValueError("expert_gate_up_weight first dimension must be even")
    intermediate = expert_gate_up_weight.shape[0] // 2
    if expert_down_weight.shape[1] != intermediate:
        raise ValueError("expert_down_weight intermediate dimension must match gate/up weight")
    if hidden_size > 4096 or intermediate > 1024:
        raise ValueError("expert MLP kernel currently supports hidden_size<=4096 and intermediate<=1024")
    lib = _lib.load()
    dev = hidden.device
    wdt = expert_gate_up_weight.dtype
    hidden = hidden.contiguous()
    gate_up = expert_gate_up_weight.contiguous()
    down = _as_weight(expert_down_weight, wdt)
    out = torch.empty((hidden_size,), device=dev, dtype=torch.float32)
    ws = workspace_for(dev, Dims(1, hidden_size, 1, intermediate, 0))
    with torch.cuda.device(dev):
        _lib.check(lib.fk_single_expert_mlp(_ptr(hidden), _dtype_code(hidden, "hidden"), _ptr(gate_up), _ptr(down),
                                            _DTYPES[wdt], _ptr(out), hidden_size, intermediate, ws.data_ptr(),
                                            ws.numel(), _stream()), "fk_single_expert_mlp")
    return out


def _check_single_routing(hidden, topk_ids, topk_weights, expert_gate_up_weight, expert_down_weight):
    if hidden.ndim != 1:
        raise ValueError("hidden must have shape [hidden_size]")
    if topk_ids.ndim != 1 or topk_weights.ndim != 1:
        raise ValueError("topk_ids and topk_weights must have shape [top_k]")
    if topk_ids.shape != topk_weights.shape:
        raise ValueError("topk_ids and topk_weights must have the same shape")
    if expert_gate_up_weight.ndim != 3:
        raise ValueError("expert_gate_up_weight must have shape [experts, 2 * intermediate, hidden_size]")
    if expert_down_weight.ndim != 3:
        raise ValueError("expert_down_weight must have shape [experts, hidden_size, intermediate]")
    if not hidden.is_cuda or not topk_ids.is_cuda or not topk_weights.is_cuda:
        raise ValueError("hidden, topk_ids, and topk_weights must be CUDA tensors")
    if not expert_gate_up_weight.is_cuda or not expert_down_weight.is_cuda:
        raise ValueError("expert weights must be CUDA tensors")


def qwen36_routed_experts_decode(hidden: Any, topk_ids: Any, topk_weights: Any, expert_gate_up_weight: Any,
                                 expert_down_weight: Any, *, flags: int = 0):
    """One token, routed experts only (no shared expert), fp32 `[H]`."""
    _check_single_routing(hidden, topk_ids, topk_weights, expert_gate_up_weight, expert_down_weight)
    _check_expert_weights(hidden.shape[0], expert_gate_up_weight, expert_down_weight)
    if topk_ids.numel() > 8:
        raise ValueError("routed expert path currently supports top_k <= 8")
    return _experts(hidden.unsqueeze(0), topk_ids.unsqueeze(0), topk_weights.unsqueeze(0), expert_gate_up_weight,
                    expert_down_weight, None, None, None, flags=flags)[0]


def qwen36_routed_shared_experts_decode(hidden: Any, topk_ids: Any, topk_weights: Any, expert_gate_up_weight: Any,
                                        expert_down_weight: Any, shared_gate_up_weight: Any = None,
                                        shared_down_weight: Any = None, shared_expert_gate_weight: Any = None, *,
                                        flags: int = 0):
    """One token, routed experts plus the (optionally sigmoid-gated) shared expert, fp32 `[H]`."""
    _check_single_routing(hidden, topk_ids, topk_weights, expert_gate_up_weight, expert_down_weight)
    hidden_size = hidden.shape[0]
    _check_expert_weights(hidden_size, expert_gate_up_weight, expert_down_weight)
    if topk_ids.numel() > 8:
        raise ValueError("routed/shared expert path currently supports top_k <= 8")
    if shared_gate_up_weight is None or shared_down_weight is None:
        raise ValueError("shared_gate_up_weight and shared_down_weight are required")
    if not shared_gate_up_weight.is_cuda or not shared_down_weight.is_cuda:
        raise ValueError("shared expert weights must be CUDA tensors")
    if shared_gate_up_weight.shape != expert_gate_up_weight.shape[1:]:
        raise ValueError("shared_gate_up_weight must have shape [2 * intermediate, hidden_size]")
    if shared_down_weight.shape != expert_down_weight.shape[1:]:
        raise ValueError("shared_down_weight must have shape [hidden_size, intermediate]")
    if shared_expert_gate_weight is not None:
        if not shared_expert_gate_weight.is_cuda:
            raise ValueError("shared_expert_gate_weight must be a CUDA tensor")
        if shared_expert_gate_weight.numel() != hidden_size:
            raise ValueError("shared_expert_gate_weight must have hidden_size elements")
    return _experts(hidden.unsqueeze(0), topk_ids.unsqueeze(0), topk_weights.unsqueeze(0), expert_gate_up_weight,
                    expert_down_weight, shared_gate_up_weight, shared_down_weight, shared_expert_gate_weight,
                    flags=flags)[0]


def _check_batched_routing(hidden, topk_ids, topk_weights, expert_gate_up_weight, expert_down_weight):
    if hidden.ndim != 2:
        raise ValueError("hidden must have shape [tokens, hidden_size]")
    if topk_ids.ndim != 2 or topk_weights.ndim != 2:
        raise ValueError("topk_ids and topk_weights must have shape [tokens, top_k]")
    if topk_ids.shape != topk_weights.shape:
        raise ValueError("topk_ids and topk_weights must have the same shape")
    if topk_ids.shape[0] != hidden.shape[0]:
        raise ValueError("topk_ids/topk_weights token dimension must match hidden")
    if expert_gate_up_weight.ndim != 3:
        raise ValueError("expert_gate_up_weight must have shape [experts, 2 * intermediate, hidden_size]")
    if expert_down_weight.ndim != 3:
        raise ValueError("expert_down_weight must have shape [experts, hidden_size, intermediate]")


def qwen36_batched_routed_experts_decode(hidden: Any, topk_ids: Any, topk_weights: Any, expert_gate_up_weight: Any,
                                         expert_down_weight: Any, *, flags: int = 0, expert_base: int = 0):
    """Batched routed experts only: the operator boundary of a generic fused-MoE op (no router, no shared
    expert, no residual), fp32 `[T,H]`."""
    _check_batched_routing(hidden, topk_ids, topk_weights, expert_gate_up_weight, expert_down_weight)
    tensors = (hidden, topk_ids, topk_weights, expert_gate_up_weight, expert_down_weight)
    if not all(t.is_cuda for t in tensors):
        raise ValueError("hidden, routing tensors, and expert weights must be CUDA tensors")
    _check_expert_weights(hidden.shape[1], expert_gate_up_weight, expert_down_weight)
    if topk_ids.shape[1] > 8:
        raise ValueError("batched routed expert path currently supports top_k <= 8")
    return _experts(hidden, topk_ids, topk_weights, expert_gate_up_weight, expert_down_weight, None, None, None,
                    flags=flags, expert_base=expert_base)


def qwen36_batched_routed_shared_experts_decode(hidden: Any, topk_ids: Any, topk_weights: Any,
                                                expert_gate_up_weight: Any, expert_down_weight: Any,
                                                shared_gate_up_weight: Any, shared_down_weight: Any,
                                                shared_expert_gate_weight: Any = None, *, flags: int = 0,
                                                expert_base: int = 0):
    """Batched routed + shared experts, fp32 `[T,H]`."""
    _check_batched_routing(hidden, topk_ids, topk_weights, expert_gate_up_weight, expert_down_weight)
    tensors = (hidden, topk_ids, topk_weights, expert_gate_up_weight, expert_down_weight, shared_gate_up_weight,
               shared_down_weight)
    if not all(t.is_cuda for t in tensors):
        raise ValueError("hidden, routing tensors, and expert weights must be CUDA tensors")
    if shared_expert_gate_weight is not None and not shared_expert_gate_weight.is_cuda:
        raise ValueError("shared_expert_gate_weight must be a CUDA tensor")
    hidden_size = hidden.shape[1]
    _check_expert_weights(hidden_size, expert_gate_up_weight, expert_down_weight)
    if topk_ids.shape[1] > 8:
        raise ValueError("batched routed/shared expert path currently supports top_k <= 8")
    if shared_gate_up_weight.shape != expert_gate_up_weight.shape[1:]:
        raise ValueError("shared_gate_up_weight must have shape [2 * intermediate, hidden_size]")
    if shared_down_weight.shape != expert_down_weight.shape[1:]:
        raise ValueError("shared_down_weight must have shape [hidden_size, intermediate]")
    if shared_expert_gate_weight is not None and shared_expert_gate_weight.numel() != hidden_size:
        raise ValueError("shared_expert_gate_weight must have hidden_size elements")
    return _experts(hidden, topk_ids, topk_weights, expert_gate_up_weight, expert_down_weight,
                    shared_gate_up_weight, shared_down_weight, shared_expert_gate_weight, flags=flags,
                    expert_base=expert_base)


# --------------------------------------------------------------------------- #
# Whole layer                                                                 #
# --------------------------------------------------------------------------- #

def _layer(hidden2d, norm_weight, router_weight, expert_gate_up_weight, expert_down_weight, shared_gate_up_weight,
           shared_down_weight, shared_expert_gate_weight, *, top_k, eps, norm_offset=1.0, router_bias=None,
           residual=False, flags=0):
    if norm_weight.ndim != 1 or norm_weight.shape[0] != hidden2d.shape[1]:
        raise ValueError("norm_weight must have shape [hidden_size]")
    if router_weight.ndim != 2 or router_weight.shape[1] != hidden2d.shape[1]:
        raise ValueError("router_weight must have shape [num_experts, hidden_size]")
    tensors = (hidden2d, norm_weight, router_weight, expert_gate_up_weight, expert_down_weight)
    if not all(t.is_cuda for t in tensors):
        raise ValueError("hidden, norm_weight, router_weight and expert weights must be CUDA tensors")
    if top_k < 1 or top_k > 8:
        raise ValueError("router kernel supports 1 <= top_k <= 8")
    tokens, hidden_size = hidden2d.shape
    num_experts, intermediate = _check_expert_weights(hidden_size, expert_gate_up_weight, expert_down_weight)
    if router_weight.shape[0] != num_experts:
        raise ValueError("router_weight and expert weights disagree on expert count")
    if top_k > num_experts:
        raise ValueError("top_k must be <= number of experts")
    if (shared_gate_up_weight is None) != (shared_down_weight is None):
        raise ValueError("shared_gate_up_weight and shared_down_weight must be given together")
    if shared_gate_up_weight is not None:
        if shared_gate_up_weight.shape != expert_gate_up_weight.shape[1:]:
            raise ValueError("shared_gate_up_weight must have shape [2 * intermediate, hidden_size]")
        if shared_down_weight.shape != expert_down_weight.shape[1:]:
            raise ValueError("shared_down_weight must have shape [hidden_size, intermediate]")
    if shared_expert_gate_weight is not None and shared_expert_gate_weight.numel() != hidden_size:
        raise ValueError("shared_expert_gate_weight must have hidden_size elements")
    lib = _lib.load()
    dev = hidden2d.device
    wdt = expert_gate_up_weight.dtype
    hidden2d = hidden2d.contiguous()
    norm_weight = _as_weight(norm_weight, wdt)
    router_weight = _as_weight(router_weight, wdt)
    gate_up = expert_gate_up_weight.contiguous()
    down = _as_weight(expert_down_weight, wdt)
    sgu = _as_weight(shared_gate_up_weight, wdt)
    sdn = _as_weight(shared_down_weight, wdt)
    sg = _as_weight(shared_expert_gate_weight, wdt)
    bias = None if router_bias is None else router_bias.to(device=dev, dtype=torch.float32).contiguous()
    out = torch.empty((tokens, hidden_size), device=dev, dtype=torch.float32)
    layer = torch.empty_like(out) if residual else None
    logits = torch.empty((tokens, num_experts), device=dev, dtype=torch.float32)
    topk_ids = torch.empty((tokens, top_k), device=dev, dtype=torch.int64)
    topk_weights = torch.empty((tokens, top_k), device=dev, dtype=torch.float32)
    call, ws = _make_call(hidden2d, tokens, hidden_size, num_experts, intermediate, top_k, wdt, eps=eps,
                          norm_offset=norm_offset, flags=flags)
    call.hidden = _ptr(hidden2d)
    call.norm_weight = _ptr(norm_weight)
    call.router_weight = _ptr(router_weight)
    call.router_bias = _ptr(bias)
    call.expert_gate_up = _ptr(gate_up)
    call.expert_down = _ptr(down)
    call.shared_gate_up = _ptr(sgu)
    call.shared_down = _ptr(sdn)
    call.shared_gate = _ptr(sg)
    call.out = _ptr(out)
    call.layer_hidden = _ptr(layer)
    call.logits = _ptr(logits)
    call.topk_ids = _ptr(topk_ids)
    call.topk_weights = _ptr(topk_weights)
    with torch.cuda.device(dev):
        _lib.check(lib.fk_moe_layer(C.byref(call), _stream()), "fk_moe_layer")
    return out, layer, logits, topk_ids, topk_weights


def qwen36_moe_decode(hidden: Any, norm_weight: Any, router_weight: Any, expert_gate_up_weight: Any,
                      expert_down_weight: Any, shared_gate_up_weight: Any, shared_down_weight: Any,
                      shared_expert_gate_weight: Any = None, *, top_k: int = 8, eps: float = 1e-6,
                      router_bias: Any = None, flags: int = 0):
    """One token through the whole MoE block: `(output [H], logits [E], topk_ids [k], topk_weights [k])`."""
    if hidden.ndim != 1:
        raise ValueError("hidden must have shape [hidden_size]")
    out, _, logits, ids, weights = _layer(hidden.unsqueeze(0), norm_weight, router_weight, expert_gate_up_weight,
                                          expert_down_weight, shared_gate_up_weight, shared_down_weight,
                                          shared_expert_gate_weight, top_k=top_k, eps=eps, router_bias=router_bias,
                                          flags=flags)
    return out[0], logits[0], ids[0], weights[0]


def qwen36_batched_moe_decode(hidden: Any, norm_weight: Any, router_weight: Any, expert_gate_up_weight: Any,
                              expert_down_weight: Any, shared_gate_up_weight: Any, shared_down_weight: Any,
                              shared_expert_gate_weight: Any = None, *, top_k: int = 8, eps: float = 1e-6,
                              router_bias: Any = None, flags: int = 0):
    """Batched tokens through the whole MoE block: `(output [T,H], logits [T,E], topk_ids, topk_weights)`."""
    if hidden.ndim != 2:
        raise ValueError("hidden must have shape [tokens, hidden_size]")
    out, _, logits, ids, weights = _layer(hidden, norm_weight, router_weight, expert_gate_up_weight,
                                          expert_down_weight, shared_gate_up_weight, shared_down_weight,
                                          shared_expert_gate_weight, top_k=top_k, eps=eps, router_bias=router_bias,
                                          flags=flags)
    return out, logits, ids, weights


def qwen36_batched_moe_layer_decode(hidden: Any, norm_weight: Any, router_weight: Any, expert_gate_up_weight: Any,
                                    expert_down_weight: Any, shared_gate_up_weight: Any, shared_down_weight: Any,
                                    shared_expert_gate_weight: Any = None, *, top_k: int = 8, eps: float = 1e-6,
                                    router_bias: Any = None, flags: int = 0):
    """MoE block plus the residual: `(layer_hidden, moe_update, logits, topk_ids, topk_weights)`, all fp32."""
    if hidden.ndim != 2:
        raise ValueError("hidden must have shape [tokens, hidden_size]")
    if not hidden.is_cuda:
        raise ValueError("hidden must be a CUDA tensor")
    out, layer, logits, ids, weights = _layer(hidden, norm_weight, router_weight, expert_gate_up_weight,
                                              expert_down_weight, shared_gate_up_weight, shared_down_weight,
                                              shared_expert_gate_weight, top_k=top_k, eps=eps,
                                              router_bias=router_bias, residual=True, flags=flags)
    return layer, out, logits, ids, weights


def synthetic_qwen36_moe_decode(hidden: Any, norm_weight: Any, router_weight: Any, expert_gate_up_weight: Any,
                                expert_down_weight: Any, shared_gate_up_weight: Any, shared_down_weight: Any, *,
                                top_k: int, eps: float = 1e-6):
    """Tiny-spec block for one token: plain-weight router norm, ungated shared expert, residual included.

    Returns a tensor shaped and typed like `hidden` (src/fastkernels/kernels/triton/qwen36_moe.py:362-444;
    oracle src/fastkernels/reference/qwen36_decode.py:212-224).
    """
    if top_k < 1 or top_k > 8:
        raise ValueError("prototype synthetic Qwen3.6 MoE kernel supports 1 <= top_k <= 8")
    if hidden.ndim != 1:
        raise ValueError("hidden must have shape [hidden_size]")
    if not hidden.is_cuda:
        raise ValueError("hidden must be a CUDA tensor")
    if expert_gate_up_weight.ndim != 3:
        raise ValueError("expert_gate_up_weight must have shape [experts, 2 * intermediate, hidden]")
    if expert_down_weight.ndim != 3:
        raise ValueError("expert_down_weight must have shape [experts, hidden, intermediate]")
    if top_k > router_weight.shape[0]:
        raise ValueError("top_k must be <= number of experts")
    _, layer, _, _, _ = _layer(hidden.unsqueeze(0), norm_weight, router_weight, expert_gate_up_weight,
                               expert_down_weight, shared_gate_up_weight, shared_down_weight, None, top_k=top_k,
                               eps=eps, norm_offset=0.0, residual=True)
    return layer[0].to(hidden.dtype)


# --------------------------------------------------------------------------- #
# Stand-alone ops                                                             #
# --------------------------------------------------------------------------- #

def fused_swiglu(gate_up: Any, *, block_size: int = 256):
    """`silu(gate) * up` for `[N, 2I]`, returned in the input dtype."""
    if gate_up.ndim != 2:
        raise ValueError("gate_up must have shape [N, 2 * intermediate]")
    if gate_up.shape[1] % 2:
        raise ValueError("last dimension must be even")
    if not gate_up.is_cuda:
        raise ValueError("gate_up must be a CUDA tensor")
    lib = _lib.load()
    gate_up = gate_up.contiguous()
    intermediate = gate_up.shape[1] // 2
    out = torch.empty((gate_up.shape[0], intermediate), device=gate_up.device, dtype=gate_up.dtype)
    with torch.cuda.device(gate_up.device):
        _lib.check(lib.fk_fused_swiglu(_ptr(gate_up), _ptr(out), _dtype_code(gate_up, "gate_up"), gate_up.shape[0],
                                       intermediate, _stream()), "fk_fused_swiglu")
    return out


def expert_histogram(topk_ids: Any, num_experts: int, *, block_size: int = 256):
    """Routes per expert, int32 `[num_experts]`."""
    if topk_ids.ndim != 2:
        raise ValueError("topk_ids must have shape [tokens, top_k]")
    if not topk_ids.is_cuda:
        raise ValueError("topk_ids must be a CUDA tensor")
    if topk_ids.dtype not in (torch.int32, torch.int64):
        topk_ids = topk_ids.to(torch.int64)
    lib = _lib.load()
    ids = topk_ids.contiguous()
    counts = torch.empty((num_experts,), device=ids.device, dtype=torch.int32)
    with torch.cuda.device(ids.device):
        _lib.check(lib.fk_expert_histogram(_ptr(ids), int(ids.dtype == torch.int64), ids.numel(), num_experts,
                                           _ptr(counts), _stream()), "fk_expert_histogram")
    return counts


def expert_permutation(topk_ids: Any, num_experts: int):
    """`(counts i32 [E], offsets i32 [E+1], order i32 [T*k])` with `order = argsort(ids.flatten(), stable=True)`."""
    if topk_ids.ndim != 2:
        raise ValueError("topk_ids must have shape [tokens, top_k]")
    if not topk_ids.is_cuda:
        raise ValueError("topk_ids must be a CUDA tensor")
    if num_experts < 1 or num_experts > 1024:
        raise ValueError("expert_permutation supports 1 <= num_experts <= 1024")
    lib = _lib.load()
    ids = topk_ids.to(torch.int64).contiguous()
    dev = ids.device
    counts = torch.empty((num_experts,), device=dev, dtype=torch.int32)
    offsets = torch.empty((num_experts + 1,), device=dev, dtype=torch.int32)
    order = torch.empty((ids.numel(),), device=dev, dtype=torch.int32)
    with torch.cuda.device(dev):
        _lib.check(lib.fk_moe_permute(_ptr(ids), ids.shape[0], ids.shape[1], num_experts, _ptr(counts),
                                      _ptr(offsets), _ptr(order), None, 0, _stream()), "fk_moe_permute")
    return counts, offsets, order
