"""A prepared MoE layer call: outputs, workspace and argument block allocated once.

The drop-in functions of `fastkernels_b200.moe` allocate their outputs on every call, as
the reference does (src/fastkernels/kernels/triton/qwen36_expert.py:1241-1242).  A decode
loop calls the same layer with the same shapes thousands of times, so `MoEDecodePlan`
fixes the weights and the token count up front; `run()` then only enqueues kernels (or
replays a captured CUDA graph), and `run_host()` takes pinned host buffers and includes
the host<->device copies.
"""

from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib
from ._lib import Call, Dims
from .moe import _DTYPES, _as_weight, _ptr
from .spec import MoEWeights


class PlanChain:
    """Several prepared layer calls captured back to back in ONE CUDA graph, as a decoder stack replays them.

    The kernels are launched with the programmatic-dependent-launch attribute, which survives capture as a
    programmatic edge: the next call's kernels become resident while the previous call's last blocks drain and
    load their constant weights meanwhile; they wait for the previous call to complete before they touch
    anything it may have written.  A replay runs every plan once, in order; each plan reads its own
    `hidden` buffer and writes its own outputs.
    """

    def __init__(self, plans):
        self.plans = list(plans)
        dev = self.plans[0].device
        s = torch.cuda.Stream(device=dev)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for p in self.plans:           # warm-up outside capture (function attributes, tensor maps, lazy loading)
                p.launch()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize(dev)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for p in self.plans:
                p.launch()
        self.graph = g

    def __len__(self):
        return len(self.plans)

    def replay(self) -> None:
        self.graph.replay()


class MoEDecodePlan:
    def __init__(self, weights: MoEWeights, tokens: int, *, hidden_dtype: torch.dtype = torch.bfloat16,
                 top_k: int = 8, eps: float = 1e-6, norm_offset: float = 1.0, residual: bool = False,
                 flags: int = 0, device: Optional[torch.device] = None, hidden_buffer: Optional[torch.Tensor] = None,
                 out_buffer: Optional[torch.Tensor] = None):
        self.lib = _lib.load()
        w = weights
        dev = device or w.expert_gate_up_weight.device
        if dev.type != "cuda":
            raise ValueError("MoEDecodePlan needs CUDA weights")
        self.device = dev
        wdt = w.expert_gate_up_weight.dtype
        E, two_i, H = w.expert_gate_up_weight.shape
        I = two_i // 2
        self.tokens, self.hidden_size, self.num_experts, self.intermediate, self.top_k = tokens, H, E, I, top_k
        self.hidden_dtype = hidden_dtype
        self._keep = [
            _as_weight(w.norm_weight, wdt), _as_weight(w.router_weight, wdt), w.expert_gate_up_weight.contiguous(),
            _as_weight(w.expert_down_weight, wdt), _as_weight(w.shared_gate_up_weight, wdt),
            _as_weight(w.shared_down_weight, wdt), _as_weight(w.shared_expert_gate_weight, wdt),
            None if w.router_bias is None else w.router_bias.to(device=dev, dtype=torch.float32).contiguous(),
        ]
        # buffers may be shared between the plans of a layer stack
        self.hidden = hidden_buffer if hidden_buffer is not None else torch.zeros((tokens, H), device=dev, dtype=hidden_dtype)
        self.out = out_buffer if out_buffer is not None else torch.empty((tokens, H), device=dev, dtype=torch.float32)
        self.layer_hidden = torch.empty_like(self.out) if residual else None
        self.logits = torch.empty((tokens, E), device=dev, dtype=torch.float32)
        self.topk_ids = torch.empty((tokens, top_k), device=dev, dtype=torch.int64)
        self.topk_weights = torch.empty((tokens, top_k), device=dev, dtype=torch.float32)
        dims = Dims(tokens, H, E, I, top_k)
        need = self.lib.fk_moe_workspace_bytes(C.byref(dims))
        if need == 0:
            raise ValueError("MoE dims outside the supported limits")
        self.workspace = torch.zeros(need, dtype=torch.uint8, device=dev)
        call = Call()
        call.dims = dims
        call.hidden_dtype = _DTYPES[hidden_dtype]
        call.weight_dtype = _DTYPES[wdt]
        call.eps, call.norm_offset, call.flags, call.expert_base = eps, norm_offset, flags, 0
        (call.norm_weight, call.router_weight, call.expert_gate_up, call.expert_down, call.shared_gate_up,
         call.shared_down, call.shared_gate, call.router_bias) = [_ptr(t) for t in self._keep]
        call.hidden = _ptr(self.hidden)
        call.out, call.layer_hidden = _ptr(self.out), _ptr(self.layer_hidden)
        call.logits, call.topk_ids, call.topk_weights = _ptr(self.logits), _ptr(self.topk_ids), _ptr(self.topk_weights)
        call.workspace, call.workspace_bytes = self.workspace.data_ptr(), self.workspace.numel()
        self.call = call
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        # host path
        self._staging = None
        self._host_call = None

    # ------------------------------------------------------------------ device-resident input
    def launch(self) -> None:
        """Enqueue the layer on the current stream, reading `self.hidden`, writing `self.out` etc."""
        _lib.check(self.lib.fk_moe_layer(C.byref(self.call), torch.cuda.current_stream().cuda_stream), "fk_moe_layer")

    def capture(self) -> None:
        """Capture one layer call into a CUDA graph; `run()` then replays it."""
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self.launch()          # warm-up outside capture (function attributes, lazy module load)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.launch()
        self.graph = g

    def run(self, hidden: Optional[torch.Tensor] = None):
        """`hidden` (device, [T,H]) is copied into the plan's input buffer if given.
        Returns `(out, logits, topk_ids, topk_weights)`: views of the plan's buffers, overwritten by the next run."""
        if hidden is not None:
            self.hidden.copy_(hidden, non_blocking=True)
        if self.graph is not None:
            self.graph.replay()
        else:
            self.launch()
        return self.out, self.logits, self.topk_ids, self.topk_weights

    def timed(self) -> list[float]:
        """One call with CUDA events between the stages; waits; returns the stage times in ms."""
        ms = (C.c_float * 12)()
        n = C.c_int(0)
        _lib.check(self.lib.fk_moe_layer_timed(C.byref(self.call), torch.cuda.current_stream().cuda_stream, ms,
                                               C.byref(n)), "fk_moe_layer_timed")
        return [ms[i] for i in range(n.value)]

    # ------------------------------------------------------------------ host input / output
    def run_host(self, hidden_host: torch.Tensor, out_host: torch.Tensor, ids_host: Optional[torch.Tensor] = None,
                 weights_host: Optional[torch.Tensor] = None, logits_host: Optional[torch.Tensor] = None) -> None:
        """Host buffers in, host buffers out (pinned memory recommended); copies and kernels are enqueued
        on the current stream.  Synchronise the stream before reading the outputs."""
        if self._staging is None:
            n = self.lib.fk_moe_host_staging_bytes(C.byref(self.call.dims), self.call.hidden_dtype)
            self._staging = torch.empty(n, dtype=torch.uint8, device=self.device)
        hc = Call.from_buffer_copy(self.call)
        if hidden_host.dtype != self.hidden_dtype or tuple(hidden_host.shape) != (self.tokens, self.hidden_size):
            raise ValueError("hidden_host must match the plan's [tokens, hidden] and dtype")
        if hidden_host.is_cuda or out_host.is_cuda:
            raise ValueError("run_host takes host tensors")
        hc.hidden = hidden_host.data_ptr()
        hc.out = out_host.data_ptr()
        hc.layer_hidden = None
        hc.logits = _ptr(logits_host)
        hc.topk_ids = _ptr(ids_host)
        hc.topk_weights = _ptr(weights_host)
        _lib.check(self.lib.fk_moe_layer_host(C.byref(hc), self._staging.data_ptr(), self._staging.numel(),
                                              torch.cuda.current_stream().cuda_stream), "fk_moe_layer_host")

    def capture_host(self) -> None:
        """Capture the host-buffer call (copy in, layer, copies out) into one CUDA graph over pinned buffers owned
        by the plan.  The eager `run_host` enqueues nine stream operations from Python per call, which costs more
        host time than the layer takes on the GPU at decode sizes; a replay is one launch."""
        T, H, k = self.tokens, self.hidden_size, self.top_k
        self.host_in = torch.empty((T, H), dtype=self.hidden_dtype).pin_memory()
        self.host_out = torch.empty((T, H), dtype=torch.float32).pin_memory()
        self.host_ids = torch.empty((T, k), dtype=torch.int64).pin_memory()
        self.host_weights = torch.empty((T, k), dtype=torch.float32).pin_memory()
        self.host_in.zero_()
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self.run_host(self.host_in, self.host_out, self.host_ids, self.host_weights)      # allocates the staging
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.run_host(self.host_in, self.host_out, self.host_ids, self.host_weights)
        self.host_graph = g

    def run_host_graph(self, hidden_host: torch.Tensor):
        """`hidden_host` (host, [T,H]) -> `(out, topk_ids, topk_weights)` in the plan's pinned host buffers, valid once
        the current stream has been synchronised; overwritten by the next call."""
        if getattr(self, "host_graph", None) is None:
            self.capture_host()
        self.host_in.copy_(hidden_host)
        self.host_graph.replay()
        return self.host_out, self.host_ids, self.host_weights

