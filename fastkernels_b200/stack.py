"""A stack of MoE layers run back to back: x <- x + MoE_l(RMSNorm(x)), unit-gain norm, eps 1e-6.

This is the decode loop of the benchmark's 40-layer configuration with the sequence mixers left
out.  The reference composes its layers in Python, one call and one residual add per layer
(src/fastkernels/kernels/triton/qwen36_layer.py:55-106; the streaming runner
bench/qwen36_full_decode.py:409-419 reloads the weights of every layer from disk).  Here all
layers stay resident in HBM, the residual add and the next layer's norm are one kernel
(fk_residual_rmsnorm), and the whole stack is one CUDA graph.

The residual stream `x` is fp32; the normed activations handed to each layer are bf16.
Works on one GPU (`MoEWeights` per layer) or expert parallel (`EPShard` per layer plus a group).
"""

from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from . import _lib
from .plan import MoEDecodePlan


class MoEStackPlan:
    def __init__(self, layers: Sequence, tokens: int, *, top_k: int = 8, eps: float = 1e-6, norm_eps: float = 1e-6,
                 act_dtype: torch.dtype = torch.bfloat16, group=None, capture: bool = True, flags: int = 0, exchange=None,
                 fused_residual: bool = True):
        from .ep import EPShard
        self.lib = _lib.load()
        self.layers = list(layers)
        self.ep = isinstance(self.layers[0], EPShard)
        w0 = self.layers[0].weights if self.ep else self.layers[0]
        dev = w0.expert_gate_up_weight.device
        H = w0.router_weight.shape[1]
        self.device, self.tokens, self.hidden_size = dev, tokens, H
        self.top_k, self.eps, self.norm_eps, self.group = top_k, eps, norm_eps, group
        self.act_code = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}[act_dtype]
        self.x = torch.zeros((tokens, H), device=dev, dtype=torch.float32)        # residual stream (input and output)
        self.xin = torch.zeros((tokens, H), device=dev, dtype=act_dtype)          # normed activations of the current layer
        self.topk_ids = []
        self.graph = None
        self.exchange = exchange
        self.result = self.x
        self.fused_residual = False
        if not self.ep:
            self.update = torch.zeros((tokens, H), device=dev, dtype=torch.float32)
            self.plans = [MoEDecodePlan(w, tokens, hidden_dtype=act_dtype, top_k=top_k, eps=eps, flags=flags,
                                        hidden_buffer=self.xin, out_buffer=self.update) for w in self.layers]
            if tokens == 1 and fused_residual:
                # one token: the residual add and the norm move into the layer's own kernel (one launch per layer); the
                # residual stream then alternates between two buffers, because a block of that kernel stores its slice
                # of the new stream while other blocks still read the old one
                self.x_alt = torch.zeros_like(self.x)
                st = self.lib.fk_moe_layer_residual(C.byref(self.plans[0].call), self.x.data_ptr(), None, self.x_alt.data_ptr(),
                                                    self.norm_eps, torch.cuda.current_stream().cuda_stream)
                torch.cuda.synchronize(dev)
                if st == 0:
                    self.fused_residual = True
                    self.result = self.x if len(self.layers) % 2 == 0 else self.x_alt
                elif st != 2:                        # 2 = unsupported shape: keep the two-kernel form
                    _lib.check(st, "fk_moe_layer_residual")
        elif exchange is not None:
            # expert parallel over peer memory: every layer's call uses the same exchange buffers, one after the other
            from .ep import PeerEPLayer
            self.update = torch.zeros((tokens, H), device=dev, dtype=torch.float32)
            self.plans = [PeerEPLayer(sh, exchange, tokens, hidden_dtype=act_dtype, top_k=top_k, eps=eps, capture=False,
                                      hidden_buffer=self.xin, out_buffer=self.update, warmup=False) for sh in self.layers]
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self._forward()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize(dev)
        if capture:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._forward()
            self.graph = g

    def _norm(self, update: Optional[torch.Tensor]) -> None:
        st = self.lib.fk_residual_rmsnorm(self.x.data_ptr(), None if update is None else update.data_ptr(), self.xin.data_ptr(),
                                          self.act_code, self.tokens, self.hidden_size, self.norm_eps,
                                          torch.cuda.current_stream().cuda_stream)
        _lib.check(st, "fk_residual_rmsnorm")

    def _forward(self) -> None:
        from .ep import ep_moe_layer
        update = None
        self.topk_ids = []
        if self.fused_residual:
            bufs = (self.x, self.x_alt)
            stream = torch.cuda.current_stream().cuda_stream
            for i, plan in enumerate(self.plans):
                st = self.lib.fk_moe_layer_residual(C.byref(plan.call), bufs[i % 2].data_ptr(),
                                                    None if i == 0 else self.update.data_ptr(), bufs[(i + 1) % 2].data_ptr(),
                                                    self.norm_eps, stream)
                _lib.check(st, "fk_moe_layer_residual")
                self.topk_ids.append(plan.topk_ids)
            st = self.lib.fk_residual_rmsnorm(self.result.data_ptr(), self.update.data_ptr(), self.xin.data_ptr(), self.act_code,
                                              self.tokens, self.hidden_size, self.norm_eps, stream)
            _lib.check(st, "fk_residual_rmsnorm")           # the last update joins the stream
            return
        for i, layer in enumerate(self.layers):
            self._norm(update)                       # x += previous update; xin = RMSNorm(x)
            if self.ep and self.exchange is None:
                update, _, ids, _ = ep_moe_layer(self.xin, layer, top_k=self.top_k, eps=self.eps, group=self.group)
            else:
                self.plans[i].launch()
                update, ids = self.update, self.plans[i].topk_ids
            self.topk_ids.append(ids)
        self._norm(update)                           # x += last update (xin then holds the norm of the result)

    def run(self, x: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Runs the stack on `self.x` (copying `x` in first if given) and returns the residual stream after the last
        layer: `self.x` itself, or the plan's second buffer in the single-token form with an odd number of layers."""
        if x is not None:
            self.x.copy_(x, non_blocking=True)
        if self.graph is not None:
            self.graph.replay()
        else:
            self._forward()
        return self.result


class ResidentMoELayers:
    """All MoE layers of a checkpoint packed once and kept in HBM, called layer by layer.

    This is the shape of the reference's decode loop at its MoE call site
    (bench/qwen36_full_decode.py:407-419: `hidden = triton_moe_layer(hidden, *weights, top_k=k)[0]`,
    where the reference reloads every layer's tensors from safetensors on every token): here the layers
    are packed from the checkpoint mapping once (`weights.pack_qwen36_moe_weights_from_state_dict`, in
    the compute dtype, straight onto the GPU), each layer owns a prepared call (`MoEDecodePlan`) for the
    fixed token count, and `layer(i, hidden)` returns the new residual stream `hidden + MoE_i(hidden)`.
    The sequence mixers between the MoE sublayers stay with the caller.
    """

    def __init__(self, layers: Sequence, tokens: int, *, hidden_dtype: torch.dtype = torch.bfloat16, top_k: int = 8,
                 eps: float = 1e-6, flags: int = 0):
        self.plans = [MoEDecodePlan(w, tokens, hidden_dtype=hidden_dtype, top_k=top_k, eps=eps, flags=flags, residual=True)
                      for w in layers]
        self.tokens = tokens

    @classmethod
    def from_state_dict(cls, tensors, layer_indices: Sequence[int], tokens: int, *, spec=None, device="cuda",
                        dtype: torch.dtype = torch.bfloat16, **kw) -> "ResidentMoELayers":
        from .weights import pack_qwen36_moe_weights_from_state_dict
        layers = [pack_qwen36_moe_weights_from_state_dict(tensors, i, spec=spec, device=device, dtype=dtype).weights
                  for i in layer_indices]
        return cls(layers, tokens, hidden_dtype=dtype, **kw)

    def layer(self, index: int, hidden: torch.Tensor) -> torch.Tensor:
        """`hidden [tokens, H]` in the plans' activation dtype -> fp32 `hidden + moe_update` (a view of the plan's
        buffer, overwritten by the next call of the same layer)."""
        plan = self.plans[index]
        plan.run(hidden)
        return plan.layer_hidden
