"""Expert-parallel MoE layer over one node: experts block-sharded over the ranks of a process group.

The reference has no distributed code at all (no torch.distributed, NCCL or MPI call site
anywhere in suryavanshi/fastkernels); its plan lists expert-parallel dispatch as future work
(docs/QWEN35_KERNEL_PLAN.md:83).  The single-device semantics this module must reproduce are
those of `qwen36_real_moe_update` (src/fastkernels/reference/qwen36_real.py:329-354) applied
to the concatenation of all ranks' tokens.

Layout: rank r owns experts [r*E/G, (r+1)*E/G) (slices of expert_gate_up_weight / expert_down_weight
along dim 0).  Norm, router, shared expert and shared gate are replicated.  Every rank routes its
own T tokens.

One layer call, per rank (all shapes fixed, so the sequence can be captured in a CUDA graph and
needs no host synchronisation):
  1. router on the local tokens -> ids, weights                      (fk_moe_router)
  2. dispatch: all-gather of hidden rows, ids and weights             (NCCL)
     A token goes to every rank that owns one of its 8 experts (5.3 of 8 ranks on average), so
     the fixed-shape gather moves 1.5x the rows a routed all-to-all would, and in exchange
     needs no split-size exchange.
  3. local experts on all G*T tokens, foreign ids skipped, routing weights applied, slots in order,
     plus the gated shared expert for the rank's own tokens         (one fk_moe_experts call,
                                                                      FK_FLAG_SKIP_FOREIGN, shared_token_base/count)
  4. combine: all-to-all of the per-rank partial rows back to the tokens' home ranks   (NCCL)
  5. home rank: the G partials of a token summed (+ residual)
Results do not depend on scheduling: every sum has a fixed order.

The exchange code is backend-agnostic (gloo on CPU in the tests); the compute steps default to
the CUDA library and can be replaced by callables for those tests.  There is no silent fallback:
without CUDA tensors and without explicit callables the call raises.

Two exchanges are implemented.  `ep_moe_layer` is the portable one (NCCL on GPUs, gloo in the CPU tests).
`PeerEPLayer` replaces it on one NVLink node: every rank maps every other rank's exchange buffer (CUDA IPC) and
the library's kernels store activations, routing and partial rows straight into the peers' memory and exchange
arrival flags themselves (`fk_moe_layer_ep`, csrc/ep_p2p.cu): one C call per layer, no collective library, no
torch glue kernels, capturable in a CUDA graph.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.distributed as dist

from . import _lib
from .spec import MoEWeights


@dataclass
class EPShard:
    """This rank's slice of one layer: `weights.expert_*` hold only the local experts."""

    weights: MoEWeights
    rank: int
    world: int
    num_experts: int            # global E

    @property
    def local_experts(self) -> int:
        return self.num_experts // self.world

    @property
    def expert_base(self) -> int:
        return self.rank * self.local_experts


def shard_weights(full: MoEWeights, rank: int, world: int) -> EPShard:
    """Slice a full layer's routed experts for `rank` (views, no copy); everything else is shared."""
    E = full.expert_gate_up_weight.shape[0]
    if E % world:
        raise ValueError("number of experts must be divisible by the number of ranks")
    lo, hi = rank * (E // world), (rank + 1) * (E // world)
    w = MoEWeights(full.norm_weight, full.router_weight, full.expert_gate_up_weight[lo:hi], full.expert_down_weight[lo:hi],
                   full.shared_gate_up_weight, full.shared_down_weight, full.shared_expert_gate_weight, full.router_bias)
    return EPShard(w, rank, world, E)


# --------------------------------------------------------------------------- default compute steps
def _cuda_router(hidden, w: MoEWeights, top_k, eps):
    from .moe import qwen36_batched_moe_router_decode
    return qwen36_batched_moe_router_decode(hidden, w.norm_weight, w.router_weight, top_k=top_k, eps=eps,
                                            router_bias=w.router_bias)


def _cuda_local_experts(hidden_all, ids_all, weights_all, shard: EPShard, own: tuple):
    """Local routed experts for every gathered token plus the (gated) shared expert for this rank's own
    tokens `[own[0], own[0] + own[1])`, in one library call."""
    from .moe import _experts
    w = shard.weights
    return _experts(hidden_all, ids_all, weights_all, w.expert_gate_up_weight, w.expert_down_weight,
                    w.shared_gate_up_weight, w.shared_down_weight, w.shared_expert_gate_weight,
                    flags=_lib.FLAG_SKIP_FOREIGN, expert_base=shard.expert_base,
                    shared_token_range=own if w.shared_gate_up_weight is not None else None)


# --------------------------------------------------------------------------- the layer
def ep_moe_layer(hidden: torch.Tensor, shard: EPShard, *, top_k: int = 8, eps: float = 1e-6,
                 group: Optional[dist.ProcessGroup] = None, residual: bool = False,
                 router_fn: Optional[Callable] = None, local_experts_fn: Optional[Callable] = None):
    """One expert-parallel layer call for this rank's `hidden [T,H]`.

    Returns `(output [T,H] f32, logits [T,E] f32, topk_ids [T,k] i64, topk_weights [T,k] f32)`;
    `output` includes the residual when `residual=True`.
    `router_fn` / `local_experts_fn` exist for the CPU (gloo) tests of the exchange logic only, which pass the
    oracle's compute there; nothing in the product passes them, and without CUDA tensors the call raises.
    """
    if hidden.ndim != 2:
        raise ValueError("hidden must have shape [tokens, hidden_size]")
    world = dist.get_world_size(group)
    if world != shard.world:
        raise ValueError("shard was built for a different world size")
    if not hidden.is_cuda and (router_fn is None or local_experts_fn is None):
        raise RuntimeError("expert-parallel MoE needs CUDA tensors: there is no CPU path in the product")
    router_fn = router_fn or _cuda_router
    local_experts_fn = local_experts_fn or _cuda_local_experts
    w = shard.weights
    T, H = hidden.shape

    logits, ids, weights = router_fn(hidden, w, top_k, eps)

    # dispatch (fixed shape): every rank sees every token and its routing.  ids and weights travel in one
    # int32 buffer (weights bit-cast), so the dispatch is two collectives.
    routing = torch.cat([ids.to(torch.int32), weights.contiguous().view(torch.int32)], dim=1).contiguous()
    hidden_all = torch.empty((world * T, H), dtype=hidden.dtype, device=hidden.device)
    routing_all = torch.empty((world * T, 2 * top_k), dtype=torch.int32, device=hidden.device)
    dist.all_gather_into_tensor(hidden_all, hidden.contiguous(), group=group)
    dist.all_gather_into_tensor(routing_all, routing, group=group)
    ids_all = routing_all[:, :top_k].to(torch.int64)
    weights_all = routing_all[:, top_k:].contiguous().view(torch.float32)

    rank = dist.get_rank(group)
    partial = local_experts_fn(hidden_all, ids_all, weights_all, shard, (rank * T, T))     # [world*T, H] f32

    # combine: rows go back to their home rank; chunk g of `recv` is rank g's partial for our tokens
    recv = torch.empty_like(partial)
    dist.all_to_all_single(recv, partial.contiguous(), group=group)
    out = recv.view(world, T, H).sum(dim=0)                # one kernel, the same order on every call
    if residual:
        out += hidden.float()
    return out, logits, ids, weights


def ep_payload_bytes(tokens: int, hidden_size: int, top_k: int, world: int, hidden_bytes: int = 2) -> dict:
    """Bytes one rank sends per layer call (what crosses NVLink), for the roofline of the exchange."""
    remote = world - 1
    return {
        "dispatch": remote * tokens * (hidden_size * hidden_bytes + top_k * 12),
        "combine": remote * tokens * hidden_size * 4,
    }


class EPDecodePlan:
    """One rank's expert-parallel layer call with fixed shapes, captured in a CUDA graph.

    The eager `ep_moe_layer` issues a dozen small launches and three collectives from Python; at
    decode sizes that host work is longer than the GPU work.  Every shape in the exchange is fixed, so
    the whole call (router, gathers, local experts, all-to-all, rank-ordered sum) is captured once and
    replayed.  All ranks must construct and run their plans in the same order.
    """

    def __init__(self, shard: EPShard, tokens: int, *, hidden_dtype=torch.bfloat16, top_k: int = 8, eps: float = 1e-6,
                 residual: bool = False, group: Optional[dist.ProcessGroup] = None, capture: bool = True):
        self.shard, self.group, self.top_k, self.eps, self.residual = shard, group, top_k, eps, residual
        dev = shard.weights.expert_gate_up_weight.device
        H = shard.weights.router_weight.shape[1]
        self.hidden = torch.zeros((tokens, H), dtype=hidden_dtype, device=dev)
        self.graph = None
        self.out = self.logits = self.topk_ids = self.topk_weights = None
        # warm-up outside capture: NCCL channels, workspaces, kernel attributes
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self._call()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize(dev)
        if capture:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._call()
            self.graph = g

    def _call(self):
        self.out, self.logits, self.topk_ids, self.topk_weights = ep_moe_layer(
            self.hidden, self.shard, top_k=self.top_k, eps=self.eps, group=self.group, residual=self.residual)

    def run(self, hidden: Optional[torch.Tensor] = None):
        """Returns `(out, logits, topk_ids, topk_weights)`; the tensors are reused by the next run."""
        if hidden is not None:
            self.hidden.copy_(hidden, non_blocking=True)
        if self.graph is not None:
            self.graph.replay()
        else:
            self._call()
        return self.out, self.logits, self.topk_ids, self.topk_weights


# --------------------------------------------------------------------------- exchange over peer memory
class PeerExchange:
    """This rank's exchange buffer plus the mapped buffers of all other ranks (one node, one process per GPU).

    Built collectively: every rank of `group` must construct it with the same arguments.  The IPC handles travel
    through the process group once; afterwards no collective call is made.
    """

    def __init__(self, tokens_per_rank: int, hidden_size: int, top_k: int, hidden_dtype: torch.dtype,
                 group: Optional[dist.ProcessGroup] = None):
        self.lib = _lib.load()
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > _lib.EP_MAX_RANKS:
            raise ValueError(f"at most {_lib.EP_MAX_RANKS} ranks")
        code = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}[hidden_dtype]
        self.bytes = self.lib.fk_ep_buffer_bytes(self.world, tokens_per_rank, hidden_size, top_k, code)
        if self.bytes == 0:
            raise ValueError("exchange buffer: arguments outside the supported limits")
        own = C.c_void_p()
        handle = C.create_string_buffer(_lib.EP_HANDLE_BYTES)
        created = None
        try:
            _lib.check(self.lib.fk_ep_buffer_create(self.bytes, C.byref(own), handle), "fk_ep_buffer_create")
        except RuntimeError as exc:              # reported to every rank below, so that nobody waits for this one
            created = str(exc)
        self.own = own.value
        handles = [None] * self.world
        dist.all_gather_object(handles, created if created is not None else bytes(handle.raw), group=group)
        if any(isinstance(h, str) for h in handles):
            if self.own:
                self.lib.fk_ep_buffer_destroy(self.own)
            self.own = None
            raise RuntimeError("peer memory exchange unavailable: " +
                               "; ".join(f"rank {i}: {h}" for i, h in enumerate(handles) if isinstance(h, str)))
        self.comm = _lib.EpComm()
        self.comm.rank, self.comm.world, self.comm.tokens_per_rank, self.comm.bytes = self.rank, self.world, tokens_per_rank, self.bytes
        self._opened = []
        failure = None
        for r in range(self.world):
            if r == self.rank:
                self.comm.base[r] = self.own
                continue
            ptr = C.c_void_p()
            try:
                _lib.check(self.lib.fk_ep_buffer_open(C.create_string_buffer(handles[r], _lib.EP_HANDLE_BYTES), C.byref(ptr)),
                           "fk_ep_buffer_open")
            except RuntimeError as exc:          # e.g. no peer access between the two GPUs
                failure = str(exc)
                break
            self.comm.base[r] = ptr.value
            self._opened.append(ptr.value)
        # every rank learns whether every rank has mapped every buffer, before anyone stores into one (and so that a
        # failure on one rank does not leave the others waiting)
        outcomes = [None] * self.world
        dist.all_gather_object(outcomes, failure, group=group)
        if any(o is not None for o in outcomes):
            for ptr in self._opened:
                self.lib.fk_ep_buffer_close(ptr)
            self._opened = []
            dist.barrier(group=group)
            self.lib.fk_ep_buffer_destroy(self.own)
            self.own = None
            raise RuntimeError("peer memory exchange unavailable: " + "; ".join(f"rank {i}: {o}" for i, o in enumerate(outcomes) if o))

    def error(self) -> int:
        """Synchronises the device; non-zero if a wait on a peer ever gave up (1: dispatch, 2: combine)."""
        e = C.c_int(0)
        _lib.check(self.lib.fk_ep_status(C.byref(self.comm), C.byref(e)), "fk_ep_status")
        return e.value

    def close(self, collective: bool = True) -> None:
        """Unmaps the peers' buffers and frees the own one once every rank has unmapped it (a barrier on the process
        group).  `collective=False` skips that barrier: for a shutdown after a failure, when the caller has already
        established on the host that no rank will touch the buffers again (or that a rank is gone)."""
        if self.own is None:
            return
        torch.cuda.synchronize()
        for ptr in self._opened:
            self.lib.fk_ep_buffer_close(ptr)
        self._opened = []
        if collective:
            dist.barrier(group=self.group)
        self.lib.fk_ep_buffer_destroy(self.own)
        self.own = None


class PeerEPLayer:
    """One rank's expert-parallel layer call over peer memory, shapes fixed, optionally one CUDA graph.

    Same results as `ep_moe_layer` (the partial rows are summed in rank order on the home rank)."""

    def __init__(self, shard: EPShard, exchange: PeerExchange, tokens: int, *, hidden_dtype=torch.bfloat16, top_k: int = 8,
                 eps: float = 1e-6, residual: bool = False, capture: bool = True, hidden_buffer: Optional[torch.Tensor] = None,
                 out_buffer: Optional[torch.Tensor] = None, warmup: bool = True):
        from ._lib import Call, Dims
        from .plan import _DTYPES, _as_weight, _ptr
        self.lib, self.exchange, self.shard = _lib.load(), exchange, shard
        w = shard.weights
        dev = w.expert_gate_up_weight.device
        wdt = w.expert_gate_up_weight.dtype
        E_local, two_i, H = w.expert_gate_up_weight.shape
        E = shard.num_experts
        if E_local * shard.world != E or shard.world != exchange.world or shard.rank != exchange.rank:
            raise ValueError("shard and exchange disagree about the ranks")
        self._keep = [_as_weight(w.norm_weight, wdt), _as_weight(w.router_weight, wdt), w.expert_gate_up_weight.contiguous(),
                      _as_weight(w.expert_down_weight, wdt), _as_weight(w.shared_gate_up_weight, wdt),
                      _as_weight(w.shared_down_weight, wdt), _as_weight(w.shared_expert_gate_weight, wdt),
                      None if w.router_bias is None else w.router_bias.to(device=dev, dtype=torch.float32).contiguous()]
        # buffers may be shared between the layers of a stack
        self.hidden = hidden_buffer if hidden_buffer is not None else torch.zeros((tokens, H), dtype=hidden_dtype, device=dev)
        self.out = out_buffer if out_buffer is not None else torch.empty((tokens, H), dtype=torch.float32, device=dev)
        self.layer_hidden = torch.empty_like(self.out) if residual else None
        self.logits = torch.empty((tokens, E), dtype=torch.float32, device=dev)
        self.topk_ids = torch.empty((tokens, top_k), dtype=torch.int64, device=dev)
        self.topk_weights = torch.empty((tokens, top_k), dtype=torch.float32, device=dev)
        need = max(self.lib.fk_moe_workspace_bytes(C.byref(Dims(shard.world * tokens, H, E_local, two_i // 2, top_k))),
                   self.lib.fk_moe_workspace_bytes(C.byref(Dims(tokens, H, E, two_i // 2, top_k))))
        if need == 0:
            raise ValueError("MoE dims outside the supported limits")
        self.workspace = torch.zeros(need, dtype=torch.uint8, device=dev)
        call = Call()
        call.dims = Dims(tokens, H, E, two_i // 2, top_k)
        call.hidden_dtype, call.weight_dtype = _DTYPES[hidden_dtype], _DTYPES[wdt]
        call.eps, call.norm_offset, call.flags, call.expert_base = eps, 1.0, 0, 0
        (call.norm_weight, call.router_weight, call.expert_gate_up, call.expert_down, call.shared_gate_up,
         call.shared_down, call.shared_gate, call.router_bias) = [_ptr(t) for t in self._keep]
        call.hidden, call.out, call.layer_hidden = _ptr(self.hidden), _ptr(self.out), _ptr(self.layer_hidden)
        call.logits, call.topk_ids, call.topk_weights = _ptr(self.logits), _ptr(self.topk_ids), _ptr(self.topk_weights)
        call.workspace, call.workspace_bytes = self.workspace.data_ptr(), self.workspace.numel()
        self.call = call
        self.graph = None
        if not warmup:
            return
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.launch()                       # all ranks make this call: the exchange is collective
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize(dev)
        if capture:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self.launch()
            self.graph = g

    def launch(self) -> None:
        _lib.check(self.lib.fk_moe_layer_ep(C.byref(self.call), C.byref(self.exchange.comm), torch.cuda.current_stream().cuda_stream),
                   "fk_moe_layer_ep")

    def timed(self) -> list[float]:
        """One eager call with CUDA events between its stages (collective: every rank makes it); waits; stage times in
        ms: router, dispatch + wait, permutation, [row gather], gate_up, down, combine + wait, reduce."""
        ms = (C.c_float * 12)()
        n = C.c_int(0)
        _lib.check(self.lib.fk_moe_layer_ep_timed(C.byref(self.call), C.byref(self.exchange.comm),
                                                  torch.cuda.current_stream().cuda_stream, ms, C.byref(n)), "fk_moe_layer_ep_timed")
        return [ms[i] for i in range(n.value)]

    def run(self, hidden: Optional[torch.Tensor] = None):
        """Returns `(out, logits, topk_ids, topk_weights)`; `out` includes the residual when asked for at construction."""
        if hidden is not None:
            self.hidden.copy_(hidden, non_blocking=True)
        if self.graph is not None:
            self.graph.replay()
        else:
            self.launch()
        return (self.layer_hidden if self.layer_hidden is not None else self.out), self.logits, self.topk_ids, self.topk_weights

