"""CPU, world size 2 and 4 over gloo: the expert-parallel exchange (gather dispatch, all-to-all combine,
rank-ordered sum) reproduces the single-device oracle on the concatenated batch.  The compute steps
are the oracle's, injected through the callables `ep_moe_layer` takes for this purpose."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import moe_oracle as O
from fastkernels_b200.ep import ep_moe_layer, ep_payload_bytes, shard_weights
from fastkernels_b200.spec import MoESpec
from fastkernels_b200.workloads import make_hidden, make_moe_weights

SPEC = MoESpec(hidden_size=64, num_experts=8, num_routed_experts=2, expert_intermediate_size=32)


def _router(hidden, w, top_k, eps):
    return O.router(hidden, w.norm_weight, w.router_weight, top_k=top_k, eps=eps, router_bias=w.router_bias)


def _local(hidden_all, ids_all, weights_all, shard, own):
    local = ids_all - shard.expert_base
    mine = (local >= 0) & (local < shard.local_experts)
    ids = torch.where(mine, local, torch.zeros_like(local))
    wts = torch.where(mine, weights_all, torch.zeros_like(weights_all))
    w = shard.weights
    out = O.routed_experts(hidden_all, ids, wts, w.expert_gate_up_weight, w.expert_down_weight)
    sl = slice(own[0], own[0] + own[1])
    out[sl] += O.shared_expert(hidden_all[sl], w.shared_gate_up_weight, w.shared_down_weight, w.shared_expert_gate_weight)
    return out


def _worker(rank, world, port, tokens, failures):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        full = make_moe_weights(3, SPEC, dtype=torch.float32, bias_std=0.5)
        shard = shard_weights(full, rank, world)
        assert shard.weights.expert_gate_up_weight.shape[0] == SPEC.num_experts // world
        hidden = make_hidden(50 + rank, tokens, SPEC, dtype=torch.float32)
        out, logits, ids, weights = ep_moe_layer(hidden, shard, top_k=2, residual=True, router_fn=_router,
                                                 local_experts_fn=_local)
        # single-device oracle on the gathered batch
        all_hidden = torch.cat([make_hidden(50 + r, tokens, SPEC, dtype=torch.float32) for r in range(world)])
        ref = O.moe_update(all_hidden, *full.tuple(), top_k=2, router_bias=full.router_bias)
        sl = slice(rank * tokens, (rank + 1) * tokens)
        assert torch.equal(ids, ref.topk_ids[sl]), "routing differs from the single-device oracle"
        assert torch.equal(logits, ref.logits[sl])
        torch.testing.assert_close(out, all_hidden[sl] + ref.output[sl], atol=1e-5, rtol=1e-5)
        # histogram over all ranks == oracle histogram
        hist = O.expert_histogram(ids, SPEC.num_experts).to(torch.int64)
        dist.all_reduce(hist)
        assert torch.equal(hist.to(torch.int32), ref.histogram)
    except Exception as exc:  # noqa: BLE001
        failures.put(f"rank {rank}: {exc!r}")
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world,tokens", [(2, 5), (4, 3)])
def test_ep_exchange_matches_single_device_oracle(world, tokens):
    ctx = mp.get_context("spawn")
    failures = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, tokens, failures)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    msgs = []
    while not failures.empty():
        msgs.append(failures.get())
    assert not msgs, msgs
    assert all(p.exitcode == 0 for p in procs)


def test_ep_rejects_cpu_tensors_without_explicit_compute():
    # no process group needed: the check comes first... it needs the world size, so use a 1-rank group
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(_free_port())
    dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        full = make_moe_weights(3, SPEC, dtype=torch.float32)
        with pytest.raises(RuntimeError, match="no CPU path"):
            ep_moe_layer(make_hidden(1, 2, SPEC, dtype=torch.float32), shard_weights(full, 0, 1), top_k=2)
    finally:
        dist.destroy_process_group()


def test_payload_bytes():
    b = ep_payload_bytes(256, 2048, 8, 8)
    assert b["dispatch"] == 7 * 256 * (4096 + 96) and b["combine"] == 7 * 256 * 2048 * 4
