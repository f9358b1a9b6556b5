"""GPU, 2 ranks over NCCL (skipped with fewer than 2 devices): the expert-parallel layer with the CUDA
kernels matches the single-device oracle on the gathered batch, and the single-GPU layer bitwise in routing.

Shutdown is ordered even when a rank fails: the failure is recorded, the rank synchronises its device, meets
the other rank at a host-side barrier with a short limit (a TCP store, no GPU work), unmaps the peers' exchange
buffers and only then leaves the process group.  A rank that learns of the other's failure stops before its
next collective step.  The parent kills whatever is still alive after the time limit and fails the test."""

import datetime
import os
import socket
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

STEP_LIMIT_S = 60


class _Peers:
    """Host-side view of the other ranks: a failure flag and a barrier with a time limit, both on the TCP store."""

    def __init__(self, rank, world, port):
        self.rank, self.world = rank, world
        self.store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=STEP_LIMIT_S))

    def fail(self, text):
        self.store.set("failed", text)

    def someone_failed(self) -> bool:
        return self.store.check(["failed"])

    def barrier(self, name, limit_s=30.0) -> bool:
        self.store.add(name, 1)
        end = time.time() + limit_s
        while time.time() < end:
            if int(self.store.add(name, 0)) >= self.world:
                return True
            time.sleep(0.01)
        return False


def _init(rank, world, port):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=STEP_LIMIT_S))


def _shutdown(peers, exchanges, failures, rank):
    try:
        torch.cuda.synchronize()
    except Exception as exc:  # noqa: BLE001
        failures.put(f"rank {rank}: synchronize at shutdown: {exc!r}")
    together = peers.barrier("shutdown")           # nobody unmaps a buffer another rank may still store into
    for ex in exchanges:
        try:
            ex.close(collective=together)
        except Exception as exc:  # noqa: BLE001
            failures.put(f"rank {rank}: closing the exchange: {exc!r}")
    try:
        dist.destroy_process_group()
    except Exception:  # noqa: BLE001
        pass


def _check_against_oracle(O, out, ids, ref, what):
    """Per token: ids bit-exact wherever the oracle's cut is not a near-tie; outputs on the tokens whose ids agree;
    at most one token in 64 may be left out, and the count is part of the failure text."""
    clear = ref.margin > 2e-6
    ids_c = ids.cpu()
    assert torch.equal(ids_c[clear], ref.topk_ids[clear]), f"{what}: ids differ from the oracle"
    same = (ids_c == ref.topk_ids).all(dim=1)
    excluded = int((~same).sum())
    assert excluded <= max(1, ids_c.shape[0] // 64), f"{what}: {excluded} tokens route differently from the oracle"
    ma, rl = O.max_abs(out.cpu()[same], ref.output[same]), O.rel_l2(out.cpu()[same], ref.output[same])
    assert ma <= 2e-2 and rl <= 5e-3, (what, ma, rl, excluded)


def _check_against_single_gpu(O, out, single, tokens, world, what):
    """The expert-parallel result against the single-GPU layer on the rank's own tokens.  Both run the same kernels on
    the same rows when the gathered batch takes the same path as the rank's batch: equal up to fp32 summation order.
    From 64 tokens on a call takes the grouped GEMM, which rounds the SwiGLU activations to bf16 (as does the
    single-launch kernel for two to four tokens): when only one of the two calls does, they agree within the bf16
    output bounds."""
    def rounds_activations(n):          # two to four tokens (single launch) and 64 or more (grouped GEMM) keep them in bf16
        return 2 <= n <= 4 or n >= 64
    same_path = rounds_activations(world * tokens) == rounds_activations(tokens)
    if same_path:
        torch.testing.assert_close(out, single, atol=2e-5, rtol=1e-4)
    else:
        ma, rl = O.max_abs(out.cpu(), single.cpu()), O.rel_l2(out.cpu(), single.cpu())
        assert ma <= 2e-2 and rl <= 5e-3, (what, ma, rl)


def _worker(rank, world, port, store_port, tokens, failures):
    _init(rank, world, port)
    peers = _Peers(rank, world, store_port)
    try:
        from oracle import moe_oracle as O
        from fastkernels_b200.ep import ep_moe_layer, shard_weights
        from fastkernels_b200.moe import qwen36_batched_moe_decode
        from fastkernels_b200.spec import MoESpec
        from fastkernels_b200.workloads import make_hidden, make_moe_weights
        spec = MoESpec()
        full = make_moe_weights(4, spec, dtype=torch.bfloat16, device="cuda", bias_std=0.5)
        shard = shard_weights(full, rank, world)
        hidden = make_hidden(70 + rank, tokens, spec, dtype=torch.bfloat16, device="cuda")
        out, logits, ids, weights = ep_moe_layer(hidden, shard, top_k=8)
        out2, _, ids2, _ = ep_moe_layer(hidden, shard, top_k=8)
        assert torch.equal(out, out2) and torch.equal(ids, ids2), "not repeatable"
        single, _, ids1, _ = qwen36_batched_moe_decode(hidden, *full.tuple(), router_bias=full.router_bias)
        assert torch.equal(ids, ids1), "routing differs between one GPU and expert parallel"
        _check_against_single_gpu(O, out, single, tokens, world, "NCCL exchange")
        cpu = [None if t is None else t.cpu() for t in full.tuple()]
        ref = O.moe_update(hidden.cpu(), *cpu, top_k=8, router_bias=full.router_bias.cpu())
        _check_against_oracle(O, out, ids, ref, "NCCL exchange")
    except Exception as exc:  # noqa: BLE001
        failures.put(f"rank {rank}: {exc!r}")
        peers.fail(repr(exc))
    finally:
        _shutdown(peers, [], failures, rank)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(target, world, *args, limit_s=300):
    ctx = mp.get_context("spawn")
    failures = ctx.Queue()
    port, store_port = _free_port(), _free_port()
    procs = [ctx.Process(target=target, args=(r, world, port, store_port, *args, failures)) for r in range(world)]
    for p in procs:
        p.start()
    end = time.time() + limit_s
    for p in procs:
        p.join(max(1.0, end - time.time()))
    stragglers = [i for i, p in enumerate(procs) if p.is_alive()]
    for i in stragglers:                       # nothing of ours stays on the shared GPU after the test
        procs[i].kill()
        procs[i].join(30)
    msgs = []
    while not failures.empty():
        msgs.append(failures.get())
    assert not stragglers, f"ranks {stragglers} did not finish within {limit_s} s and were killed; {msgs}"
    assert not msgs, msgs
    assert all(p.exitcode == 0 for p in procs)


def test_ep_two_gpus_matches_oracle_and_single_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    _run(_worker, 2, 6)


def _peer_worker(rank, world, port, store_port, tokens, failures):
    """Expert parallel over peer memory (no collective library in the layer call) against the NCCL exchange and
    the single-GPU layer; eager and as a replayed CUDA graph, several calls with changing inputs."""
    _init(rank, world, port)
    peers = _Peers(rank, world, store_port)
    exchanges = []
    try:
        from oracle import moe_oracle as O
        from fastkernels_b200.ep import PeerEPLayer, PeerExchange, ep_moe_layer, shard_weights
        from fastkernels_b200.moe import qwen36_batched_moe_decode
        from fastkernels_b200.spec import MoESpec
        from fastkernels_b200.workloads import make_hidden, make_moe_weights
        spec = MoESpec()
        full = make_moe_weights(4, spec, dtype=torch.bfloat16, device="cuda", bias_std=0.5)
        cpu = [None if t is None else t.cpu() for t in full.tuple()]
        shard = shard_weights(full, rank, world)
        exchange = PeerExchange(tokens, spec.hidden_size, 8, torch.bfloat16)
        exchanges.append(exchange)
        for capture in (False, True):
            layer = PeerEPLayer(shard, exchange, tokens, capture=capture)
            # the replayed graph runs many steps with changing inputs: a flag that overtook its rows would show as a
            # mismatch with the collective-library exchange
            for step in range(24 if capture else 4):
                assert not peers.someone_failed(), "another rank failed"
                hidden = make_hidden(70 + rank + 10 * step, tokens, spec, dtype=torch.bfloat16, device="cuda")
                out, logits, ids, weights = layer.run(hidden)
                out, ids, weights = out.clone(), ids.clone(), weights.clone()
                ref_out, _, ref_ids, ref_w = ep_moe_layer(hidden, shard, top_k=8)
                assert torch.equal(ids, ref_ids) and torch.equal(weights, ref_w), f"routing differs (capture={capture}, step {step})"
                # same routed sums; the shared gate's dot product is taken by another kernel there (other summation order)
                torch.testing.assert_close(out, ref_out, atol=2e-5, rtol=1e-4)
                single, _, ids1, _ = qwen36_batched_moe_decode(hidden, *full.tuple(), router_bias=full.router_bias)
                assert torch.equal(ids, ids1)
                _check_against_single_gpu(O, out, single, tokens, world, f"peer memory (capture={capture}, step {step})")
                if step == 0:
                    ref = O.moe_update(hidden.cpu(), *cpu, top_k=8, router_bias=full.router_bias.cpu())
                    _check_against_oracle(O, out, ids, ref, f"peer memory (capture={capture})")
            assert exchange.error() == 0
        # top-2 routing: half of the tokens have both experts on one rank, so the other rank sends no row for them
        # and the home rank must leave that slot out of its sum
        ex2 = PeerExchange(tokens, spec.hidden_size, 2, torch.bfloat16)
        exchanges.append(ex2)
        layer2 = PeerEPLayer(shard, ex2, tokens, top_k=2)
        lonely = 0
        for step in range(3):
            assert not peers.someone_failed(), "another rank failed"
            hidden = make_hidden(170 + rank + 10 * step, tokens, spec, dtype=torch.bfloat16, device="cuda")
            out, _, ids, weights = layer2.run(hidden)
            out, ids = out.clone(), ids.clone()
            ref_out, _, ref_ids, _ = ep_moe_layer(hidden, shard, top_k=2)
            assert torch.equal(ids, ref_ids)
            torch.testing.assert_close(out, ref_out, atol=2e-5, rtol=1e-4)
            lonely += int(((ids // (spec.num_experts // world)).min(dim=1).values ==
                           (ids // (spec.num_experts // world)).max(dim=1).values).sum())
        assert ex2.error() == 0
        assert tokens < 16 or lonely > 0, "no token was routed to a single rank: the case was not exercised"
        del layer2
        if tokens <= 8:
            # two-layer stack over the same exchange buffers against the single-GPU stack on the full weights
            from fastkernels_b200.stack import MoEStackPlan
            fulls = [full, make_moe_weights(5, spec, dtype=torch.bfloat16, device="cuda", bias_std=0.5)]
            x0 = make_hidden(90, tokens, spec, dtype=torch.float32, device="cuda")      # same tokens on every rank
            assert not peers.someone_failed(), "another rank failed"
            ep_stack = MoEStackPlan([shard_weights(f, rank, world) for f in fulls], tokens, exchange=exchange)
            got = ep_stack.run(x0).clone()
            got2 = ep_stack.run(x0).clone()
            assert torch.equal(got, got2), "stack over peer memory is not repeatable"
            one = MoEStackPlan(fulls, tokens)
            want = one.run(x0).clone()
            for a, b in zip(ep_stack.topk_ids, one.topk_ids):
                assert torch.equal(a, b)
            torch.testing.assert_close(got, want, atol=1e-4, rtol=1e-4)
            assert exchange.error() == 0
    except Exception as exc:  # noqa: BLE001
        failures.put(f"rank {rank}: {exc!r}")
        peers.fail(repr(exc))
    finally:
        _shutdown(peers, exchanges, failures, rank)


@pytest.mark.parametrize("tokens", [6, 40, 256])
def test_ep_two_gpus_over_peer_memory(tokens):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    _run(_peer_worker, 2, tokens)
