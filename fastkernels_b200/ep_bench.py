"""Expert-parallel leg of bench.py (N > 1): one process per GPU, NCCL over NVLink.

Weak scaling in tokens: every rank brings `--batch` tokens per step; the 256 experts are split
evenly, so each rank streams 1/N of the routed weights plus the replicated router and shared
expert.  Timing: barrier + synchronize on both sides of the K steps, CUDA events, maximum over ranks.
"""

from __future__ import annotations

import datetime
import json
import os
import statistics
import time

import torch
import torch.distributed as dist


def run_ep(args, workload_config, measured_peak, ClockSampler, METRIC, UNIT):
    from . import _lib
    from .ep import EPDecodePlan, ep_payload_bytes, EPShard, PeerEPLayer, PeerExchange
    from .spec import MoESpec
    from .workloads import make_hidden, make_moe_weights

    lib = _lib.load()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        # a rank that fails must not leave the others waiting for the default ten minutes
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=90))
    spec = MoESpec()
    peak, peak_src = measured_peak()
    B, K, W, L = args.batch, args.steps, max(args.warmup, 3), args.layers
    E, H, I = spec.num_experts, spec.hidden_size, spec.expert_intermediate_size
    per = E // world
    shards = []
    for layer in range(L):
        w = make_moe_weights(layer, spec, dtype=torch.bfloat16, device=dev, bias_std=0.5,
                             expert_range=(rank * per, (rank + 1) * per))
        shards.append(EPShard(w, rank, world, E))
    pool = 8
    hid_host = [make_hidden(1000 + i * world + rank, B, spec, dtype=torch.bfloat16).pin_memory() for i in range(pool)]
    hid_dev = [h.to(dev) for h in hid_host]

    # default: exchange over peer memory inside the library's own kernels; --ep-nccl: NCCL collectives from torch
    exchange = None
    exchange_note = None
    if not args.ep_nccl:
        try:
            exchange = PeerExchange(B, H, 8, torch.bfloat16)
        except RuntimeError as exc:              # raised on every rank together: fall back to the collective library
            exchange_note = str(exc)
            args.ep_nccl = True
    if args.ep_nccl:
        plans = [EPDecodePlan(sh, B, capture=not args.ep_eager) for sh in shards]
    else:
        plans = [PeerEPLayer(sh, exchange, B, capture=not args.ep_eager) for sh in shards]
    for i, pl in enumerate(plans):              # inputs are resident before the timed region starts
        pl.hidden.copy_(hid_dev[i % pool])

    def step(i, hidden=None):
        return plans[i % L].run(hidden)

    def timed(fn, steps):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        dist.barrier()
        t = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for i in range(W):
        step(i)
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    ms = timed(lambda i: step(i), K)
    # graph replays bypass the library's launch counter: count what one eager call enqueues
    c0 = lib.fk_launch_count()
    if args.ep_nccl:
        plans[0]._call()
    else:
        plans[0].launch()
    torch.cuda.synchronize()
    launches = (lib.fk_launch_count() - c0) * K

    # end to end: pinned host hidden in, output back to pinned host memory, every step
    out_host = torch.empty(B, H, dtype=torch.float32).pin_memory()
    stage = torch.empty(B, H, dtype=torch.bfloat16, device=dev)

    def e2e_step(i):
        stage.copy_(hid_host[i % pool], non_blocking=True)
        out, _, _, _ = step(i, stage)
        out_host.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for i in range(W):
        e2e_step(i)
    t0 = time.perf_counter()
    e2e_ms = timed(e2e_step, K)
    clocks = sampler.stop() if sampler else None

    # distinct local experts hit per step (for the per-rank algorithmic bytes)
    us = []
    for i in range(min(L, 3)):
        _, _, ids, _ = step(i)
        torch.cuda.synchronize()
        ids_all = torch.empty((world * B, 8), dtype=ids.dtype, device=dev)
        dist.all_gather_into_tensor(ids_all, ids)
        mine = ids_all[(ids_all >= rank * per) & (ids_all < (rank + 1) * per)]
        us.append(int(torch.unique(mine).numel()))
    u_local = statistics.mean(us)
    per_expert = 3 * H * I * 2
    rank_bytes = (u_local + 1) * per_expert + E * H * 2 + 2 * H * 2 + B * H * 2 + B * H * 4 + B * E * 4 + B * 8 * 12
    payload = ep_payload_bytes(B, H, 8, world)
    # optional: the layer stack (x <- x + MoE_l(RMSNorm(x))) expert parallel over the same peer-memory exchange
    stack = None
    if args.stack_layers > 0 and not args.ep_nccl:
        from .stack import MoEStackPlan
        del plans
        if exchange is not None:
            if exchange.error():
                raise RuntimeError("exchange error before the stack leg")
            exchange.close()
        torch.cuda.empty_cache()
        for layer in range(len(shards), args.stack_layers):
            w = make_moe_weights(layer, spec, dtype=torch.bfloat16, device=dev, bias_std=0.5,
                                 expert_range=(rank * per, (rank + 1) * per))
            shards.append(EPShard(w, rank, world, E))
        stack = {"layers": args.stack_layers, "runs": []}
        for tok in (1, 64):
            ex = PeerExchange(tok, H, 8, torch.bfloat16)
            sp = MoEStackPlan(shards[:args.stack_layers], tok, exchange=ex)
            x0 = make_hidden(3000 + tok + rank, tok, spec, dtype=torch.float32, device=dev)
            for _ in range(3):
                sp.run(x0)
            t_ms = timed(lambda i: sp.run(x0), 10)
            stack["runs"].append({"tokens_per_gpu": tok, "ms_per_stack_pass": t_ms, "us_per_layer": t_ms * 1e3 / args.stack_layers,
                                  "tokens_per_s": world * tok / (t_ms * 1e-3)})
            if ex.error():
                raise RuntimeError("exchange error in the stack leg")
            del sp
            ex.close()
        exchange = None
    if rank == 0:
        achieved = rank_bytes / (ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": world * B / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": workload_config(B, world, L),
            "roofline": {"bound": "hbm", "kernel": "per-rank layer call (router, local experts of all ranks' tokens, shared expert)",
                         "achieved": achieved, "peak": peak, "peak_source": peak_src, "unit": "GB/s", "frac": achieved / peak,
                         "algorithmic_bytes_per_launch": rank_bytes, "ms_per_launch": ms, "traffic": None,
                         "distinct_local_experts": u_local,
                         "nvlink_bytes_per_rank_per_step": payload,
                         "nvlink_floor_us": (max(payload["dispatch"], 0) + payload["combine"]) / 770e9 * 1e6},
            "cpu_baseline": None,
            "e2e": {"value": world * B / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": world * B * H * 2, "d2h_bytes_per_step": world * B * H * 4},
            "gpu_launches": int(launches) * world, "clocks": clocks,
        }
        if stack is not None:
            line["stack"] = stack
        if exchange_note:
            line["config"]["exchange_note"] = exchange_note
        line["config"]["exchange"] = "NCCL all-gather + all-to-all" if args.ep_nccl else \
            "peer-memory stores + flags inside the library's kernels (CUDA IPC over NVLink), no collective call"
        print(json.dumps(line), flush=True)
    if exchange is not None:
        err = exchange.error()
        if err:
            raise RuntimeError(f"rank {rank}: a wait on a peer gave up (code {err})")
    dist.barrier()
    torch.cuda.synchronize()
    # Tearing down an NCCL communicator while captured graphs that hold its kernels are alive has been
    # seen to block for minutes; the results are out, so leave without the teardown.
    import sys
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)
