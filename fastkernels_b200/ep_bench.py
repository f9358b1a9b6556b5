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
import sys
import time

import torch
import torch.distributed as dist


def check_parity(plan, hidden, shard, layer_seed, spec, rank, world, dev, make_expert_subset, sample: int = 8) -> dict:
    """Runs `plan` on `hidden` and checks it: ids of every token against the stand-alone router kernel (bit-exact), and
    `sample` of the rank's tokens against the CPU oracle (routing by the oracle's rule on the kernel's own logits and,
    away from near-ties, against the oracle's logits; outputs within max-abs 2e-2 and rel-L2 5e-3).
    The oracle is test infrastructure: it is the checker here, never what is timed."""
    from oracle import moe_oracle as O
    from .moe import qwen36_batched_moe_router_decode
    w = shard.weights
    out, logits, ids, weights = [t.clone() for t in plan.run(hidden)]
    torch.cuda.synchronize()
    _, ids_ref, w_ref = qwen36_batched_moe_router_decode(hidden, w.norm_weight, w.router_weight, top_k=8, router_bias=w.router_bias)
    ids_exact = bool(torch.equal(ids, ids_ref)) and bool(torch.allclose(weights, w_ref, atol=1e-6, rtol=1e-5))
    T = hidden.shape[0]
    pick = torch.linspace(0, T - 1, steps=min(sample, T)).round().long().unique()
    hs = hidden[pick].cpu()
    cpu = lambda t: None if t is None else t.detach().cpu()
    lg_o, ids_o, w_o = O.router(hs, cpu(w.norm_weight), cpu(w.router_weight), top_k=8, router_bias=cpu(w.router_bias))
    own_ids, own_w = O.route_from_logits(logits[pick].cpu(), 8)
    ids_k = ids[pick].cpu()
    ids_exact = ids_exact and bool(torch.equal(ids_k, own_ids))
    probs = torch.softmax(lg_o, dim=-1).sort(dim=-1, descending=True).values
    clear = (probs[:, 7] - probs[:, 8]) > 2e-6
    ids_exact = ids_exact and bool(torch.equal(ids_k[clear], ids_o[clear]))
    logits_ok = bool(torch.allclose(logits[pick].cpu(), lg_o, atol=1e-4, rtol=1e-4))
    # the sampled tokens' experts, drawn again from the layer's seed on this GPU, then moved to the host
    need = sorted(set(ids_k.flatten().tolist()))
    sub = make_expert_subset(layer_seed, spec, need, dtype=torch.bfloat16, device=dev)
    gu = {e: v[0].cpu() for e, v in sub.items()}
    dn = {e: v[1].cpu() for e, v in sub.items()}
    ref = O.routed_shared_experts(hs, ids_k, weights[pick].cpu(), gu, dn, cpu(w.shared_gate_up_weight), cpu(w.shared_down_weight),
                                  cpu(w.shared_expert_gate_weight))
    got = out[pick].cpu()
    ma, rl = O.max_abs(got, ref), O.rel_l2(got, ref)
    ok = ids_exact and logits_ok and ma <= 2e-2 and rl <= 5e-3
    return {"ok": ok, "ids_exact": ids_exact, "logits_ok": logits_ok, "max_abs": ma, "rel_l2": rl, "tokens_checked": int(pick.numel()),
            "near_ties": int((~clear).sum())}


def run_ep(args, workload_config, measured_peak, ClockSampler, METRIC, UNIT):
    from . import _lib
    from .ep import EPDecodePlan, ep_payload_bytes, EPShard, PeerEPLayer, PeerExchange
    from .spec import MoESpec
    from .workloads import make_expert_subset, make_hidden, make_moe_weights

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
    B, K, W, L = args.batch or 256, args.steps, max(args.warmup, 3), args.layers
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

    # ---- correctness of what was just timed, on every rank: (a) the ids of the expert-parallel call equal the stand-alone
    # router's on the same tokens, (b) a sample of the rank's own tokens against the CPU oracle, whose experts are drawn
    # again from the seeds (a rank holds only its shard), (c) agreed over the ranks.
    parity = check_parity(plans[0], hid_dev[0], shards[0], 0, spec, rank, world, dev, make_expert_subset)
    flags = torch.tensor([1.0 if parity["ok"] else 0.0, parity["max_abs"], parity["rel_l2"], float(parity["tokens_checked"]),
                          float(parity["near_ties"])], device=dev)
    worst = flags.clone()
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    allok = flags[:1].clone()
    dist.all_reduce(allok, op=dist.ReduceOp.MIN)
    total_checked = flags[3:4].clone()
    dist.all_reduce(total_checked, op=dist.ReduceOp.SUM)
    parity_line = {"ids_exact": bool(allok.item() == 1.0) and parity["ids_exact"], "ok": bool(allok.item() == 1.0),
                   "max_abs": float(worst[1]), "rel_l2": float(worst[2]), "tokens_checked": int(total_checked.item()),
                   "near_tie_tokens_excluded": int(worst[4]), "limits": {"max_abs": 2e-2, "rel_l2": 5e-3},
                   "what": "per rank: ids of all tokens vs the stand-alone router (bit-exact); 8 own tokens vs the CPU oracle "
                           "(ids bit-exact by the oracle's rule on the kernel's logits, outputs within the limits)"}

    # ---- per-stage times of the same call (CUDA events between the kernels; eager; maximum over the ranks)
    stages_ms = None
    if not args.ep_nccl:
        acc = None
        reps = 5
        for i in range(reps + 1):
            dist.barrier()
            st = plans[i % L].timed()
            if i:                                  # the first one warms the eager path up
                acc = st if acc is None else [a + b for a, b in zip(acc, st)]
        t = torch.tensor([a / reps for a in acc], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        names = (["router", "dispatch+wait", "permute", "gather", "gate_up", "down", "combine+wait", "reduce"] if len(acc) == 8 else
                 ["router", "dispatch+wait", "permute", "gate_up", "down", "combine+wait", "reduce"])
        stages_ms = dict(zip(names, [float(v) for v in t.tolist()]))

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
            # bytes all ranks together must move per pass: every expert some token of any rank selected, once, on its
            # owner; router, shared expert, gate and norm on every rank; activations in and out
            torch.cuda.synchronize()
            agg = 0.0
            for ids_l in sp.topk_ids:
                ids_all = torch.empty((world * tok, 8), dtype=ids_l.dtype, device=dev)
                dist.all_gather_into_tensor(ids_all, ids_l.contiguous())
                agg += int(torch.unique(ids_all).numel()) * per_expert
            agg += args.stack_layers * world * (per_expert + E * H * 2 + 2 * H * 2 + tok * (H * 2 + H * 4 + E * 4 + 8 * 12))
            stack["runs"].append({"tokens_per_gpu": tok, "ms_per_stack_pass": t_ms, "us_per_layer": t_ms * 1e3 / args.stack_layers,
                                  "us_per_token": t_ms * 1e3, "tokens_per_s": world * tok / (t_ms * 1e-3),
                                  "aggregate_algorithmic_bytes": agg, "aggregate_gbs": agg / (t_ms * 1e-3) / 1e9,
                                  "frac_of_world_hbm_peak": agg / (t_ms * 1e-3) / 1e9 / (world * peak)})
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
                         "distinct_local_experts": u_local, "stages_ms": stages_ms,
                         "nvlink_bytes_per_rank_per_step": payload,
                         "nvlink_floor_us": (max(payload["dispatch"], 0) + payload["combine"]) / 770e9 * 1e6},
            "cpu_baseline": None, "parity": parity_line,
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
    if not parity_line["ok"]:
        sys.stdout.flush()
        sys.stderr.write(f"rank {rank}: parity check failed: {parity}\n")
        sys.stderr.flush()
        os._exit(3)
    torch.cuda.synchronize()
    # Tearing down an NCCL communicator while captured graphs that hold its kernels are alive has been
    # seen to block for minutes; the results are out, so leave without the teardown.
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)
