#!/usr/bin/env python
"""Benchmark of the Qwen3.6 MoE decode layer on B200 (one JSON line on stdout).

    python bench.py --gpus N --steps K --warmup W [--batch B] [--impl reference]

A step is one MoE layer call (router -> top-8 -> routed + shared experts) over one batch of
synthetic decode tokens.  Shapes are the real layer (hidden 2048, 256 experts, top-8,
intermediate 512, gated shared expert); weights ~ N(0, 0.02) bf16, hidden ~ N(0, 1) bf16, router
logit bias ~ N(0, 0.5).  Consecutive steps use different layers' weights (a rotation of several
resident copies, as a decoder stack does), so no step finds its weights in L2.

value      tokens/s with the step's input already in HBM: CUDA events around blocks of K steps, repeated until the
           timed region is at least 0.2 s, median block.  The steps are replayed as CUDA graphs of `--layers`
           consecutive layer calls (one per resident weight copy), the way a decoder stack issues them.
e2e        the same through the host-buffer entry point: every step copies its hidden batch from
           pinned host memory, runs the layer and copies output, ids and weights back, then waits.
roofline   the dominant kernel (gate_up GEMV + SwiGLU): its algorithmic bytes / its mean duration
           (CUDA events between the stages of the same steps), against the measured copy bandwidth.
cpu_baseline  the oracle port of the reference's PyTorch CPU path on this box's host cores.

--impl reference times that CPU path alone (all host threads) on the same workload.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "moe_layer_decode_tokens_per_s"
UNIT = "tokens/s"
FALLBACK_HBM_GBS = 6650.0


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="own", choices=["own", "reference"])
    ap.add_argument("--batch", type=int, default=None,
                    help="decode tokens per GPU per step (default: 32 on one GPU, 256 per GPU expert parallel)")
    ap.add_argument("--layers", type=int, default=6, help="resident weight copies rotated between steps")
    ap.add_argument("--no-sweep", action="store_true", help="skip the per-batch sweep (1..256 tokens)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--flags", type=int, default=0)
    ap.add_argument("--stack-layers", type=int, default=None,
                    help="also time a stack of this many layers (x <- x + MoE(RMSNorm(x)), one CUDA graph) at 1 and 64 tokens "
                         "(default: 40 layers when run on 8 GPUs, none otherwise; 0 turns it off)")
    ap.add_argument("--ep-eager", action="store_true", help="expert-parallel leg: no CUDA-graph capture of the layer call")
    ap.add_argument("--ep-nccl", action="store_true",
                    help="expert-parallel leg: exchange with NCCL collectives instead of the peer-memory kernels")
    return ap.parse_args()


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """SM clock and throttle-reason samples while the timed regions run (read-only NVML queries every
    few milliseconds from a thread; `nvidia-smi` polling as the fallback)."""

    REASONS = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, index: int, period_s: float = 0.004):
        self.index, self.period = index, period_s
        self.sm, self.reasons, self.smax = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        self._proc = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            # NVML enumerates physical devices; honour CUDA_VISIBLE_DEVICES when it is a plain index list
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = self.index
            if vis:
                parts = [v.strip() for v in vis.split(",") if v.strip()]
                if self.index < len(parts) and parts[self.index].isdigit():
                    phys = int(parts[self.index])
            self._h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.smax = float(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
            self._thread = threading.Thread(target=self._poll, daemon=True)
            self._thread.start()
        except Exception:
            self._thread = None
            self._start_smi()

    def _poll(self):
        nv = self._nvml
        while not self._stop.is_set():
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._h))
                for name, bit in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def _start_smi(self):
        fields = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
                  "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
                  "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self._proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={fields}", "--format=csv,noheader,nounits",
                                           "-i", str(self.index), "-lms", "20"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self._proc = None

    def _pump(self):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self._proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                self.sm.append(float(parts[1]))
                self.smax = max(self.smax or 0.0, float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower() == "active":
                    self.reasons.add(name)

    def stop(self) -> dict:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=1.0)
        if self._proc is not None:
            time.sleep(0.05)
            self._proc.terminate()
        if not self.sm:
            return {"sm_mhz": None, "sm_max_mhz": self.smax, "samples": 0, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(self.sm), "sm_min_mhz": min(self.sm), "sm_max_mhz": self.smax,
                "samples": len(self.sm), "reasons": sorted(self.reasons)}


# --------------------------------------------------------------------------------------------- CPU arm
def cpu_weights(seed: int, bias_std: float):
    import torch
    from fastkernels_b200.spec import MoESpec
    from fastkernels_b200.workloads import make_moe_weights
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    w = make_moe_weights(seed, MoESpec(), dtype=torch.bfloat16, device=dev, bias_std=bias_std)
    return w.to("cpu") if dev == "cuda" else w


def time_cpu_port(weights, hidden_cpu, *, budget_s: float = 20.0, min_reps: int = 2):
    """Seconds per call of the oracle's token-loop port on `hidden_cpu` (all host threads)."""
    import torch
    from oracle import moe_oracle as O
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    args = weights.tuple()
    O.moe_update_token_loop(hidden_cpu[:1], *args, top_k=8, router_bias=weights.router_bias)   # warm-up
    times = []
    t_end = time.perf_counter() + budget_s
    while len(times) < min_reps or (time.perf_counter() < t_end and len(times) < 8):
        t0 = time.perf_counter()
        O.moe_update_token_loop(hidden_cpu, *args, top_k=8, router_bias=weights.router_bias)
        times.append(time.perf_counter() - t0)
    return statistics.median(times), threads, len(times)


def cpu_sample_tokens(batch: int) -> int:
    return min(batch, 32)


def run_reference(args):
    """The reference's CPU implementation of the path (oracle port), timed on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    from fastkernels_b200.spec import MoESpec
    from fastkernels_b200.workloads import make_hidden
    spec = MoESpec()
    batch = args.batch or (32 if args.gpus == 1 else 256)
    sample = cpu_sample_tokens(batch)
    w = cpu_weights(0, 0.5)
    from oracle import moe_oracle as O
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    steps = max(1, args.steps)
    warm = max(0, args.warmup)
    hs = [make_hidden(1000 + i, sample, spec, dtype=torch.bfloat16) for i in range(4)]
    for i in range(warm):
        O.moe_update_token_loop(hs[i % 4], *w.tuple(), top_k=8, router_bias=w.router_bias)
    t0 = time.perf_counter()
    for i in range(steps):
        O.moe_update_token_loop(hs[i % 4], *w.tuple(), top_k=8, router_bias=w.router_bias)
    dt = (time.perf_counter() - t0) / steps
    # a step of the full workload is `batch * n_gpus` tokens; the token loop is linear in tokens
    tokens_per_s = sample / dt
    total = batch * args.gpus
    line = {
        "impl": "reference", "metric": METRIC, "value": tokens_per_s, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warm, "ms_per_step": dt * 1e3 * total / sample, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(batch, args.gpus, args.layers),
        "cpu_baseline": {"value": tokens_per_s, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"{sample} of {total} tokens per step, {steps} steps; token x route loop is linear in tokens"},
        "e2e": {"value": tokens_per_s, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(batch: int, gpus: int, layers: int) -> dict:
    which = "configs[1]" if batch <= 32 else "configs[2]"
    if gpus > 1:
        which = "configs[3]: expert parallel, 256 tokens per GPU" if batch == 256 else "expert parallel as configs[3], other batch"
    return {"workload": f"Qwen3.6 MoE layer decode, bf16, {batch} tokens per GPU ({which})", "hidden": 2048,
            "experts": 256, "top_k": 8, "intermediate": 512, "tokens_per_gpu": batch, "global_tokens": batch * gpus,
            "router_bias_std": 0.5, "parallelism": "single GPU" if gpus == 1 else f"ep{gpus}",
            "l2": f"weights rotate over {layers} resident layer copies per GPU; a step's weights were last touched "
                  f"{layers} steps earlier, more than L2 apart",
            "replay": f"steps are replayed as CUDA graphs of {layers} consecutive layer calls (one per weight copy)"}


# --------------------------------------------------------------------------------------------- own arm
def distinct_experts(ids) -> int:
    import torch
    return int(torch.unique(ids).numel())


MIN_TIMED_S = 0.2


def time_steps(plans, hiddens, steps: int, warmup: int, chain=None):
    """ms per step of `steps` layer calls rotating over the plans (= resident weight copies): CUDA events around a
    block of exactly `steps` calls, blocks repeated until at least MIN_TIMED_S has been timed, median block.
    Whole rotations are replayed as one CUDA graph of len(plans) calls, the remainder as single-call graphs."""
    import torch
    from fastkernels_b200.plan import PlanChain
    n, m = len(plans), len(hiddens)
    for i, p in enumerate(plans):          # inputs are resident before the timed region starts
        p.hidden.copy_(hiddens[i % m])
    chain = chain or PlanChain(plans)
    full, rest = divmod(steps, n)
    for p in plans[:rest]:
        if p.graph is None:
            p.capture()

    def block():
        for _ in range(full):
            chain.replay()
        for i in range(rest):
            plans[i].run()

    for _ in range(max(1, -(-warmup // n))):
        chain.replay()
    torch.cuda.synchronize()
    per_step, total = [], 0.0
    while (total < MIN_TIMED_S or len(per_step) < 3) and len(per_step) < 2000:
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        block()
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop)
        per_step.append(ms / steps)
        total += ms * 1e-3
    return statistics.median(per_step), len(per_step)


def run_single(args):
    import torch
    from fastkernels_b200 import _lib
    from fastkernels_b200.plan import MoEDecodePlan
    from fastkernels_b200.spec import MoESpec
    from fastkernels_b200.workloads import algorithmic_bytes, make_hidden, make_moe_weights

    lib = _lib.load()                      # fails loudly if the CUDA library is missing
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU path in the product")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    spec = MoESpec()
    peak, peak_src = measured_peak()
    B, K, W, L = args.batch or 32, args.steps, max(args.warmup, 3), args.layers

    weights = [make_moe_weights(layer, spec, dtype=torch.bfloat16, device=dev, bias_std=0.5) for layer in range(L)]
    pool = 8
    hid_host = [make_hidden(1000 + i, B, spec, dtype=torch.bfloat16).pin_memory() for i in range(pool)]
    hid_dev = [h.to(dev) for h in hid_host]

    plans = [MoEDecodePlan(w, B, flags=args.flags) for w in weights]
    for p in plans:
        p.capture()
    sampler = ClockSampler(local)
    sampler.start()
    ms, blocks_timed = time_steps(plans, hid_dev, K, W)
    # the timed steps replay CUDA graphs, which bypass the library's launch counter: count the
    # kernels one direct call enqueues (the graph holds exactly these) and multiply by the steps
    c0 = lib.fk_launch_count()
    plans[0].launch()
    per_call = lib.fk_launch_count() - c0
    torch.cuda.synchronize()
    launches = per_call * K

    # per-stage durations of the same steps (events between the kernels), for the roofline
    stage_sum = None
    for i in range(W):
        plans[i % L].timed()
    ucount = []
    for i in range(K):
        p = plans[i % L]
        st = p.timed()
        stage_sum = st if stage_sum is None else [a + b for a, b in zip(stage_sum, st)]
        if i < L * pool:
            ucount.append(distinct_experts(p.topk_ids))
    stage_ms = [s / K for s in stage_sum]
    stage_names = (["router", "permute", "gather", "gate_up", "down", "combine"] if len(stage_ms) == 6 else
                   ["router", "permute", "gate_up", "down", "combine"][:len(stage_ms)])
    U = statistics.mean(ucount)
    layer_bytes = algorithmic_bytes(spec, B, 0) + U * spec.expert_bytes_bf16
    H, I = spec.hidden_size, spec.expert_intermediate_size
    gate_up_bytes = (U + 1) * 2 * I * H * 2 + B * H * 2
    dom = stage_names.index("gate_up") if "gate_up" in stage_names else 0
    dom_ms = stage_ms[dom]
    # Which kernel that is depends on the batch (csrc/api.cu picks the path).  `traffic` is DRAM read + write bytes
    # of that kernel from an ncu capture of the same workload on one layer copy (profiles/), expressed per
    # algorithmic byte and scaled to this launch's bytes: the kernels stream every weight byte exactly once, so
    # traffic grows in proportion to the experts touched.
    if len(stage_ms) == 1:
        # the step is this one kernel: its duration is the graph-replayed step (the stage events add their own gap)
        if B == 1:
            dom_kernel, traffic_ratio, traffic_file = ("decode1_kernel (whole layer, one token, one launch)",
                                                       NCU_TRAFFIC_PER_BYTE["decode1"], "profiles/decode1_fused_b1.md")
        else:
            dom_kernel, traffic_ratio, traffic_file = ("decode_few_kernel (whole layer, two to four tokens, one launch)",
                                                       NCU_TRAFFIC_PER_BYTE.get("decode_few"), "profiles/decode_few_b4.md")
        dom_bytes = layer_bytes
        dom_ms = ms
    elif B < 64:
        dom_kernel, dom_bytes, traffic_ratio = ("stream_gemv_kernel<8,true,false> (gate_up GEMV + SwiGLU, "
                                                "TMA ring, mma.sync consumers)"), gate_up_bytes, NCU_TRAFFIC_PER_BYTE["stream_gate_up"]
        traffic_file = "profiles/stream_gemv_b32.md"
    else:
        dom_kernel, dom_bytes, traffic_ratio = ("tc_grouped_kernel<true> (tcgen05 grouped gate_up GEMM + SwiGLU)",
                                                gate_up_bytes, NCU_TRAFFIC_PER_BYTE["tc_gate_up"])
        traffic_file = "profiles/tc_grouped_gemm_b256.md"
    achieved = dom_bytes / (dom_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": dom_kernel, "achieved": achieved,
                "peak": peak, "peak_source": peak_src, "unit": "GB/s", "frac": achieved / peak,
                "algorithmic_bytes_per_launch": dom_bytes, "ms_per_launch": dom_ms,
                "traffic": None if traffic_ratio is None else traffic_ratio * dom_bytes,
                "traffic_source": None if traffic_ratio is None else
                f"not a live counter: algorithmic bytes x {traffic_ratio:.3f}, the DRAM read + write bytes per algorithmic "
                f"byte of this kernel in the ncu capture summarised in {traffic_file}",
                "stages_ms": dict(zip(stage_names, stage_ms)),
                "layer": {"algorithmic_bytes": layer_bytes, "achieved": layer_bytes / (ms * 1e-3) / 1e9,
                          "frac": layer_bytes / (ms * 1e-3) / 1e9 / peak, "distinct_experts": U}}

    # end to end through the host-buffer entry point
    out_host = torch.empty(B, H, dtype=torch.float32).pin_memory()
    ids_host = torch.empty(B, 8, dtype=torch.int64).pin_memory()
    w_host = torch.empty(B, 8, dtype=torch.float32).pin_memory()
    # Eager on purpose: the copy in starts at once and the remaining launches are issued while the GPU works.  The
    # same call captured in one graph (MoEDecodePlan.run_host_graph) pays the graph's launch latency up front and
    # measured slower with a synchronise per step (185 vs 177 us at 32 tokens).
    for i in range(W):
        plans[i % L].run_host(hid_host[i % pool], out_host, ids_host, w_host)
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(K):
        plans[i % L].run_host(hid_host[i % pool], out_host, ids_host, w_host)
        torch.cuda.current_stream().synchronize()
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1) / K
    wall_ms = (time.perf_counter() - t0) * 1e3 / K
    clocks = sampler.stop()
    e2e = {"value": B / (max(e2e_ms, wall_ms) * 1e-3), "unit": UNIT, "ms_per_step": max(e2e_ms, wall_ms),
           "h2d_bytes_per_step": B * H * 2, "d2h_bytes_per_step": B * H * 4 + B * 8 * 12}

    sweep, roofline_b1 = [], None
    if not args.no_sweep:
        import dataclasses
        from fastkernels_b200.workloads import HOT_EXPERT_IDS

        def sweep_entry(b, ws, variant):
            ps = plans if (b == B and variant == "bias") else [MoEDecodePlan(w, b, flags=args.flags) for w in ws]
            hs = [make_hidden(2000 + i, b, spec, dtype=torch.bfloat16, device=dev) for i in range(pool)]
            t, _ = time_steps(ps, hs, max(20, K // 2), W)
            us = []
            for i in range(min(L, 2)):
                ps[i].run(hs[i])
                torch.cuda.synchronize()
                us.append(distinct_experts(ps[i].topk_ids))
            u = statistics.mean(us)
            by = algorithmic_bytes(spec, b, 0) + u * spec.expert_bytes_bf16
            return {"batch": b, "routing": variant, "us_per_step": t * 1e3, "tokens_per_s": b / (t * 1e-3),
                    "distinct_experts": u, "algorithmic_bytes": by, "achieved_gbs": by / (t * 1e-3) / 1e9,
                    "frac_of_hbm_peak": by / (t * 1e-3) / 1e9 / peak}

        for b in (1, 4, 16, 32, 64, 128, 256):
            sweep.append(sweep_entry(b, weights, "bias"))
        # hot-expert variant: +3.0 on eight fixed expert logits, so that about half of all routes hit them
        hot = []
        for w in weights:
            bias = torch.zeros(spec.num_experts, dtype=torch.float32, device=dev)
            bias[list(HOT_EXPERT_IDS)] += 3.0
            hot.append(dataclasses.replace(w, router_bias=bias))
        for b in (64, 128, 256):
            sweep.append(sweep_entry(b, hot, "hot"))
        one = sweep[0]
        roofline_b1 = {"bound": "hbm", "kernel": "decode1_kernel (whole layer, one token, one launch)",
                       "achieved": one["achieved_gbs"], "peak": peak, "peak_source": peak_src, "unit": "GB/s",
                       "frac": one["frac_of_hbm_peak"], "algorithmic_bytes_per_launch": one["algorithmic_bytes"],
                       "ms_per_launch": one["us_per_step"] * 1e-3,
                       "traffic": NCU_TRAFFIC_PER_BYTE["decode1"] * one["algorithmic_bytes"],
                       "traffic_source": "not a live counter: algorithmic bytes x the DRAM bytes per algorithmic byte of the "
                                         "ncu capture summarised in profiles/decode1_fused_b1.md"}

    cpu = None
    if not args.no_cpu:
        sample = cpu_sample_tokens(B)
        wc = weights[0].to("cpu")
        sec, threads, reps = time_cpu_port(wc, hid_host[0][:sample].clone(), budget_s=15.0)
        cpu = {"value": sample / sec, "unit": UNIT, "cores": threads, "kind": "port",
               "sample": f"{sample} of {B} tokens of one step, median of {reps} calls of the token x route loop "
                         f"(fp32 PyTorch on the host cores)", "ms_per_call": sec * 1e3}

    stack = None
    if args.stack_layers > 0:
        from fastkernels_b200.stack import MoEStackPlan
        del plans
        torch.cuda.empty_cache()
        layers = list(weights)
        for layer in range(len(layers), args.stack_layers):
            layers.append(make_moe_weights(layer, spec, dtype=torch.bfloat16, device=dev, bias_std=0.5))
        stack = {"layers": args.stack_layers, "runs": []}
        for tok in (1, 64):
            sp = MoEStackPlan(layers, tok)
            x0 = make_hidden(3000 + tok, tok, spec, dtype=torch.float32, device=dev)
            for _ in range(3):
                sp.run(x0)
            torch.cuda.synchronize()
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 10
            s0.record()
            for _ in range(reps):
                sp.run(x0)
            s1.record()
            torch.cuda.synchronize()
            t_ms = s0.elapsed_time(s1) / reps
            u = statistics.mean(distinct_experts(i) for i in sp.topk_ids)
            by = args.stack_layers * (algorithmic_bytes(spec, tok, 0) + u * spec.expert_bytes_bf16)
            stack["runs"].append({"tokens": tok, "ms_per_stack_pass": t_ms, "us_per_layer": t_ms * 1e3 / args.stack_layers,
                                  "tokens_per_s": tok / (t_ms * 1e-3), "aggregate_gbs": by / (t_ms * 1e-3) / 1e9,
                                  "frac_of_hbm_peak": by / (t_ms * 1e-3) / 1e9 / peak})
            del sp

    line = {
        "metric": METRIC, "value": B / (ms * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": workload_config(B, 1, L), "roofline": roofline, "roofline_b1": roofline_b1,
        "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches) * blocks_timed, "launches_per_step": int(per_call),
        "timed_blocks": blocks_timed, "clocks": clocks, "sweep": sweep,
    }
    if stack is not None:
        line["stack"] = stack
    print(json.dumps(line), flush=True)


# DRAM bytes (read + write) per algorithmic byte of the dominant kernel, from the ncu captures summarised in
# profiles/stream_gemv_b32.md, profiles/tc_grouped_gemm_b256.md and profiles/decode1_fused_b1.md.
NCU_TRAFFIC_PER_BYTE = {"stream_gate_up": 1.008, "tc_gate_up": 1.015, "decode1": 1.008, "decode_few": 1.019}      # profiles/*.md


def main():
    args = parse_args()
    if args.stack_layers is None:
        args.stack_layers = 40 if args.gpus == 8 else 0
    if args.impl == "reference":
        run_reference(args)
        return
    if args.gpus > 1 or int(os.environ.get("WORLD_SIZE", "1")) > 1:
        from fastkernels_b200.ep_bench import run_ep
        run_ep(args, workload_config, measured_peak, ClockSampler, METRIC, UNIT)
        return
    run_single(args)


if __name__ == "__main__":
    main()
