#!/usr/bin/env python
"""Benchmark of the fused MoE layer on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c4] [--sub c2,c5,c3] [--impl reference]

One step = one pass of the layer (route -> sort -> quantise -> FC1+activation -> FC2 -> combine)
over one batch of seeded synthetic input.  The headline workload is the Mixtral-shaped NVFP4 prefill
layer with skewed routing (hidden 4096, intermediate 14336, 8 experts, top-2, 8192 tokens per GPU):
the large-batch, tensor-bound configuration.  The other benchmark shapes (DeepSeek-V3-shaped decode,
GPT-OSS-shaped w4a8_mx, Qwen3-shaped W4A16) are timed in the same run and reported as compact
sub-records under ``"workloads"``.  With N > 1 the expert-parallel shapes block-partition their
experts over the ranks (tokens are exchanged by the library's own kernels over NVLink peer memory;
``--ep nccl`` selects the NCCL all-to-all variant) and every rank brings its own batch; the Qwen3
shape shards the intermediate dimension (tensor parallelism, NCCL all-reduce).  Rank 0 prints ONE
JSON line.

Every timed shape is also checked: after the timed loop the CPU oracle evaluates the routed rows of
a few experts and is compared with the rows the kernels left in the scratch arena (the whole
permutation bit for bit, the FC2 rows within 1e-2 x their RMS); a failed check exits non-zero.

``--impl reference`` times the CPU oracle (the restatement of the reference library's own torch
implementation of this layer) on the host cores for the headline configuration.
"""

from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from dataclasses import replace
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from b12x_b200 import synth  # noqa: E402

# DRAM bytes per FC1 launch of the decode shape: an ncu capture of its 32-expert case read 1.014 x
# the algorithmic bytes (dram__bytes_read + write; summary under profiles/); every active expert's
# weights are read once per launch, so the traffic scales with the algorithmic bytes
# (c4: the 2048-token case read 538 + 35 MB against 528 MB of weights + 9.4 MB of token codes + 33 MB of
# intermediate codes and scales = 1.005 x algorithmic; more tokens add row bytes one for one)
NCU_FC1_TRAFFIC_RATIO = {"c2_dsv3_decode_nvfp4": 1.014, "c4_mixtral_skew_nvfp4": 1.005}
# experts of the CPU-baseline sample: a pass over them takes a few seconds on 16 cores
CPU_EXPERTS = {"c1": 8, "c2": 8, "c3": 8, "c4": 4, "c5": 8}
PARITY_EXPERTS = 4
PARITY_ROWS_PER_EXPERT = 48
PARITY_TOL = 1e-2


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="c4", choices=sorted(synth.SHAPES))
    ap.add_argument("--sub", default="c2,c5,c3",
                    help="comma-separated workloads reported as sub-records ('none' to skip them)")
    ap.add_argument("--tokens", type=int, default=None, help="tokens per GPU of the headline workload")
    ap.add_argument("--experts", type=int, default=None, help="override the expert count (small profiling cases)")
    ap.add_argument("--ep", default="peer", choices=["peer", "nccl"],
                    help="expert-parallel exchange: own kernels over peer memory, or NCCL all-to-all")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch the step kernel by kernel instead of replaying a CUDA graph")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-experts", type=int, default=None, help="experts in the CPU-baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the sampled oracle check (profiling runs)")
    return ap.parse_args()


def load_peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clock / throttle sampling during the timed region (read-only queries)."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.gpu)], stdout=f, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def _lines(self):
        try:
            return Path(self.path).read_text().splitlines()
        except (OSError, TypeError):
            return []

    def wait_first(self, timeout_s: float = 4.0) -> None:
        """Block until nvidia-smi has written its first sample (its start-up takes about a second)."""
        t0 = time.perf_counter()
        while self.proc is not None and not self._lines() and time.perf_counter() - t0 < timeout_s:
            time.sleep(0.02)

    def mark(self) -> int:
        """Index of the next sample: brackets a timed region."""
        return len(self._lines())

    def window(self, lo: int, hi: int) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        lines = self._lines()
        # a region shorter than the sampling period: take the samples either side of it
        win = lines[lo:hi] if hi > lo else lines[max(lo - 1, 0):hi + 1]
        sm, smax, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in win:
            c = [x.strip() for x in line.split(",")]
            if len(c) < 9:
                continue
            try:
                sm.append(float(c[1]))
                smax.append(float(c[2]))
            except ValueError:
                continue
            for name, val in zip(names, c[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(smax) if smax else None, "samples": len(sm), "reasons": sorted(reasons)}

    def stop(self) -> None:
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        try:
            os.unlink(self.path)
        except OSError:
            pass


class StageTimer:
    """Records a CUDA event on the current stream at each stage boundary of one layer call."""

    def __init__(self):
        self.steps = []
        self.cur = None

    def __call__(self, name: str):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        if name == "begin":
            self.cur = [("begin", ev)]
            self.steps.append(self.cur)
        else:
            self.cur.append((name, ev))

    def mean_ms(self) -> dict:
        acc: dict = {}
        for marks in self.steps:
            for (_, e0), (n1, e1) in zip(marks[:-1], marks[1:]):
                acc.setdefault(n1, []).append(e0.elapsed_time(e1))
        return {k: sum(v) / len(v) for k, v in acc.items()}


# ---------------------------------------------------------------------------------------------
# CPU oracle legs (the only places this file touches oracle/)
# ---------------------------------------------------------------------------------------------
def _oracle_call(shp, x, w1, s1, g1, w2, s2, g2, a1, a2, ids, weights, expert_map=None, taps=None):
    from oracle import moe_oracle as O
    if shp.recipe == "nvfp4":
        return O.moe_nvfp4(x, w1, s1, g1 / a1, w2, s2, g2 / a2, a1, a2, ids, weights, activation=shp.activation,
                           expert_map=expert_map, taps=taps)
    if shp.recipe == "w4a16":
        return O.moe_w4a16(x, w1, s1, g1, w2, s2, g2, ids, weights, activation=shp.activation,
                           expert_map=expert_map, taps=taps)
    ones = torch.ones(w1.shape[0])
    return O.moe_w4a8_mx(x, w1, s1, ones, w2, s2, ones, ids, weights, activation=shp.activation,
                         expert_map=expert_map, taps=taps)


def oracle_sample(shp, inp_cpu, ids, weights, experts_lo: int, n_experts: int):
    """CPU oracle on the routes of the batch that land on experts [experts_lo, experts_lo + n)."""
    emap = torch.full((shp.experts,), -1, dtype=torch.int32)
    emap[experts_lo:experts_lo + n_experts] = torch.arange(n_experts, dtype=torch.int32)
    kept = int(((ids >= experts_lo) & (ids < experts_lo + n_experts)).sum())
    t0 = time.perf_counter()
    _oracle_call(shp, inp_cpu.x, inp_cpu.w1_fp4, inp_cpu.w1_blockscale, inp_cpu.w1_global_scale, inp_cpu.w2_fp4,
                 inp_cpu.w2_blockscale, inp_cpu.w2_global_scale, inp_cpu.a1_gscale, inp_cpu.a2_gscale, ids, weights,
                 expert_map=emap)
    return time.perf_counter() - t0, kept


def cpu_sample_inputs(shp, n_experts: int):
    """Host copy of the workload restricted to the sample's experts, its routing, and where the sample
    sits: the first experts, or -- where routing is skewed and the first experts are the hot ones --
    the last, so that one pass stays within seconds."""
    from oracle import moe_oracle as O
    n_e = min(n_experts, shp.experts)
    inp = synth.make_inputs(shp, seed=0, device="cpu", experts=n_e)
    if shp.router == "sigmoid":
        _, ids, w = O.route_topk(inp.router_logits, shp.topk, mode="sigmoid", route_scale=shp.route_scale)
    else:
        _, ids, w = O.route_topk(inp.router_logits, shp.topk)
    lo = shp.experts - n_e if shp.zipf_s > 0 else 0
    return inp, ids, w, lo, n_e


def sample_text(shp, lo, n_e, kept) -> str:
    return (f"routes of one {shp.tokens}-token batch that land on experts {lo}..{lo + n_e - 1} "
            f"({kept} of {shp.rows} routed rows); tokens = rows / top-k")


def run_reference(args, shp):
    """The reference's CPU implementation of the path (oracle port), all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    inp, ids, w, lo, n_e = cpu_sample_inputs(shp, args.cpu_experts or CPU_EXPERTS.get(args.workload, 8))
    times, kept = [], 0
    for i in range(args.warmup + args.steps):
        dt, kept = oracle_sample(shp, inp, ids, w, lo, n_e)
        if i >= args.warmup:
            times.append(dt)
    sec = sum(times) / len(times)
    tok_s = (kept / shp.topk) / sec
    line = {
        "impl": "reference", "metric": "moe_layer_tokens_per_s", "value": tok_s, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dtype_of(shp),
        "data": "synthetic", "config": config_of(shp, args.gpus),
        "cpu_baseline": {"value": tok_s, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": sample_text(shp, lo, n_e, kept)},
        "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "tflops": kept * shp.flops / shp.rows / sec / 1e12,
    }
    print(json.dumps(line), flush=True)


def parity_sample(layer) -> dict:
    """Check the last step of ``layer`` against the CPU oracle on a sample: the whole permutation
    bit for bit, and the activation codes and fp32 FC2 rows of up to ``PARITY_ROWS_PER_EXPERT``
    routes of ``PARITY_EXPERTS`` experts (``tests/gpu_utils.sampled_parity``)."""
    from tests.gpu_utils import sampled_parity
    # a quantised expert-parallel dispatch leaves no bf16 rows on the expert rank: look them up
    # in the ranks' inputs (a collective; every rank gets here)
    rows = layer.received_rows(layer.last_x) if getattr(layer, "packed", None) is not None else None
    return sampled_parity(layer.last_binding, layer.inputs, experts=PARITY_EXPERTS,
                          rows_per_expert=PARITY_ROWS_PER_EXPERT, tolerance=PARITY_TOL, a=rows)


# ---------------------------------------------------------------------------------------------
def dtype_of(shp) -> str:
    return {"nvfp4": "nvfp4 (e2m1 x ue4m3, fp32 accumulate)", "w4a8_mx": "mxfp8 x mxfp4 (fp32 accumulate)",
            "w4a16": "bf16 x fp4-dequant (fp32 accumulate)"}[shp.recipe]


def config_of(shp, n_gpus: int, ep: str = "peer", graph: bool = False) -> dict:
    return {"workload": shp.name, "tokens_per_gpu": shp.tokens, "hidden": shp.hidden,
            "intermediate": shp.intermediate, "experts": shp.experts, "top_k": shp.topk,
            "recipe": shp.recipe, "activation": shp.activation, "router": shp.router,
            "parallelism": ("single" if n_gpus == 1 else f"{shp.parallelism}{n_gpus}"),
            "exchange": ("none" if n_gpus == 1 else ("nccl all-reduce" if shp.parallelism == "tp" else ep)),
            "launch": "step replayed from a CUDA graph" if graph else "kernel by kernel",
            "l2": "no flush: the operands read per step (weights, or tokens x weights at prefill) exceed the 126 MB L2"}


def make_layer(shp, dev, rank, world, ep):
    from b12x_b200.moe.distributed import ExpertParallelMoE, TensorParallelMoE
    if world > 1 and shp.parallelism == "tp":
        return TensorParallelMoE.from_synthetic(shp, dev, rank, world)
    if world > 1 and ep == "peer":
        # dispatch / combine by this library's kernels over NVLink peer memory
        from b12x_b200.moe.ep_peer import PeerExpertParallelMoE
        # skewed routing: one spare expert slot per rank, filled with copies of the hot experts
        return PeerExpertParallelMoE.from_synthetic(shp, dev, rank, world,
                                                    replica_slots=1 if shp.zipf_s > 0 else 0)
    return ExpertParallelMoE.from_synthetic(shp, dev, rank, world)


def run_workload(key, shp, args, dev, rank, world, sampler, *, steps, warmup) -> dict:
    """Time one workload: device-resident leg (graph replay where the step allows it), a short eager
    leg for per-stage times, the end-to-end leg with host buffers, the sampled oracle check."""
    layer = make_layer(shp, dev, rank, world, args.ep)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    # host-side inputs (pinned) for the end-to-end leg, device-resident copies for the kernel leg
    x_host = layer.inputs.x.cpu().pin_memory()
    lg_host = layer.inputs.router_logits.cpu().pin_memory()
    out_host = torch.empty((shp.tokens, shp.hidden), dtype=torch.bfloat16).pin_memory()
    x_dev = layer.inputs.x.to(dev)
    lg_dev = layer.inputs.router_logits.to(dev)

    for _ in range(max(warmup, 3)):
        layer.forward(x_dev, lg_dev)
    barrier()
    # a step without host-dependent arguments (one GPU; the peer-memory expert-parallel step) is
    # captured once in a CUDA graph and replayed, the way the reference times its layer
    graph = None
    if layer.can_capture and not args.no_graph:
        layer.x_stage.copy_(x_dev)
        layer.lg_stage.copy_(lg_dev)
        graph = layer.capture()
        for _ in range(3):
            graph.replay()
        barrier()
    sampler.wait_first()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    mark_lo = sampler.mark()
    e0.record()
    if graph is not None:
        for _ in range(steps):
            graph.replay()
    else:
        for _ in range(steps):
            layer.forward(x_dev, lg_dev)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / steps
    # per-stage times: a short kernel-by-kernel leg with an event at every stage boundary, inside
    # the clock-sampled region
    timer = StageTimer()
    for _ in range(max(min(steps // 4, 16), 4)):
        layer.forward(x_dev, lg_dev, stage_timer=timer)
    barrier()
    layer.check_status()

    # ---------------- end-to-end leg: host buffers in, host buffer out ----------------
    for _ in range(3):
        layer.forward_host(x_host, lg_host, out_host)
    barrier()
    h0, h1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_steps = max(steps // 2, 1)
    barrier()
    h0.record()
    for _ in range(e2e_steps):
        layer.forward_host(x_host, lg_host, out_host)
    h1.record()
    barrier()
    ms_e2e = h0.elapsed_time(h1) / e2e_steps
    clocks = sampler.window(mark_lo, sampler.mark())   # all timed legs run between the marks
    # the end-to-end leg may have run the batch in chunks: one more whole step, so that the work
    # statistics and the oracle check below see the full batch
    layer.forward(x_dev, lg_dev)
    barrier()

    stages = timer.mean_ms()
    stats = layer.work_stats()   # algorithmic bytes / flops of the dominant kernel on this rank
    peaks = load_peaks()
    # per-GPU step roofline: what this rank's share of the work needs at the peak that bounds it
    dom = stats["dominant"]
    rate = dom["bf16_rate_multiple"]
    step_flops = stats["rows"] * shp.flops / shp.rows * (1.0 / world if (world > 1 and shp.parallelism == "tp") else 1.0)
    step_bytes = stats["active_experts"] * replace(shp, intermediate=layer.local_intermediate).expert_weight_bytes()
    ideal_ms = max(step_flops / (peaks["bf16_tflops"] * rate * 1e12), step_bytes / (peaks["hbm_gbs"] * 1e9)) * 1e3
    if world > 1:
        red = torch.tensor([ms, ms_e2e, ideal_ms, float(stats["rows"])], device=dev, dtype=torch.float64)
        mx = red.clone()
        torch.distributed.all_reduce(mx, op=torch.distributed.ReduceOp.MAX)
        torch.distributed.all_reduce(red, op=torch.distributed.ReduceOp.SUM)
        ms, ms_e2e, ideal_max, rows_max = mx.tolist()
        ideal_mean, rows_mean = red[2].item() / world, red[3].item() / world
    else:
        ideal_max = ideal_mean = ideal_ms
        rows_max = rows_mean = float(stats["rows"])

    parity = None if args.no_parity else parity_sample(layer)

    tp = world > 1 and shp.parallelism == "tp"
    total_tokens = shp.tokens if tp else shp.tokens * world
    dom_ms = stages.get(dom["stage"], float("nan"))
    if dom["bound"] == "hbm":
        achieved = dom["bytes"] / (dom_ms * 1e-3) / 1e9
        peak, unit = peaks["hbm_gbs"], "GB/s"
    else:
        achieved = dom["flops"] / (dom_ms * 1e-3) / 1e12
        peak, unit = peaks["bf16_tflops"] * rate, "TFLOP/s"
    ratio = NCU_FC1_TRAFFIC_RATIO.get(shp.name)
    traffic = dom["bytes"] * ratio if ratio is not None else None
    rec = {
        "value": total_tokens / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms,
        "scaling": "strong" if tp else "weak", "dtype": dtype_of(shp),
        "config": dict(config_of(shp, world, args.ep, graph is not None),
                       **({"replicated_experts": {"spare_slots_per_rank": layer.replicas.slots_per_rank,
                                                  "copies": [list(x) for x in layer.replicas.extra]}}
                          if getattr(layer, "replicas", None) is not None else {})), "clocks": clocks,
        "e2e": {"value": total_tokens / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": x_host.numel() * 2 + lg_host.numel() * 4,
                "d2h_bytes_per_step": out_host.numel() * 2},
        "gpu_launches": steps * layer.kernels_per_step,
        "tflops": shp.flops * (1 if tp else world) / (ms * 1e-3) / 1e12,
        "stage_ms": stages,
        "roofline": {"kernel": dom["kernel"], "bound": dom["bound"], "achieved": achieved, "peak": peak,
                     "unit": unit, "frac": achieved / peak, "peak_source": peaks["source"] + dom.get("peak_note", ""),
                     "traffic": traffic, "algorithmic_bytes": dom["bytes"],
                     "algorithmic_flops": dom["flops"], "ms_per_launch": dom_ms,
                     "launches_timed": len(timer.steps), "active_experts": stats.get("active_experts")},
        # the whole step of one GPU against the peak that bounds it (expert weights owned / HBM peak,
        # or flops owned / tensor peak): the slowest rank's ideal over the measured step time
        "step_roofline": {"ideal_ms_max_rank": ideal_max, "ideal_ms_mean_rank": ideal_mean,
                          "frac": ideal_max / ms, "frac_balanced": ideal_mean / ms,
                          "load_balance": rows_mean / max(rows_max, 1.0)},
        "parity_sample": parity,
    }
    del layer, x_dev, lg_dev
    gc.collect()
    torch.cuda.empty_cache()
    return rec


def compact(rec: dict) -> dict:
    r = rec["roofline"]
    return {"workload": rec["config"]["workload"], "parallelism": rec["config"]["parallelism"],
            "tokens_per_gpu": rec["config"]["tokens_per_gpu"], "value": rec["value"], "unit": rec["unit"],
            "scaling": rec["scaling"], "ms_per_step": rec["ms_per_step"], "tflops": rec["tflops"],
            "e2e_ms_per_step": rec["e2e"]["ms_per_step"], "stage_ms": rec["stage_ms"],
            "roofline": {k: r[k] for k in ("kernel", "bound", "achieved", "peak", "unit", "frac", "ms_per_launch")},
            "step_roofline": rec["step_roofline"], "clocks": rec["clocks"], "parity_sample": rec["parity_sample"],
            "gpu_launches": rec["gpu_launches"], "config": rec["config"]}


def main():
    args = parse_args()
    shp = synth.shape(args.workload)
    over = {}
    if args.tokens is not None:
        over["tokens"] = args.tokens
    if args.experts is not None:
        over["experts"] = args.experts
        over["name"] = f"{shp.name}_e{args.experts}"
    if over:
        shp = synth.shape(args.workload, **over)
    if args.impl == "reference":
        run_reference(args, shp)
        return

    from b12x_b200.moe import fused_moe
    from b12x_b200.moe.distributed import init_process_group

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run")
    if not torch.cuda.is_available():
        raise SystemExit("this benchmark needs an sm_100 GPU and the built extension (no fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        init_process_group(dev)
    if not fused_moe.is_supported(dev):
        raise SystemExit("this benchmark needs an sm_100 GPU and the built extension (no fallback)")

    sampler = ClockSampler(local_rank)
    sampler.start()
    head = run_workload(args.workload, shp, args, dev, rank, world, sampler, steps=args.steps, warmup=args.warmup)
    subs = []
    if args.sub.lower() != "none":
        for key in [k.strip() for k in args.sub.split(",") if k.strip()]:
            if key == args.workload or key not in synth.SHAPES:
                continue
            s_shp = synth.shape(key)
            if world > 1 and s_shp.parallelism != "tp" and s_shp.experts % world:
                continue
            sub_steps = max(args.steps // 2, 5)
            subs.append(compact(run_workload(key, s_shp, args, dev, rank, world, sampler, steps=sub_steps,
                                             warmup=args.warmup)))
    sampler.stop()

    failed = []
    if rank == 0:
        line = {"metric": "moe_layer_tokens_per_s", "value": head["value"], "unit": head["unit"], "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": head["ms_per_step"],
                "higher_is_better": True, "scaling": head["scaling"], "vs_baseline": None, "dtype": head["dtype"],
                "data": "synthetic"}
        line.update({k: head[k] for k in ("config", "clocks", "e2e", "gpu_launches", "tflops", "stage_ms",
                                          "roofline", "step_roofline", "parity_sample")})
        line["workloads"] = subs
        if not args.no_cpu_baseline and world == 1:
            cores = os.cpu_count() or 1
            torch.set_num_threads(cores)
            inp, ids, w, lo, n_e = cpu_sample_inputs(shp, args.cpu_experts or CPU_EXPERTS.get(args.workload, 8))
            # bounded sample: repeat the pass until about ten seconds of CPU work are on the clock
            total, reps, kept = 0.0, 0, 0
            while total < 10.0 and reps < 64:
                sec, kept = oracle_sample(shp, inp, ids, w, lo, n_e)
                total += sec
                reps += 1
            sec = total / reps
            line["cpu_baseline"] = {"value": (kept / shp.topk) / sec, "unit": "tokens/s", "cores": cores,
                                    "kind": "port", "seconds": total, "passes": reps,
                                    "sample": sample_text(shp, lo, n_e, kept) + f", {reps} passes"}
        print(json.dumps(line), flush=True)
        for rec in [head] + subs:
            p = rec.get("parity_sample")
            if p is not None and not p["ok"]:
                failed.append((rec.get("workload") or rec["config"]["workload"], p))
    if world > 1:
        torch.distributed.destroy_process_group()
    if failed:
        print(f"parity sample failed: {failed}", file=sys.stderr)
        raise SystemExit(3)


if __name__ == "__main__":
    main()
