#!/usr/bin/env python
"""Benchmark of the fused MoE layer on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--tokens T] [--impl reference]

One step = one pass of the layer (route -> sort -> quantise -> FC1+activation -> FC2 -> combine)
over one batch of seeded synthetic input.  The default workload is the DeepSeek-V3-shaped decode
layer (hidden 7168, intermediate 2048, 256 experts, top-8, NVFP4 W4A4, 64 tokens per GPU); with
N > 1 the experts are block-partitioned over the ranks (expert parallelism; tokens are exchanged by
the library's own kernels over NVLink peer memory, `--ep nccl` selects the NCCL all-to-all variant)
and every rank brings its own batch (weak scaling).  Rank 0 prints ONE JSON line.

`--impl reference` times the CPU oracle (the restatement of the reference library's own torch
implementation of this layer) on the host cores for the same configuration.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from b12x_b200 import synth  # noqa: E402

KERNELS_PER_STEP = 6  # route_topk, expert_sort, permute_quant, gemm1, gemm2, combine
NCU_FC1_TRAFFIC_RATIO = 1.014


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="c2", choices=sorted(synth.SHAPES))
    ap.add_argument("--tokens", type=int, default=None, help="tokens per GPU (default: the workload's)")
    ap.add_argument("--experts", type=int, default=None, help="override the expert count (small profiling cases)")
    ap.add_argument("--ep", default="peer", choices=["peer", "nccl"],
                    help="expert-parallel exchange: own kernels over peer memory, or NCCL all-to-all")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch the step kernel by kernel instead of replaying a CUDA graph")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-experts", type=int, default=8, help="experts in the CPU-baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    return ap.parse_args()


def load_peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clock / throttle sampling during the timed region."""

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
        except OSError:
            return []

    def wait_first(self, timeout_s: float = 4.0) -> None:
        """Block until nvidia-smi has written its first sample (its start-up takes about a second)."""
        t0 = time.perf_counter()
        while self.proc is not None and not self._lines() and time.perf_counter() - t0 < timeout_s:
            time.sleep(0.02)

    def mark(self) -> int:
        """Index of the next sample: brackets the timed region."""
        return len(self._lines())

    def stop(self, lo: int = 0, hi: int | None = None) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        lines = self._lines()
        hi = len(lines) if hi is None else hi
        # a region shorter than the sampling period: take the samples either side of it
        window = lines[lo:hi] if hi > lo else lines[max(lo - 1, 0):hi + 1]
        sm, smax, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in window:
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
        os.unlink(self.path)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(smax) if smax else None, "samples": len(sm), "reasons": sorted(reasons)}


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


def oracle_sample(shp, inp_cpu, ids, weights, n_experts: int):
    """CPU oracle on the routes of the batch that land on the first ``n_experts`` experts."""
    from oracle import moe_oracle as O
    emap = torch.full((shp.experts,), -1, dtype=torch.int32)
    emap[:n_experts] = torch.arange(n_experts, dtype=torch.int32)
    kept = int((ids < n_experts).sum())
    t0 = time.perf_counter()
    if shp.recipe == "nvfp4":
        a1 = inp_cpu.w1_global_scale / inp_cpu.a1_gscale
        a2 = inp_cpu.w2_global_scale / inp_cpu.a2_gscale
        O.moe_nvfp4(inp_cpu.x, inp_cpu.w1_fp4, inp_cpu.w1_blockscale, a1, inp_cpu.w2_fp4, inp_cpu.w2_blockscale,
                    a2, inp_cpu.a1_gscale, inp_cpu.a2_gscale, ids, weights, activation=shp.activation,
                    expert_map=emap)
    elif shp.recipe == "w4a16":
        O.moe_w4a16(inp_cpu.x, inp_cpu.w1_fp4, inp_cpu.w1_blockscale, inp_cpu.w1_global_scale, inp_cpu.w2_fp4,
                    inp_cpu.w2_blockscale, inp_cpu.w2_global_scale, ids, weights, activation=shp.activation,
                    expert_map=emap)
    else:
        ones = torch.ones(n_experts)
        O.moe_w4a8_mx(inp_cpu.x, inp_cpu.w1_fp4, inp_cpu.w1_blockscale, ones, inp_cpu.w2_fp4,
                      inp_cpu.w2_blockscale, ones, ids, weights, activation=shp.activation, expert_map=emap)
    return time.perf_counter() - t0, kept


def cpu_inputs(shp, n_experts: int, seed: int):
    """Host copy of the workload restricted to ``n_experts`` experts' weights (seeded on the host)."""
    return synth.make_inputs(shp, seed=seed, device="cpu", experts=n_experts)


def run_reference(args, shp):
    """The reference's CPU implementation of the path (oracle port), all host threads."""
    from oracle import moe_oracle as O
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    n_e = min(args.cpu_experts, shp.experts)
    inp = cpu_inputs(shp, n_e, seed=0)
    if shp.router == "sigmoid":
        _, ids, w = O.route_topk(inp.router_logits, shp.topk, mode="sigmoid", route_scale=shp.route_scale)
    else:
        _, ids, w = O.route_topk(inp.router_logits, shp.topk)
    times, kept = [], 0
    for i in range(args.warmup + args.steps):
        dt, kept = oracle_sample(shp, inp, ids, w, n_e)
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
                         "sample": f"routes of one {shp.tokens}-token batch that land on experts 0..{n_e - 1} "
                                   f"({kept} of {shp.rows} routed rows); tokens = rows / top-k"},
        "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "tflops": kept * shp.flops / shp.rows / sec / 1e12,
    }
    print(json.dumps(line), flush=True)


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
            "l2": "no flush: the expert weights read per step exceed the 126 MB L2"}


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
    from b12x_b200.moe.distributed import ExpertParallelMoE, TensorParallelMoE, init_process_group

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        init_process_group(dev)
    if not fused_moe.is_supported(dev):
        raise SystemExit("this benchmark needs an sm_100 GPU and the built extension (no fallback)")

    if world > 1 and shp.parallelism == "tp":
        layer = TensorParallelMoE.from_synthetic(shp, dev, rank, world)
    elif world > 1 and args.ep == "peer":
        # dispatch / combine by this library's kernels over NVLink peer memory
        from b12x_b200.moe.ep_peer import PeerExpertParallelMoE
        layer = PeerExpertParallelMoE.from_synthetic(shp, dev, rank, world)
    else:
        layer = ExpertParallelMoE.from_synthetic(shp, dev, rank, world)

    # host-side inputs (pinned) for the end-to-end leg, device-resident copies for the kernel leg
    x_host = layer.inputs.x.cpu().pin_memory()
    lg_host = layer.inputs.router_logits.cpu().pin_memory()
    out_host = torch.empty((shp.tokens, shp.hidden), dtype=torch.bfloat16).pin_memory()
    x_dev = layer.inputs.x.to(dev)
    lg_dev = layer.inputs.router_logits.to(dev)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    # ---------------- device-resident leg ----------------
    sampler = ClockSampler(local_rank)
    sampler.start()
    timer = StageTimer()
    for i in range(args.warmup):
        layer.forward(x_dev, lg_dev, stage_timer=timer if i >= args.warmup // 2 else None)
    barrier()
    # a step without host-dependent arguments (one GPU; the peer-memory expert-parallel step) is
    # captured once in a CUDA graph and replayed, the way the reference times its layer
    # (per-stage events then come from the eager warm-up passes above)
    graph = None
    if layer.can_capture and not args.no_graph:
        layer.x_stage.copy_(x_dev)
        layer.lg_stage.copy_(lg_dev)
        graph = layer.capture()
        for _ in range(3):
            graph.replay()
        barrier()
        timer.steps = timer.steps[-max(args.warmup - args.warmup // 2, 1):]
    else:
        timer = StageTimer()
    sampler.wait_first()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    mark_lo = sampler.mark()
    e0.record()
    if graph is not None:
        for _ in range(args.steps):
            graph.replay()
    else:
        for _ in range(args.steps):
            layer.forward(x_dev, lg_dev, stage_timer=timer)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / args.steps
    layer.check_status()

    # ---------------- end-to-end leg: host buffers in, host buffer out ----------------
    for _ in range(min(args.warmup, 5)):
        layer.forward_host(x_host, lg_host, out_host)
    barrier()
    h0, h1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_steps = max(args.steps // 2, 1)
    barrier()
    h0.record()
    for _ in range(e2e_steps):
        layer.forward_host(x_host, lg_host, out_host)
    h1.record()
    barrier()
    ms_e2e = h0.elapsed_time(h1) / e2e_steps
    clocks = sampler.stop(mark_lo, sampler.mark())   # both timed legs run between the marks

    if world > 1:
        tmax = torch.tensor([ms, ms_e2e], device=dev, dtype=torch.float64)
        torch.distributed.all_reduce(tmax, op=torch.distributed.ReduceOp.MAX)
        ms, ms_e2e = tmax.tolist()

    stages = timer.mean_ms()
    peaks = load_peaks()
    stats = layer.work_stats()   # algorithmic bytes / flops of the dominant kernel on this rank
    if rank == 0:
        # tensor parallelism replicates the tokens (strong scaling); expert parallelism gives every rank its own batch
        tp = world > 1 and shp.parallelism == "tp"
        total_tokens = shp.tokens if tp else shp.tokens * world
        dom = stats["dominant"]
        dom_ms = stages.get(dom["stage"], float("nan"))
        if dom["bound"] == "hbm":
            achieved = dom["bytes"] / (dom_ms * 1e-3) / 1e9
            peak, unit = peaks["hbm_gbs"], "GB/s"
        else:
            achieved = dom["flops"] / (dom_ms * 1e-3) / 1e12
            peak, unit = peaks["bf16_tflops"] * dom["bf16_rate_multiple"], "TFLOP/s"
        # DRAM bytes per FC1 launch: ncu on the 32-expert case of this workload read 1.014 x the
        # algorithmic bytes (dram__bytes_read + write; summary under profiles/); every active
        # expert's weights are read once per launch, so the traffic scales with the algorithmic bytes
        traffic = dom["bytes"] * NCU_FC1_TRAFFIC_RATIO if (dom["bound"] == "hbm" and shp.recipe == "nvfp4") else None
        line = {
            "metric": "moe_layer_tokens_per_s", "value": total_tokens / (ms * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong" if tp else "weak", "vs_baseline": None, "dtype": dtype_of(shp),
            "data": "synthetic", "config": config_of(shp, world, args.ep, graph is not None), "clocks": clocks,
            "e2e": {"value": total_tokens / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": x_host.numel() * 2 + lg_host.numel() * 4,
                    "d2h_bytes_per_step": out_host.numel() * 2},
            "gpu_launches": args.steps * layer.kernels_per_step,
            "tflops": shp.flops * (1 if tp else world) / (ms * 1e-3) / 1e12,
            "stage_ms": stages,
            "roofline": {"kernel": dom["kernel"], "bound": dom["bound"], "achieved": achieved, "peak": peak,
                         "unit": unit, "frac": achieved / peak, "peak_source": peaks["source"] + dom.get("peak_note", ""),
                         "traffic": traffic, "algorithmic_bytes": dom["bytes"],
                         "algorithmic_flops": dom["flops"], "ms_per_launch": dom_ms,
                         "active_experts": stats.get("active_experts")},
        }
        if not args.no_cpu_baseline:
            cores = os.cpu_count() or 1
            torch.set_num_threads(cores)
            n_e = min(args.cpu_experts, shp.experts)
            inp_cpu = cpu_inputs(shp, n_e, seed=0)
            from oracle import moe_oracle as O
            if shp.router == "sigmoid":
                _, ids, w = O.route_topk(inp_cpu.router_logits, shp.topk, mode="sigmoid", route_scale=shp.route_scale)
            else:
                _, ids, w = O.route_topk(inp_cpu.router_logits, shp.topk)
            # bounded sample: repeat the pass until about ten seconds of CPU work are on the clock
            total, reps, kept = 0.0, 0, 0
            while total < 10.0 and reps < 64:
                sec, kept = oracle_sample(shp, inp_cpu, ids, w, n_e)
                total += sec
                reps += 1
            sec = total / reps
            line["cpu_baseline"] = {
                "value": (kept / shp.topk) / sec, "unit": "tokens/s", "cores": cores, "kind": "port",
                "seconds": total, "passes": reps,
                "sample": f"routes of one {shp.tokens}-token batch that land on experts 0..{n_e - 1} "
                          f"({kept} of {shp.rows} routed rows), {reps} passes; tokens = rows / top-k"}
        print(json.dumps(line), flush=True)
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
