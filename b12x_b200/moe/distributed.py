"""Multi-GPU partitioning of the MoE layer: one process per GPU, NCCL over NVLink.

* ``ExpertParallelMoE``: experts are block-partitioned over the ranks, every rank routes its own
  tokens, rows travel to the rank that owns their expert (all-to-all-v), the per-route FC2 rows
  travel back as fp32 and are combined on the home rank in slot order -- so the result is
  bit-identical to the single-GPU layer.  With one rank it is the plain layer.
* ``TensorParallelMoE``: every rank holds an ``I / n`` slice of every expert (FC1 rows of both
  halves, FC2 columns), inputs and routing are replicated, partial outputs are summed with an
  all-reduce -- the contract of the reference's "tensor-parallel" use of fused_moe
  (b12x/moe/__init__.py:3-8).

The reference has no token all-to-all: its ``ep_moe`` replicates the input on every rank and lets
the caller sum partial outputs (b12x/moe/ep_moe/_impl.py:1-14).
"""

from __future__ import annotations

import os
import time
from dataclasses import replace
from datetime import timedelta

import torch
import torch.distributed as dist

from .. import synth
from .._lib import ext
from . import fused_moe
from .fused_moe.stages import StageArena

_ACT_API = {"silu": "silu", "relu2": "relu2", "swigluoai": "swigluoai_uninterleave", "situ": "situ"}
_SOURCE = {"nvfp4": "modelopt_nvfp4", "w4a16": "modelopt_nvfp4", "w4a8_mx": "fp4_e8m0_k32"}


def init_process_group(device: torch.device, timeout_s: float | None = None) -> None:
    """One process per GPU over NCCL (gloo for CPU ranks).  ``timeout_s`` bounds every collective:
    a rank that never joins one ends it with an error on the others instead of a hang."""
    if dist.is_initialized():
        return
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    backend = "nccl" if device.type == "cuda" else "gloo"
    kw = {"device_id": device} if device.type == "cuda" else {}
    if timeout_s is not None:
        kw["timeout"] = timedelta(seconds=float(timeout_s))
    dist.init_process_group(backend=backend, **kw)


# ---------------------------------------------------------------------------------------------
# host-side failure detection (no device involvement: everything here runs before a launch)
# ---------------------------------------------------------------------------------------------
ERR_OVERFLOW = 1      # a rank would receive more rows than its receive capacity
ERR_BAD_TABLE = 2     # a rank's split table is malformed


def validate_split_tables(send_counts, recv_counts, world: int, max_send_rows: int) -> None:
    """Shape and range checks of one rank's split tables (rows it sends to / receives from every
    rank).  Raises ``ValueError`` naming the defect."""
    for name, tab in (("send", send_counts), ("recv", recv_counts)):
        if len(tab) != world:
            raise ValueError(f"{name} split table has {len(tab)} entries for {world} ranks")
        if any(int(c) < 0 for c in tab):
            raise ValueError(f"{name} split table holds a negative count: {list(tab)}")
    if sum(int(c) for c in send_counts) > max_send_rows:
        raise ValueError(f"send split table sums to {sum(send_counts)} rows, this rank has {max_send_rows}")


def agree_on_error(code: int, device: torch.device) -> int:
    """All ranks learn the largest error code any of them raised (one tiny all-reduce): a failure
    that one rank sees on the host becomes an exception on every rank BEFORE any of them enters the
    row exchange, instead of leaving the others inside a collective that never completes."""
    flag = torch.tensor([int(code)], dtype=torch.int32, device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    return int(flag.item())


def check_same_plan(signature: tuple, device: torch.device) -> None:
    """Every rank must have built the layer from the same plan (shape, top-k, expert count,
    recipe ...).  Raises ``ValueError`` on all ranks if any two signatures differ."""
    mine = torch.tensor([int(v) for v in signature], dtype=torch.int64, device=device)
    world = dist.get_world_size()
    every = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(every, mine)
    base = every[0].tolist()
    for r, sig in enumerate(every):
        if sig.tolist() != base:
            raise ValueError(f"rank {r} planned the layer as {sig.tolist()}, rank 0 as {base}")


class PeerLiveness:
    """Heartbeat over the rendezvous store: every rank records the step it is about to run; before
    launching, a rank checks that all peers got there too.  A rank that left between steps is found
    on the host, within ``timeout_s``, with none of this rank's kernels or collectives in flight."""

    def __init__(self, store, rank: int, world: int, *, prefix: str = "b200moe/alive", timeout_s: float = 5.0):
        self.store, self.rank, self.world = store, rank, world
        self.prefix, self.timeout_s = prefix, float(timeout_s)

    def beat(self, step: int) -> None:
        self.store.set(f"{self.prefix}/{self.rank}", str(int(step)))

    def check(self, step: int) -> None:
        deadline = time.monotonic() + self.timeout_s
        for r in range(self.world):
            if r == self.rank:
                continue
            key = f"{self.prefix}/{r}"
            while True:
                seen = -1
                try:
                    if self.store.check([key]):
                        seen = int(self.store.get(key).decode())
                except (RuntimeError, ValueError):
                    seen = -1
                if seen >= step:
                    break
                if time.monotonic() > deadline:
                    raise RuntimeError(f"rank {r} did not reach step {step} within {self.timeout_s:g} s "
                                       f"(last seen at step {seen})")
                time.sleep(0.01)


def prepare_experts(inp: synth.MoEInputs, dev: torch.device):
    """``plan_weights`` + ``prepare_weights`` for synthetic inputs."""
    shp = inp.shape
    wp = fused_moe.plan_weights(
        quant_modes=shp.recipe, source_format=_SOURCE[shp.recipe], activation=_ACT_API[shp.activation],
        params_dtype=torch.bfloat16, num_experts=inp.w1_fp4.shape[0], hidden_size=shp.hidden,
        intermediate_size=inp.w2_fp4.shape[2] * 2)
    kw = dict(plan=wp, params_dtype=torch.bfloat16, w1_fp4=inp.w1_fp4.to(dev), w2_fp4=inp.w2_fp4.to(dev),
              w1_blockscale=inp.w1_blockscale.to(dev), w2_blockscale=inp.w2_blockscale.to(dev))
    if shp.recipe == "nvfp4":
        kw.update(w1_global_scale=inp.w1_global_scale.to(dev), w2_global_scale=inp.w2_global_scale.to(dev),
                  a1_gscale=inp.a1_gscale.to(dev), a2_gscale=inp.a2_gscale.to(dev))
    elif shp.recipe == "w4a16":
        kw.update(w1_global_scale=inp.w1_global_scale.to(dev), w2_global_scale=inp.w2_global_scale.to(dev))
    return fused_moe.prepare_weights(**kw)


def split_counts_exchange(send_counts: torch.Tensor, group=None) -> torch.Tensor:
    """recv_counts[r] = rows rank r will send to this rank (tiny all-to-all of int32)."""
    recv = torch.empty_like(send_counts)
    dist.all_to_all_single(recv, send_counts, group=group)
    return recv


def sort_launches(routes: int) -> int:
    """Kernels of one expert sort: one CTA up to 16 383 routes, count / scan / scatter above."""
    return 3 if routes >= 16384 else 1


def gemm_launches(rows: int, experts: int) -> int:
    """Kernels of FC1 + FC2: one each; plans with two to eight row tiles per expert run the CTA-pair
    kernel on full pairs and a single-CTA kernel on the left-over row tiles (two each)."""
    return 4 if 256 * experts <= rows < 1024 * experts else 2


class _LayerBase:
    kernels_per_step = 6

    def __init__(self, shp: synth.MoEShape, inputs: synth.MoEInputs, experts, dev, rank: int, world: int):
        self.shape, self.inputs, self.experts = shp, inputs, experts
        self.dev, self.rank, self.world = dev, rank, world
        t, k = shp.tokens, shp.topk
        self.topk_logits = torch.empty((t, k), dtype=torch.float32, device=dev)
        self.topk_ids = torch.empty((t, k), dtype=torch.int32, device=dev)
        self.topk_weights = torch.empty((t, k), dtype=torch.float32, device=dev)
        self.out = torch.empty((t, shp.hidden), dtype=torch.bfloat16, device=dev)
        self.x_stage = torch.empty((t, shp.hidden), dtype=torch.bfloat16, device=dev)
        self.lg_stage = torch.empty((t, shp.experts), dtype=torch.float32, device=dev)
        self.last_binding = None
        self.graph = None     # a captured step on (x_stage, lg_stage), where the layer offers one
        self._copy_streams = None
        self._chunk_graphs = None

    @property
    def local_intermediate(self) -> int:
        """Intermediate columns this rank holds (the whole of it unless the layer is tensor-parallel)."""
        return int(self.inputs.w2_fp4.shape[2]) * 2

    def route(self, logits: torch.Tensor, lo: int = 0) -> None:
        shp = self.shape
        hi = lo + int(logits.shape[0])
        tl, ti, tw = self.topk_logits[lo:hi], self.topk_ids[lo:hi], self.topk_weights[lo:hi]
        if shp.router == "sigmoid":
            fused_moe.route_topk(logits, tl, ti, tw, renormalize=True, score_func="sigmoid",
                                 route_scale=shp.route_scale)
        else:
            fused_moe.route_topk(logits, tl, ti, tw, renormalize=True)

    def host_chunks(self) -> int:
        """Token chunks ``forward_host`` pipelines (1 = no pipelining).  A layer that can run a token
        slice on its own overrides ``forward_slice`` and this."""
        return 1

    def forward_slice(self, lo: int, hi: int) -> None:
        raise NotImplementedError

    @staticmethod
    def _chunk_bounds(tokens: int, n: int) -> list:
        """Token ranges of the pipeline's chunks.  The first and the last chunk are half as large as
        the others: nothing overlaps the first copy in and the last copy out, so they are kept short."""
        parts = [1] + [2] * (n - 1) + [1] if n >= 2 else [1]
        total, acc, bounds = sum(parts), 0, []
        for p in parts:
            lo, acc = acc, acc + p
            bounds.append((lo * tokens // total // 8 * 8, acc * tokens // total // 8 * 8 if acc < total else tokens))
        return [(lo, hi) for lo, hi in bounds if hi > lo]

    def _capture_chunks(self, bounds) -> dict:
        """One CUDA graph per token chunk of the staging buffers (the chunk's route + layer)."""
        torch.cuda.synchronize(self.dev)
        graphs = {}
        for lo, hi in bounds:
            self.forward_slice(lo, hi)          # warm-up outside the capture
            torch.cuda.synchronize(self.dev)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self.forward_slice(lo, hi)
            graphs[(lo, hi)] = g
        torch.cuda.synchronize(self.dev)
        return graphs

    def forward_host(self, x_host: torch.Tensor, logits_host: torch.Tensor, out_host: torch.Tensor) -> None:
        """Host buffers in, host buffer out.

        One chunk: H2D copies, the layer, D2H copy, all on the current stream.  Several chunks (large
        batches on one GPU): the copies of chunk c+1 / c-1 run on two side streams while chunk c
        computes, so the step costs about max(copy in, compute, copy out) plus one chunk's copy at
        either end instead of their sum.  Every token's result is the same either way: a token's
        rows meet no other token's data anywhere in the layer."""
        n = self.host_chunks()
        main = torch.cuda.current_stream(self.dev)
        if n <= 1:
            self.x_stage.copy_(x_host, non_blocking=True)
            self.lg_stage.copy_(logits_host, non_blocking=True)
            if self.graph is not None:
                self.graph.replay()
                out = self.out
            else:
                out = self.forward(self.x_stage, self.lg_stage)
            out_host.copy_(out, non_blocking=True)
            main.synchronize()
            return
        if self._copy_streams is None:
            self._copy_streams = (torch.cuda.Stream(self.dev), torch.cuda.Stream(self.dev))
            self._chunk_events = [(torch.cuda.Event(), torch.cuda.Event()) for _ in range(16)]
        s_in, s_out = self._copy_streams
        bounds = self._chunk_bounds(int(x_host.shape[0]), n)
        s_in.wait_stream(main)
        s_out.wait_stream(main)
        with torch.cuda.stream(s_in):
            for c, (lo, hi) in enumerate(bounds):
                self.x_stage[lo:hi].copy_(x_host[lo:hi], non_blocking=True)
                self.lg_stage[lo:hi].copy_(logits_host[lo:hi], non_blocking=True)
                self._chunk_events[c][0].record(s_in)
        if self._chunk_graphs is None:
            self._chunk_graphs = self._capture_chunks(bounds) if self.can_capture else {}
        for c, (lo, hi) in enumerate(bounds):
            arrived, computed = self._chunk_events[c]
            main.wait_event(arrived)
            g = self._chunk_graphs.get((lo, hi))
            if g is not None:
                g.replay()          # one launch per chunk: the host never falls behind the GPU
            else:
                self.forward_slice(lo, hi)
            computed.record(main)
            s_out.wait_event(computed)
            with torch.cuda.stream(s_out):
                out_host[lo:hi].copy_(self.out[lo:hi], non_blocking=True)
        main.wait_stream(s_out)
        main.synchronize()

    @property
    def can_capture(self) -> bool:
        """True where one step has no host-dependent argument and no host sync, so that it can be
        recorded into a CUDA graph (the reference times its layer the same way: graph replay,
        benchmarks/benchmark_moe.py:155-222)."""
        return False

    def capture(self) -> torch.cuda.CUDAGraph:
        """Record one step on the staging buffers (``x_stage``, ``lg_stage``) into a CUDA graph;
        ``graph.replay()`` is then a full layer pass on whatever those buffers hold, its result in
        ``self.out``.  With several ranks, all must replay the same number of times."""
        if not self.can_capture:
            raise RuntimeError("this layer's step needs the host between its kernels and cannot be captured")
        torch.cuda.synchronize(self.dev)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.forward(self.x_stage, self.lg_stage)
        self.graph = g
        return g

    def check_status(self) -> None:
        if self.last_binding is not None:
            fused_moe.check_device_status(self.last_binding)

    def _local_plan(self, max_tokens: int, topk: int):
        caps = fused_moe.Caps(max_tokens=max_tokens, num_topk=topk, device=self.dev,
                              weight_plan=self.experts.plan, quant_mode=self.shape.recipe)
        plan = fused_moe.plan(caps)
        spec = plan.scratch_specs()[0]
        return plan, torch.empty(spec.shape, dtype=spec.dtype, device=self.dev)

    def _dominant(self, local_shape: synth.MoEShape, active_experts: int, rows: int) -> dict:
        """Algorithmic bytes / flops of the FC1 launch (the largest kernel of the layer)."""
        k, i = local_shape.hidden, local_shape.intermediate
        g = 32 if local_shape.recipe == "w4a8_mx" else 16
        w1_rows = i if local_shape.activation == "relu2" else 2 * i
        a_bytes = {"nvfp4": k / 2 + k / 16, "w4a8_mx": k + k / 32, "w4a16": 2.0 * k}[local_shape.recipe]
        o_bytes = {"nvfp4": i / 2 + i / 16, "w4a8_mx": i + i / 32, "w4a16": 2.0 * i}[local_shape.recipe]
        weight_bytes = active_experts * w1_rows * k * (0.5 + 1.0 / g)
        total_bytes = weight_bytes + rows * (a_bytes + o_bytes)
        flops = 2.0 * rows * w1_rows * k
        # the layer is weight-streaming bound while the rows per expert are few
        # (a 128-row tile needs ~64 rows per active expert before the tensor pipe, not HBM, limits)
        bound = "hbm" if rows < 64 * max(active_experts, 1) else "tensor"
        # tensor rate of the operand type relative to dense bf16 (the measured peak is a bf16 GEMM)
        rate = {"nvfp4": 4.0, "w4a8_mx": 2.0, "w4a16": 1.0}[local_shape.recipe]
        return {"kernel": "grouped_gemm1_act", "stage": "gemm1", "bound": bound, "bytes": total_bytes,
                "flops": flops, "bf16_rate_multiple": rate,
                "peak_note": "" if bound == "hbm" else
                f" bf16 GEMM peak x {rate:g} (the operand type's tensor rate relative to bf16)"}


class ExpertParallelMoE(_LayerBase):
    def __init__(self, shp, inputs, experts, dev, rank=0, world=1, *, recv_capacity_factor: float | None = None):
        super().__init__(shp, inputs, experts, dev, rank, world)
        self.e_local = shp.experts // world
        if shp.experts % world:
            raise ValueError("experts must divide evenly over the ranks")
        t, k = shp.tokens, shp.topk
        if world == 1:
            self.plan, self.scratch = self._local_plan(t, k)
            # route, sort, quantise (w4a16: row gather), FC1, FC2, combine
            self.kernels_per_step = 3 + sort_launches(t * k) + gemm_launches(t * k, shp.experts)
            return
        # home side: sort routes by destination rank, pack rows, later combine returned rows
        self.home = StageArena(t, k, world, shp.hidden, dev)
        self.rank_of_expert = (torch.arange(shp.experts, dtype=torch.int32, device=dev) // self.e_local).contiguous()
        rows = t * k
        self.send_rows = torch.empty((rows, shp.hidden), dtype=torch.bfloat16, device=dev)
        self.send_ids = torch.empty((rows,), dtype=torch.int32, device=dev)
        # expert side: worst case every route of every rank lands here
        cap = rows * world if recv_capacity_factor is None else int(rows * recv_capacity_factor)
        self.recv_cap = cap
        self.recv_rows = torch.empty((cap, shp.hidden), dtype=torch.bfloat16, device=dev)
        self.recv_ids = torch.empty((cap, 1), dtype=torch.int32, device=dev)
        self.recv_ones = torch.ones((cap, 1), dtype=torch.float32, device=dev)
        self.recv_out = torch.empty((cap, shp.hidden), dtype=torch.float32, device=dev)
        self.plan, self.scratch = self._local_plan(cap, 1)
        self.kernels_per_step = 9  # route, rank sort, gather, expert sort, quant, gemm1, gemm2, un-permute, combine
        self.bounded_capacity = recv_capacity_factor is not None
        self.liveness: PeerLiveness | None = None     # set by the caller to have peers checked before every step
        self.step = 0
        check_same_plan((shp.tokens, shp.hidden, shp.intermediate, shp.experts, shp.topk,
                         sorted(synth.SHAPES_RECIPES).index(shp.recipe), cap), dev)

    @property
    def can_capture(self) -> bool:
        return self.world == 1      # the NCCL exchange reads the split sizes on the host

    def host_chunks(self) -> int:
        """On one GPU a large batch is pipelined in up to four token chunks, each with at least 256
        rows per expert so that the grouped GEMMs keep their large-batch tiles."""
        if self.world != 1:
            return 1
        shp = self.shape
        chunk_min = max(256 * shp.experts // shp.topk, 1024)
        cap = int(os.environ.get("B200MOE_HOST_CHUNKS", "4"))
        return max(1, min(cap, shp.tokens // chunk_min))

    def forward_slice(self, lo: int, hi: int) -> None:
        """The layer on tokens [lo, hi) of the staging buffers, result into ``out[lo:hi]``."""
        self.route(self.lg_stage[lo:hi], lo)
        b = fused_moe.bind(self.plan, scratch=self.scratch, a=self.x_stage[lo:hi], experts=self.experts,
                           topk_weights=self.topk_weights[lo:hi], topk_ids=self.topk_ids[lo:hi],
                           output=self.out[lo:hi])
        self.last_binding = b
        fused_moe.run(binding=b)

    @classmethod
    def from_synthetic(cls, shp: synth.MoEShape, dev, rank: int, world: int):
        e_local = shp.experts // world
        inp = synth.make_inputs(shp, seed=1000 + rank, device=dev, experts=e_local)
        return cls(shp, inp, prepare_experts(inp, dev), dev, rank, world)

    @classmethod
    def from_global(cls, full: synth.MoEInputs, dev, rank: int, world: int, tokens_per_rank: int):
        """Shard a global problem: experts [rank*E/n, (rank+1)*E/n) and this rank's token slice."""
        shp = replace(full.shape, tokens=tokens_per_rank)
        e_local = shp.experts // world
        local = synth.slice_experts(full, rank * e_local, (rank + 1) * e_local)
        lo = rank * tokens_per_rank
        local = replace(local, shape=shp, x=full.x[lo:lo + tokens_per_rank].contiguous(),
                        router_logits=full.router_logits[lo:lo + tokens_per_rank].contiguous())
        return cls(shp, local, prepare_experts(local, dev), dev, rank, world)

    def forward(self, x: torch.Tensor, logits: torch.Tensor, stage_timer=None) -> torch.Tensor:
        self.route(logits)
        if self.world == 1:
            b = fused_moe.bind(self.plan, scratch=self.scratch, a=x, experts=self.experts,
                               topk_weights=self.topk_weights, topk_ids=self.topk_ids, output=self.out)
            self.last_binding = b
            return fused_moe.run(binding=b, stage_timer=stage_timer)
        shp = self.shape
        home = self.home
        if self.liveness is not None:
            # a peer that left since the last step is found here, on the host, before anything is launched
            self.liveness.beat(self.step)
            self.liveness.check(self.step)
        self.step += 1
        home.sort(self.topk_ids, self.rank_of_expert)
        send_counts = home.group_counts
        recv_counts = split_counts_exchange(send_counts)
        home.gather_rows(x, self.topk_ids, self.send_rows, self.send_ids, self.e_local)
        counts = torch.stack([send_counts, recv_counts]).cpu()     # the one host sync of the step
        sc, rc = counts[0].tolist(), counts[1].tolist()
        n_send, n_recv = sum(sc), sum(rc)
        if self.bounded_capacity:
            # With a receive capacity below the worst case a rank can overflow.  The decision to stop
            # is collective: every rank raises, none is left inside the row exchange.
            code = 0
            try:
                validate_split_tables(sc, rc, self.world, shp.tokens * shp.topk)
            except ValueError:
                code = ERR_BAD_TABLE
            if n_recv > self.recv_cap:
                code = max(code, ERR_OVERFLOW)
            worst = agree_on_error(code, self.dev)
            if worst == ERR_OVERFLOW:
                raise RuntimeError(f"a rank would receive more rows than its capacity (this rank: "
                                   f"{n_recv} of {self.recv_cap}); no row was exchanged")
            if worst != 0:
                raise RuntimeError("a rank's split table is malformed; no row was exchanged")
        dist.all_to_all_single(self.recv_rows[:n_recv], self.send_rows[:n_send], rc, sc)
        dist.all_to_all_single(self.recv_ids.view(-1)[:n_recv], self.send_ids[:n_send], rc, sc)
        if n_recv > 0:
            b = fused_moe.bind(self.plan, scratch=self.scratch, a=self.recv_rows[:n_recv], experts=self.experts,
                               topk_weights=self.recv_ones[:n_recv], topk_ids=self.recv_ids[:n_recv],
                               output_f32=self.recv_out[:n_recv], f32_only=True)
            self.last_binding = b
            fused_moe.run(binding=b, stage_timer=stage_timer)
        dist.all_to_all_single(home.routed[:n_send], self.recv_out[:n_recv], sc, rc)
        home.combine(self.topk_weights, self.out)
        return self.out

    def work_stats(self) -> dict:
        b = self.last_binding
        counts = b.expert_counts.cpu()
        active = int((counts > 0).sum())
        rows = int(counts.sum())
        local = replace(self.shape, experts=self.e_local)
        return {"dominant": self._dominant(local, active, rows), "active_experts": active, "rows": rows}


class TensorParallelMoE(_LayerBase):
    def __init__(self, shp, inputs, experts, dev, rank=0, world=1):
        super().__init__(shp, inputs, experts, dev, rank, world)
        self.local_shape = replace(shp, intermediate=inputs.w2_fp4.shape[2] * 2)
        self.plan, self.scratch = self._local_plan(shp.tokens, shp.topk)
        self.partial = torch.empty((shp.tokens, shp.hidden), dtype=torch.float32, device=dev)
        # route, sort, row gather / quantise, FC1, FC2, fp32 combine, rounding
        self.kernels_per_step = (4 + sort_launches(shp.tokens * shp.topk)
                                 + gemm_launches(shp.tokens * shp.topk, shp.experts))

    @classmethod
    def from_synthetic(cls, shp: synth.MoEShape, dev, rank: int, world: int):
        if shp.intermediate % world:
            raise ValueError("intermediate size must divide evenly over the ranks")
        local = replace(shp, intermediate=shp.intermediate // world)
        inp = synth.make_inputs(local, seed=2000 + rank, device=dev)
        # tokens and router logits are replicated: every rank draws them from the same seed
        rep = synth.make_inputs(replace(local, experts=shp.experts), seed=7, device=dev, experts=0)
        inp.x, inp.router_logits = rep.x, rep.router_logits
        inp.shape = shp
        return cls(shp, inp, prepare_experts(inp, dev), dev, rank, world)

    @classmethod
    def from_global(cls, full: synth.MoEInputs, dev, rank: int, world: int):
        """Shard a global problem on the intermediate dimension; tokens and routing replicated."""
        local = synth.slice_intermediate(full, rank, world)
        local = replace(local, shape=full.shape)
        return cls(full.shape, local, prepare_experts(local, dev), dev, rank, world)

    def forward(self, x: torch.Tensor, logits: torch.Tensor, stage_timer=None) -> torch.Tensor:
        self.route(logits)
        b = fused_moe.bind(self.plan, scratch=self.scratch, a=x, experts=self.experts,
                           topk_weights=self.topk_weights, topk_ids=self.topk_ids,
                           output_f32=self.partial, f32_only=True)
        self.last_binding = b
        fused_moe.run(binding=b, stage_timer=stage_timer)
        if self.world > 1:
            dist.all_reduce(self.partial)
        ext.check(ext.load().b200moe_round_rows_bf16(
            self.partial.data_ptr(), self.out.data_ptr(), self.partial.numel(),
            torch.cuda.current_stream(self.dev).cuda_stream), "round_rows_bf16")
        return self.out

    def work_stats(self) -> dict:
        counts = self.last_binding.expert_counts.cpu()
        active = int((counts > 0).sum())
        rows = int(counts.sum())
        return {"dominant": self._dominant(self.local_shape, active, rows), "active_experts": active, "rows": rows}
