"""Expert parallelism with the dispatch and the combine done by this library's own kernels over
NVLink peer memory (no NCCL call and no host synchronisation on the step).

Per step, all on one CUDA stream per rank::

    route -> sort by destination rank -> ep_dispatch (peer stores + flags)
          -> expert sort (first waits, bounded, for every peer's flag) / quantise / FC1 / FC2 on
             the received slots
          -> ep_combine (signal "FC2 done", bounded wait for all peers, then peer loads of the
             fp32 FC2 rows + weighted sum, one launch)

Receive buffers, flags and the expert-side scratch arena live in symmetric memory
(``torch.distributed._symmetric_memory``); every rank therefore holds device pointers to all
peers' copies.  Rank ``r`` owns slots ``[r*cap, (r+1)*cap)`` of every receive buffer
(``cap = tokens * top_k``, the worst case), so no counts have to be exchanged: unused slots carry
expert id -1 and the expert-side sort drops them.  The result is bit-identical to the single-GPU
layer (fp32 per-route rows, combined in slot order).
"""

from __future__ import annotations

import ctypes as C
import os
from dataclasses import replace

import torch
import torch.distributed as dist

from .. import synth
from .._lib import ext
from . import fused_moe
from .distributed import _LayerBase, gemm_launches, prepare_experts, sort_launches
from .fused_moe.stages import StageArena
from .placement import plan_expert_replicas


def _symm_empty(shape, dtype, device):
    import torch.distributed._symmetric_memory as symm_mem

    t = symm_mem.empty(*shape, dtype=dtype, device=device)
    hdl = symm_mem.rendezvous(t, dist.group.WORLD)
    # the tensor may sit at an offset inside the symmetric allocation: same offset on every rank
    base = [int(p) for p in hdl.buffer_ptrs]
    off = t.data_ptr() - base[dist.get_rank()]
    if off < 0 or off + t.numel() * t.element_size() > int(hdl.buffer_size):
        raise RuntimeError("symmetric-memory tensor lies outside its rendezvoused buffer")
    return t, [p + off for p in base], hdl


_PAYLOAD_OF_RECIPE = {"nvfp4": "nvfp4", "w4a8_mx": "mxfp8", "w4a16": "bf16"}


class _ReceivedRows:
    """The bf16 rows behind this rank's receive slots, looked up in the ranks' gathered inputs
    (checking aid: with a quantised dispatch the expert rank never holds them)."""

    def __init__(self, xs, sorted_ids, offsets, me: int, cap: int, topk: int):
        self.xs, self.sorted_ids, self.offsets, self.me, self.cap, self.topk = xs, sorted_ids, offsets, me, cap, topk

    def index_select(self, dim: int, slots: torch.Tensor) -> torch.Tensor:
        assert dim == 0
        slots = slots.cpu().long()
        out = torch.empty((slots.numel(), self.xs[0].shape[1]), dtype=self.xs[0].dtype)
        for i, s in enumerate(slots.tolist()):
            src, j = divmod(s, self.cap)
            route = int(self.sorted_ids[src][int(self.offsets[src][self.me]) + j])
            out[i] = self.xs[src][route // self.topk]
        return out


class PeerExpertParallelMoE(_LayerBase):
    kernels_per_step = 12

    def __init__(self, shp, inputs, experts, dev, rank: int, world: int, *,
                 recv_capacity_factor: float | None = None, payload: str | None = None,
                 replica_slots: int = 0, calibration_logits: torch.Tensor | None = None):
        super().__init__(shp, inputs, experts, dev, rank, world)
        if world < 2 or world > ext.MAX_RANKS:
            raise ValueError(f"needs 2..{ext.MAX_RANKS} ranks")
        if shp.experts % world:
            raise ValueError("experts must divide evenly over the ranks")
        self.e_local = shp.experts // world
        # Spare expert slots against skewed routing: hot experts are copied into cold ranks' spare
        # slots (placement from the routing of a calibration batch) and their routes spread over
        # the holders.  Every holder computes the same bytes, so the output does not change.
        self.replicas = None
        gs_own = experts.a1_gscale.reshape(-1).float()
        if replica_slots > 0:
            loads = self._measure_loads(inputs.router_logits if calibration_logits is None else calibration_logits)
            self.replicas = plan_expert_replicas(loads, world, int(replica_slots))
            inputs = self._with_replica_weights(inputs, self.replicas)
            experts = prepare_experts(inputs, dev)
            self.inputs, self.experts = inputs, experts
            pr, pl = self.replicas.pattern_tables()
            self.pattern_rank = torch.tensor(pr, dtype=torch.int32, device=dev)
            self.pattern_local = torch.tensor(pl, dtype=torch.int32, device=dev)
            self.dest_rank = torch.empty((shp.tokens, shp.topk), dtype=torch.int32, device=dev)
            self.dest_local = torch.empty((shp.tokens, shp.topk), dtype=torch.int32, device=dev)
        self.n_local = self.e_local + (int(replica_slots) if self.replicas is not None else 0)
        t, k = shp.tokens, shp.topk
        # Slots one source rank owns in every receive buffer.  Worst case (every route of a rank
        # to one destination) by default; with a capacity factor f, f x the balanced share
        # t*k/world -- a route beyond it is not sent and the step ends with an error status.
        self.cap = t * k
        if recv_capacity_factor is not None:
            if recv_capacity_factor <= 0:
                raise ValueError("recv_capacity_factor must be positive")
            self.cap = max(1, min(t * k, -(-int(t * k * recv_capacity_factor) // world)))
        self.bounded_capacity = self.cap < t * k
        slots = world * self.cap
        self.home = StageArena(t, k, world, shp.hidden, dev)
        self.rank_of_expert = (torch.arange(shp.experts, dtype=torch.int32, device=dev) // self.e_local).contiguous()
        # the two cross-rank waits of a step ride inside the expert sort and the combine kernel
        # unless B200MOE_FOLD_WAITS=0 makes them three launches of their own
        self.fold_waits = os.environ.get("B200MOE_FOLD_WAITS", "1") == "1"
        # route, home sort, dispatch, expert sort, file / quantise rows, FC1, FC2, combine (+ wait, signal, wait)
        self.kernels_per_step = (4 + sort_launches(t * k) + sort_launches(slots) + (0 if self.fold_waits else 3)
                                 + gemm_launches(slots, self.n_local)
                                 + (1 if self.replicas is not None else 0))
        # what crosses the link per route: the row quantised on this rank (the recipe's activation
        # format) or, for recipes whose GEMM reads bf16 rows, the row as it is
        self.payload = payload or os.environ.get("B200MOE_EP_PAYLOAD") or _PAYLOAD_OF_RECIPE[shp.recipe]
        if self.payload not in ext.EP_PAYLOADS or (self.payload != "bf16" and self.payload != _PAYLOAD_OF_RECIPE[shp.recipe]):
            raise ValueError(f"payload {self.payload!r} does not fit recipe {shp.recipe!r}")
        self.done_counter = torch.zeros(1, dtype=torch.int32, device=dev)
        # the step counter lives on the device, so that a captured step can be replayed
        self.epoch_dev = torch.zeros(1, dtype=torch.int32, device=dev)
        # expert side: one plan over all slots, top-1, scratch in symmetric memory
        # the slot capacity is the worst case; with balanced routing an expert receives
        # world * tokens * top_k / experts rows, which decides the tile height of the plan
        expected_rows = world * t * k // shp.experts
        caps = fused_moe.Caps(max_tokens=slots, num_topk=1, device=dev, weight_plan=experts.plan,
                              quant_mode=shp.recipe, tile_rows=64 if expected_rows <= 48 else 128)
        self.plan = fused_moe.plan(caps)
        nbytes = self.plan.scratch_specs()[0].shape[0]
        self.scratch, self.scratch_ptrs, self._h0 = _symm_empty((nbytes,), torch.uint8, dev)
        if self.payload == "bf16":
            self.recv_rows, self.rows_ptrs, self._h1 = _symm_empty((slots, shp.hidden), torch.bfloat16, dev)
            self.recv_sf, self.sf_ptrs, self.packed = None, [0] * world, None
        else:
            row_bytes = shp.hidden // 2 if self.payload == "nvfp4" else shp.hidden
            nsf = shp.hidden // (16 if self.payload == "nvfp4" else 32)
            self.recv_q, self.rows_ptrs, self._h1 = _symm_empty((slots, row_bytes), torch.uint8, dev)
            # scale rows padded to 16 bytes: the sender then stores them 16 bytes at a time
            self.recv_sf, self.sf_ptrs, self._h4 = _symm_empty((slots, (nsf + 15) // 16 * 16), torch.uint8, dev)
            self.packed = (self.recv_q, self.recv_sf)
            # the binding wants a [slots, K] bf16 tensor; it is never read on this path
            self.recv_rows = torch.zeros((1, shp.hidden), dtype=torch.bfloat16, device=dev).expand(slots, shp.hidden)
        self.recv_ids, self.ids_ptrs, self._h2 = _symm_empty((slots, 1), torch.int32, dev)
        self.flags, flag_ptrs, self._h3 = _symm_empty((2 * ext.MAX_RANKS,), torch.int32, dev)
        self.flags.zero_()
        self.recv_ids.fill_(-1)
        self.flag1_ptrs = flag_ptrs
        self.flag2_ptrs = [p + 4 * ext.MAX_RANKS for p in flag_ptrs]
        self.ones = torch.ones((slots, 1), dtype=torch.float32, device=dev)
        self._flag2_arr = (C.c_void_p * world)(*self.flag2_ptrs)
        core = self.plan._core_layout
        self._inv_perm_off = self.plan.layout.route_workspace_nbytes + int(core.inv_perm)
        self._routed_off = self.plan.layout.route_workspace_nbytes + int(core.routed)
        # Status words of the cross-rank waits and of the receive-capacity check.  A buffer of its own,
        # which no kernel clears (the sorts zero the status words of their arenas at every step): an
        # expiry in step n is still there when check_status() is called after step n + 100.
        self.home_status = torch.zeros(16, dtype=torch.int32, device=dev)
        # the senders quantise with the destination expert's input scale: every rank holds all of them
        gs = gs_own.expand(self.e_local).contiguous() if gs_own.numel() == 1 else gs_own.contiguous()
        if gs.numel() != self.e_local:
            raise ValueError("a1_gscale must hold one value or one per local expert")
        parts = [torch.empty_like(gs) for _ in range(world)]
        dist.all_gather(parts, gs)
        self.a1_gscale_all = torch.cat(parts).contiguous()
        torch.cuda.synchronize(dev)
        dist.barrier()

    def _measure_loads(self, logits: torch.Tensor) -> list:
        """COLLECTIVE: routes per global expert over all ranks' calibration batches."""
        if tuple(logits.shape) != (self.shape.tokens, self.shape.experts):
            raise ValueError(f"calibration logits must be [{self.shape.tokens}, {self.shape.experts}], "
                             f"got {tuple(logits.shape)}")
        self.route(logits.to(self.dev))
        counts = torch.bincount(self.topk_ids.reshape(-1).long().clamp(0, self.shape.experts - 1),
                                minlength=self.shape.experts).to(torch.float32)
        dist.all_reduce(counts)
        return counts.cpu().tolist()

    def _with_replica_weights(self, inputs, plan):
        """COLLECTIVE: the local problem with ``slots_per_rank`` more experts appended -- the weights of
        the experts this rank holds copies of, broadcast from their owners (unused spare slots repeat
        the rank's first expert; no route goes there)."""
        names = ("w1_fp4", "w1_blockscale", "w1_global_scale", "w2_fp4", "w2_blockscale", "w2_global_scale",
                 "a1_gscale", "a2_gscale")
        own = {n: getattr(inputs, n).to(self.dev) for n in names}
        got: dict = {n: [] for n in names}
        for holder in range(self.world):
            for e in plan.extra[holder]:
                owner, idx = divmod(e, self.e_local)
                for n in names:
                    t = own[n][idx:idx + 1].contiguous().clone()
                    raw = t.view(torch.uint8) if t.element_size() == 1 else t
                    dist.broadcast(raw, src=owner)
                    if holder == self.rank:
                        got[n].append(t)
        out = {}
        for n in names:
            pad = [own[n][0:1]] * (plan.slots_per_rank - len(got[n]))
            out[n] = torch.cat([own[n]] + got[n] + pad, dim=0).contiguous()
        return replace(inputs, **out)

    def check_status(self) -> None:
        super().check_status()
        st = self.home_status.cpu()
        if int(st[0]) != 0:
            code = int(st[1])
            if code >= 48:
                raise RuntimeError(f"rank {code - 48} was sent more rows than its receive capacity "
                                   f"({self.cap} per source rank) holds; the step's output is invalid")
            raise RuntimeError(f"expert-parallel wait gave up (code {code}: 16 + missing peer rank)")

    @classmethod
    def from_synthetic(cls, shp: synth.MoEShape, dev, rank: int, world: int, **kw):
        e_local = shp.experts // world
        inp = synth.make_inputs(shp, seed=1000 + rank, device=dev, experts=e_local)
        return cls(shp, inp, prepare_experts(inp, dev), dev, rank, world, **kw)

    @classmethod
    def from_global(cls, full: synth.MoEInputs, dev, rank: int, world: int, tokens_per_rank: int, **kw):
        shp = replace(full.shape, tokens=tokens_per_rank)
        e_local = shp.experts // world
        local = synth.slice_experts(full, rank * e_local, (rank + 1) * e_local)
        lo = rank * tokens_per_rank
        local = replace(local, shape=shp, x=full.x[lo:lo + tokens_per_rank].contiguous(),
                        router_logits=full.router_logits[lo:lo + tokens_per_rank].contiguous())
        return cls(shp, local, prepare_experts(local, dev), dev, rank, world, **kw)

    def received_rows(self, x: torch.Tensor) -> _ReceivedRows:
        """COLLECTIVE checking aid: the bf16 rows behind this rank's receive slots after a step on
        ``x``, rebuilt from every rank's input and destination sort (a quantised dispatch leaves
        only codes on the expert rank).  Slot s = source rank * cap + j."""
        torch.cuda.synchronize(self.dev)
        n = self.shape.tokens * self.shape.topk

        def gather(t):
            parts = [torch.empty_like(t) for _ in range(self.world)]
            dist.all_gather(parts, t.contiguous())
            return [p.cpu() for p in parts]

        xs = gather(x)
        sorted_ids = gather(self.home.sorted_route_ids[:n])
        offsets = gather(self.home.group_offsets)
        return _ReceivedRows(xs, sorted_ids, offsets, self.rank, self.cap, self.shape.topk)

    def forward(self, x: torch.Tensor, logits: torch.Tensor, stage_timer=None) -> torch.Tensor:
        lib = ext.load()
        shp, home, world, rank = self.shape, self.home, self.world, self.rank
        stream = torch.cuda.current_stream(self.dev).cuda_stream
        mark = stage_timer if stage_timer is not None else (lambda _name: None)
        mark("begin")
        self.last_x = x
        self.route(logits)
        mark("route")
        if self.replicas is not None:
            ext.check(lib.b200moe_ep_place_routes(
                self.topk_ids.data_ptr(), self.topk_ids.numel(), shp.experts, self.pattern_rank.data_ptr(),
                self.pattern_local.data_ptr(), self.dest_rank.data_ptr(), self.dest_local.data_ptr(), stream),
                "ep_place_routes")
            home.sort(self.dest_rank, None)
        else:
            home.sort(self.topk_ids, self.rank_of_expert)
        mark("home_sort")
        d = ext.EpDispatchArgs(
            x.data_ptr(), self.topk_ids.data_ptr(), ext.peer_array(self.rows_ptrs),
            ext.peer_array(self.ids_ptrs), ext.peer_array(self.flag1_ptrs), self.done_counter.data_ptr(),
            self.epoch_dev.data_ptr(), home.scratch.data_ptr(), C.pointer(home.layout), x.stride(0), x.shape[0], shp.topk, world, rank,
            shp.hidden, self.e_local, self.cap, 0, ext.EP_PAYLOADS[self.payload],
            0 if self.recv_sf is None else int(self.recv_sf.shape[1]), int(self.a1_gscale_all.numel()), 0,
            ext.peer_array(self.sf_ptrs), self.a1_gscale_all.data_ptr(), self.home_status.data_ptr(),
            None if self.replicas is None else self.dest_local.data_ptr())
        ext.check(lib.b200moe_ep_dispatch(C.byref(d), stream), "ep_dispatch")
        mark("dispatch")
        ep = self.epoch_dev.data_ptr()
        fold = self.fold_waits
        # folded: the expert-side sort waits for all peers' dispatch flags before it reads the ids
        b = fused_moe.bind(self.plan, scratch=self.scratch, a=self.recv_rows, experts=self.experts,
                           topk_weights=self.ones, topk_ids=self.recv_ids, skip_combine=True, a_packed=self.packed,
                           sort_wait=(self.flags.data_ptr(), world, ep, self.home_status.data_ptr()) if fold else None)
        self.last_binding = b
        if not fold:
            ext.check(lib.b200moe_ep_wait(self.flags.data_ptr(), world, 0, ep, self.home_status.data_ptr(), 0,
                                          stream), "ep_wait")
            mark("wait_tokens")
        fused_moe.run(binding=b, stage_timer=(lambda n: None if n == "begin" else mark(n)) if stage_timer else None)
        # "my FC2 rows are complete" + "wait for everybody's": folded into the combine launch, or
        # two launches of their own
        flags2 = self.flags.data_ptr() + 4 * ext.MAX_RANKS
        if not fold:
            ext.check(lib.b200moe_ep_signal(self._flag2_arr, world, rank, 0, ep, stream), "ep_signal")
            ext.check(lib.b200moe_ep_wait(flags2, world, 0, ep, self.home_status.data_ptr(), 0, stream), "ep_wait")
            mark("wait_results")
        c = ext.EpCombineArgs(
            self.topk_weights.data_ptr(), self.out.data_ptr(), ext.peer_array(self.scratch_ptrs),
            home.scratch.data_ptr(), C.pointer(home.layout), self._inv_perm_off, self._routed_off,
            self.out.stride(0), x.shape[0], shp.topk, world, rank, shp.hidden, self.cap, 1.0, 0,
            ext.peer_array(self.flag2_ptrs), flags2 if fold else None, ep if fold else None,
            self.home_status.data_ptr())
        ext.check(lib.b200moe_ep_combine(C.byref(c), stream), "ep_combine")
        mark("combine")
        return self.out

    @property
    def can_capture(self) -> bool:
        return True     # nothing in the step depends on a host value that changes between steps

    def work_stats(self) -> dict:
        counts = self.last_binding.expert_counts.cpu()
        active = int((counts > 0).sum())
        rows = int(counts.sum())
        local = replace(self.shape, experts=self.n_local)
        return {"dominant": self._dominant(local, active, rows), "active_experts": active, "rows": rows}
