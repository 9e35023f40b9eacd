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
from .distributed import _LayerBase, prepare_experts
from .fused_moe.stages import StageArena


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


class PeerExpertParallelMoE(_LayerBase):
    kernels_per_step = 12

    def __init__(self, shp, inputs, experts, dev, rank: int, world: int):
        super().__init__(shp, inputs, experts, dev, rank, world)
        if world < 2 or world > ext.MAX_RANKS:
            raise ValueError(f"needs 2..{ext.MAX_RANKS} ranks")
        if shp.experts % world:
            raise ValueError("experts must divide evenly over the ranks")
        self.e_local = shp.experts // world
        t, k = shp.tokens, shp.topk
        self.cap = t * k
        slots = world * self.cap
        self.home = StageArena(t, k, world, shp.hidden, dev)
        self.rank_of_expert = (torch.arange(shp.experts, dtype=torch.int32, device=dev) // self.e_local).contiguous()
        # the two cross-rank waits of a step either ride inside the expert sort and the combine
        # kernel (9 launches per step) or are launches of their own (12)
        self.fold_waits = os.environ.get("B200MOE_FOLD_WAITS", "0") == "1"
        self.kernels_per_step = 9 if self.fold_waits else 12
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
        self.recv_rows, self.rows_ptrs, self._h1 = _symm_empty((slots, shp.hidden), torch.bfloat16, dev)
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
        self.home_status = self.home._view("status", 16, torch.int32)
        torch.cuda.synchronize(dev)
        dist.barrier()

    def check_status(self) -> None:
        super().check_status()
        st = self.home_status.cpu()
        if int(st[0]) != 0:
            raise RuntimeError(f"expert-parallel wait gave up (code {int(st[1])}: 16 + missing peer rank)")

    @classmethod
    def from_synthetic(cls, shp: synth.MoEShape, dev, rank: int, world: int):
        e_local = shp.experts // world
        inp = synth.make_inputs(shp, seed=1000 + rank, device=dev, experts=e_local)
        return cls(shp, inp, prepare_experts(inp, dev), dev, rank, world)

    @classmethod
    def from_global(cls, full: synth.MoEInputs, dev, rank: int, world: int, tokens_per_rank: int):
        shp = replace(full.shape, tokens=tokens_per_rank)
        e_local = shp.experts // world
        local = synth.slice_experts(full, rank * e_local, (rank + 1) * e_local)
        lo = rank * tokens_per_rank
        local = replace(local, shape=shp, x=full.x[lo:lo + tokens_per_rank].contiguous(),
                        router_logits=full.router_logits[lo:lo + tokens_per_rank].contiguous())
        return cls(shp, local, prepare_experts(local, dev), dev, rank, world)

    def forward(self, x: torch.Tensor, logits: torch.Tensor, stage_timer=None) -> torch.Tensor:
        lib = ext.load()
        shp, home, world, rank = self.shape, self.home, self.world, self.rank
        stream = torch.cuda.current_stream(self.dev).cuda_stream
        mark = stage_timer if stage_timer is not None else (lambda _name: None)
        mark("begin")
        self.route(logits)
        mark("route")
        home.sort(self.topk_ids, self.rank_of_expert)
        mark("home_sort")
        d = ext.EpDispatchArgs(
            x.data_ptr(), self.topk_ids.data_ptr(), ext.peer_array(self.rows_ptrs),
            ext.peer_array(self.ids_ptrs), ext.peer_array(self.flag1_ptrs), self.done_counter.data_ptr(),
            self.epoch_dev.data_ptr(), home.scratch.data_ptr(), C.pointer(home.layout), x.stride(0), x.shape[0], shp.topk, world, rank,
            shp.hidden, self.e_local, self.cap, 0)
        ext.check(lib.b200moe_ep_dispatch(C.byref(d), stream), "ep_dispatch")
        mark("dispatch")
        ep = self.epoch_dev.data_ptr()
        fold = self.fold_waits
        # folded: the expert-side sort waits for all peers' dispatch flags before it reads the ids
        b = fused_moe.bind(self.plan, scratch=self.scratch, a=self.recv_rows, experts=self.experts,
                           topk_weights=self.ones, topk_ids=self.recv_ids, skip_combine=True,
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
        local = replace(self.shape, experts=self.e_local)
        return {"dominant": self._dominant(local, active, rows), "active_experts": active, "rows": rows}
