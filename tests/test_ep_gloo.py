"""Expert-parallel host logic on CPU ranks (gloo, world size 2 and 3).

The product class ``b12x_b200.moe.distributed.ExpertParallelMoE`` runs unchanged -- its split
tables, receive capacity, collectives, plan agreement and liveness checks are the code under test --
with the device kernels replaced by CPU stand-ins built on the oracle (the reference tests its
planner the same way, with monkey-patched launchers: tests/moe/test_tp_moe_scratch_bindings.py:1017-1078).
Failures are injected on the host: a receive capacity that overflows, a rank built from another
plan, a rank that arrives late, a rank that leaves between steps, malformed split tables."""

import os
import socket
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from b12x_b200 import synth
from oracle import moe_oracle as O


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


# ---------------------------------------------------------------------------------------------
# CPU stand-ins for the kernels behind the layer
# ---------------------------------------------------------------------------------------------
def _install_fake_backend(monkey: list, layer_inputs: dict):
    """Replace the C-ABI launches the expert-parallel layer makes by oracle calls on CPU tensors."""
    from b12x_b200.moe import distributed as D
    from b12x_b200.moe import fused_moe
    from b12x_b200.moe.fused_moe.stages import StageArena

    def fake_sort(self, topk_ids, group_map=None):
        srt = O.expert_sort(topk_ids, self.num_groups, group_map)
        kept = srt.sorted_route_ids.numel()
        self.group_counts.copy_(srt.expert_counts)
        self.group_offsets.copy_(srt.expert_offsets)
        self.inv_perm[: srt.inv_perm.numel()].copy_(srt.inv_perm)
        self.sorted_route_ids[:kept].copy_(srt.sorted_route_ids)

    def fake_gather(self, x, topk_ids, out_rows, out_ids, local_modulus):
        kept = int(self.group_offsets[self.num_groups])
        route = self.sorted_route_ids[:kept].long()
        out_rows[:kept].copy_(x[route // self.num_topk])
        out_ids[:kept].copy_((topk_ids.reshape(-1)[route] % local_modulus).to(torch.int32))

    def fake_combine(self, topk_weights, out, *, output_scale=1.0):
        t = topk_weights.shape[0]
        res = O.combine(self.routed, self.inv_perm[: t * self.num_topk], topk_weights, t, self.num_topk, self.hidden)
        out.copy_(res.to(out.dtype))

    def fake_run(*, binding, stage_timer=None):
        inp = layer_inputs["inp"]
        taps = O.MoETaps()
        a1 = inp.w1_global_scale / inp.a1_gscale
        a2 = inp.w2_global_scale / inp.a2_gscale
        O.moe_nvfp4(binding.a, inp.w1_fp4, inp.w1_blockscale, a1, inp.w2_fp4, inp.w2_blockscale, a2,
                    inp.a1_gscale, inp.a2_gscale, binding.topk_ids, binding.topk_weights, taps=taps)
        binding.output_f32.copy_(taps.out_f32)
        return binding.output_f32

    def fake_route(self, logits):
        _, ids, w = O.route_topk(logits, self.shape.topk)
        self.topk_ids.copy_(ids)
        self.topk_weights.copy_(w)

    for obj, name, fn in ((StageArena, "sort", fake_sort), (StageArena, "gather_rows", fake_gather),
                          (StageArena, "combine", fake_combine), (fused_moe, "run", fake_run),
                          (D._LayerBase, "route", fake_route)):
        monkey.append((obj, name, getattr(obj, name)))
        setattr(obj, name, fn)


def _make_layer(rank, world, tokens_per_rank, *, topk=3, capacity=None, seed=21):
    from b12x_b200.moe.distributed import ExpertParallelMoE
    shp = synth.shape("c1", name="ep", tokens=tokens_per_rank * world, hidden=256, intermediate=128,
                      experts=2 * world if world == 3 else 8, topk=topk)
    full = synth.make_inputs(shp, seed=seed)      # every rank builds the same global problem
    from dataclasses import replace
    tshp = replace(shp, tokens=tokens_per_rank)
    e_local = shp.experts // world
    local = synth.slice_experts(full, rank * e_local, (rank + 1) * e_local)
    lo = rank * tokens_per_rank
    local = replace(local, shape=tshp, x=full.x[lo:lo + tokens_per_rank].contiguous(),
                    router_logits=full.router_logits[lo:lo + tokens_per_rank].contiguous())
    from b12x_b200.moe.distributed import prepare_experts
    holder = {"inp": local}
    patches: list = []
    _install_fake_backend(patches, holder)
    layer = ExpertParallelMoE(tshp, local, prepare_experts(local, torch.device("cpu")), torch.device("cpu"),
                              rank, world, recv_capacity_factor=capacity)
    return layer, full, shp


def _reference(full, shp, x, lg):
    _, ids, w = O.route_topk(lg, shp.topk)
    taps = O.MoETaps()
    a1 = full.w1_global_scale / full.a1_gscale
    a2 = full.w2_global_scale / full.a2_gscale
    O.moe_nvfp4(x, full.w1_fp4, full.w1_blockscale, a1, full.w2_fp4, full.w2_blockscale, a2,
                full.a1_gscale, full.a2_gscale, ids, w, taps=taps)
    return taps.out_f32.to(torch.bfloat16)


def _init(rank, world, port, timeout_s=None):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    from b12x_b200.moe.distributed import init_process_group
    init_process_group(torch.device("cpu"), timeout_s=timeout_s)


# ---------------------------------------------------------------------------------------------
# workers
# ---------------------------------------------------------------------------------------------
def _w_matches(rank, world, port, ret):
    _init(rank, world, port)
    try:
        layer, full, shp = _make_layer(rank, world, 12)
        ok = True
        for step in range(2):        # buffers and split tables are reused
            out = layer.forward(layer.inputs.x, layer.inputs.router_logits).clone()
            ok = ok and torch.equal(out, _reference(full, shp, layer.inputs.x, layer.inputs.router_logits))
        ret[rank] = ok
    finally:
        dist.destroy_process_group()


def _w_overflow(rank, world, port, ret):
    _init(rank, world, port)
    try:
        # capacity factor 0.25: a rank may receive at most a quarter of one rank's routes; with
        # 8 experts over 2 ranks either rank receives about half of all routes -> both overflow,
        # and even a rank that would not must raise with the others
        layer, _, _ = _make_layer(rank, world, 16, capacity=0.25)
        try:
            layer.forward(layer.inputs.x, layer.inputs.router_logits)
            ret[rank] = "no error"
        except RuntimeError as e:
            ret[rank] = "capacity" in str(e) and "no row was exchanged" in str(e)
        # the group is still usable: nobody is stuck inside a collective
        t = torch.ones(1)
        dist.all_reduce(t)
        ret[f"alive{rank}"] = int(t.item()) == world
    finally:
        dist.destroy_process_group()


def _w_one_sided_overflow(rank, world, port, ret):
    _init(rank, world, port)
    try:
        layer, _, shp = _make_layer(rank, world, 16, capacity=0.6)
        # every token of every rank goes to experts of rank 0 only: rank 0 overflows, rank 1 receives nothing
        lg = torch.full_like(layer.inputs.router_logits, -50.0)
        lg[:, : shp.experts // world] = torch.randn(lg.shape[0], shp.experts // world)
        try:
            layer.forward(layer.inputs.x, lg)
            ret[rank] = "no error"
        except RuntimeError as e:
            ret[rank] = "no row was exchanged" in str(e)
    finally:
        dist.destroy_process_group()


def _w_plan_mismatch(rank, world, port, ret):
    _init(rank, world, port)
    try:
        try:
            _make_layer(rank, world, 12, topk=3 if rank == 0 else 2)
            ret[rank] = "no error"
        except ValueError as e:
            ret[rank] = "planned the layer" in str(e)
    finally:
        dist.destroy_process_group()


def _w_late_rank(rank, world, port, ret):
    _init(rank, world, port, timeout_s=3.0)
    try:
        layer, _, _ = _make_layer(rank, world, 12)
        if rank == 1:
            time.sleep(9.0)           # never joins rank 0's step in time
            ret[rank] = True
            return
        t0 = time.monotonic()
        try:
            layer.forward(layer.inputs.x, layer.inputs.router_logits)
            ret[rank] = "no error"
        except RuntimeError:
            ret[rank] = time.monotonic() - t0 < 8.0      # ended by the timeout, not by the peer waking up
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def _w_rank_leaves(rank, world, port, ret):
    _init(rank, world, port)
    from b12x_b200.moe.distributed import PeerLiveness
    store = dist.distributed_c10d._get_default_store()
    try:
        layer, full, shp = _make_layer(rank, world, 12)
        layer.liveness = PeerLiveness(store, rank, world, timeout_s=1.5)
        out = layer.forward(layer.inputs.x, layer.inputs.router_logits)
        first_ok = torch.equal(out, _reference(full, shp, layer.inputs.x, layer.inputs.router_logits))
        if rank == 1:
            ret[rank] = first_ok        # leaves between steps, nothing of it in flight
            return
        t0 = time.monotonic()
        try:
            layer.forward(layer.inputs.x, layer.inputs.router_logits)
            ret[rank] = "no error"
        except RuntimeError as e:
            ret[rank] = first_ok and "rank 1 did not reach step 1" in str(e) and time.monotonic() - t0 < 4.0
    finally:
        if rank == 0:
            time.sleep(0.2)
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def _spawn(fn, world=2):
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(fn, args=(world, port, ret), nprocs=world, join=True)
        return dict(ret)


# ---------------------------------------------------------------------------------------------
# tests
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("world", [2, 3])
@pytest.mark.timeout(300)
def test_expert_parallel_forward_matches_single_process_oracle(world):
    assert _spawn(_w_matches, world) == {r: True for r in range(world)}


@pytest.mark.timeout(300)
def test_receive_overflow_raises_on_every_rank_before_the_exchange():
    assert _spawn(_w_overflow) == {0: True, 1: True, "alive0": True, "alive1": True}


@pytest.mark.timeout(300)
def test_overflow_on_one_rank_stops_the_other_too():
    assert _spawn(_w_one_sided_overflow) == {0: True, 1: True}


@pytest.mark.timeout(300)
def test_ranks_built_from_different_plans_refuse_to_start():
    assert _spawn(_w_plan_mismatch) == {0: True, 1: True}


@pytest.mark.timeout(300)
def test_late_rank_ends_the_collective_with_an_error_not_a_hang():
    assert _spawn(_w_late_rank) == {0: True, 1: True}


@pytest.mark.timeout(300)
def test_rank_that_left_between_steps_is_found_before_launch():
    assert _spawn(_w_rank_leaves) == {0: True, 1: True}


def test_split_table_validation():
    from b12x_b200.moe.distributed import validate_split_tables
    validate_split_tables([3, 4], [2, 5], 2, 7)
    with pytest.raises(ValueError, match="1 entries for 2 ranks"):
        validate_split_tables([7], [2, 5], 2, 7)              # truncated table
    with pytest.raises(ValueError, match="negative"):
        validate_split_tables([3, -1], [2, 5], 2, 7)
    with pytest.raises(ValueError, match="sums to 9"):
        validate_split_tables([4, 5], [2, 5], 2, 7)
