"""Expert-parallel host logic on CPU: two gloo ranks run the dispatch / return algebra of
``b12x_b200.moe.distributed.ExpertParallelMoE`` with the oracle standing in for the kernels, and
must reproduce the single-process oracle bit for bit."""

import os
import socket

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


def _a2a(out_rows, in_rows, recv_counts, send_counts):
    """all_to_all_single with split sizes (rows viewed as bytes: gloo has no bf16)."""
    o = out_rows.view(torch.uint8).reshape(out_rows.shape[0], -1) if out_rows.ndim > 1 else out_rows
    i = in_rows.view(torch.uint8).reshape(in_rows.shape[0], -1) if in_rows.ndim > 1 else in_rows
    dist.all_to_all_single(o, i, recv_counts, send_counts)


def _worker(rank: int, world: int, port: int, tokens_per_rank: int, ret: dict):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        shp = synth.shape("c1", name="ep", tokens=tokens_per_rank * world, hidden=256, intermediate=128,
                          experts=8, topk=3)
        full = synth.make_inputs(shp, seed=21)      # every rank builds the same global problem
        e_local = shp.experts // world
        lo = rank * tokens_per_rank
        x = full.x[lo:lo + tokens_per_rank]
        _, ids, w = O.route_topk(full.router_logits[lo:lo + tokens_per_rank], shp.topk)
        # home side: stable sort of the routes by destination rank
        rank_of_expert = (torch.arange(shp.experts) // e_local).to(torch.int32)
        home = O.expert_sort(ids, world, rank_of_expert)
        send_counts = home.expert_counts.clone()
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts)
        sc, rc = send_counts.tolist(), recv_counts.tolist()
        route = home.sorted_route_ids.long()
        send_rows = x[route // shp.topk].contiguous()
        send_ids = (ids.reshape(-1)[route] % e_local).to(torch.int32)
        recv_rows = torch.empty((sum(rc), shp.hidden), dtype=torch.bfloat16)
        recv_ids = torch.empty((sum(rc),), dtype=torch.int32)
        _a2a(recv_rows, send_rows, rc, sc)
        _a2a(recv_ids, send_ids, rc, sc)
        # expert side: the local layer on the received rows, top-1, weight 1, fp32 rows back
        sl = slice(rank * e_local, (rank + 1) * e_local)
        taps = O.MoETaps()
        a1 = full.w1_global_scale / full.a1_gscale
        a2 = full.w2_global_scale / full.a2_gscale
        O.moe_nvfp4(recv_rows, full.w1_fp4[sl], full.w1_blockscale[sl], a1[sl], full.w2_fp4[sl],
                    full.w2_blockscale[sl], a2[sl], full.a1_gscale[sl], full.a2_gscale[sl],
                    recv_ids.reshape(-1, 1), torch.ones(sum(rc), 1), taps=taps)
        back = taps.out_f32
        returned = torch.empty((sum(sc), shp.hidden), dtype=torch.float32)
        _a2a(returned, back, sc, rc)
        out = O.combine(returned, home.inv_perm, w, tokens_per_rank, shp.topk, shp.hidden)
        # single-process answer for this rank's tokens
        ref_taps = O.MoETaps()
        O.moe_nvfp4(x, full.w1_fp4, full.w1_blockscale, a1, full.w2_fp4, full.w2_blockscale, a2,
                    full.a1_gscale, full.a2_gscale, ids, w, taps=ref_taps)
        ret[rank] = bool(torch.equal(out, ref_taps.out_f32)) and sum(sc) == ids.numel()
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_ep_dispatch_return_algebra_two_gloo_ranks():
    world = 2
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, 12, ret), nprocs=world, join=True)
        assert dict(ret) == {0: True, 1: True}
