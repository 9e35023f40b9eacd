"""-m gpu, needs >= 2 GPUs: expert-parallel and tensor-parallel layers as one process per GPU over
NCCL, against the single-process CPU oracle, at 2, 4 and 8 ranks (as many as the box has)."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from b12x_b200 import synth

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, mode: str, ret: dict):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    from b12x_b200.moe.distributed import ExpertParallelMoE, TensorParallelMoE, init_process_group
    from oracle import moe_oracle as O
    init_process_group(dev)
    try:
        tpr = 40
        if mode == "ep":
            shp = synth.shape("c1", name="ep", tokens=tpr * world, hidden=512, intermediate=256, experts=8, topk=3)
            full = synth.make_inputs(shp, seed=31)
            layer = ExpertParallelMoE.from_global(full, dev, rank, world, tpr)
            lo = rank * tpr
            x, lg = full.x[lo:lo + tpr], full.router_logits[lo:lo + tpr]
        else:
            shp = synth.shape("c1", name="tp", tokens=tpr, hidden=512, intermediate=256 * world, experts=4, topk=2)
            full = synth.make_inputs(shp, seed=32)
            layer = TensorParallelMoE.from_global(full, dev, rank, world)
            x, lg = full.x, full.router_logits
        out = None
        for _ in range(2):                     # twice: scratch and split tables are reused
            out = layer.forward(x.to(dev), lg.to(dev)).float().cpu()
        torch.cuda.synchronize()
        layer.check_status()
        _, ids, w = O.route_topk(lg, shp.topk)
        a1 = full.w1_global_scale / full.a1_gscale
        a2 = full.w2_global_scale / full.a2_gscale
        taps = O.MoETaps()
        ref = O.moe_nvfp4(x, full.w1_fp4, full.w1_blockscale, a1, full.w2_fp4, full.w2_blockscale, a2,
                          full.a1_gscale, full.a2_gscale, ids, w, taps=taps).float()
        rms = taps.out_f32.square().mean().sqrt().item()
        err = (out - ref).abs().max().item()
        # EP returns fp32 rows and combines in slot order: identical to one GPU up to the bf16 rounding.
        # TP sums per-shard partial products in a different order: fp32 round-off only.
        ret[rank] = err <= (2.0 ** -7) * ref.abs().max().item() and err <= 1e-2 * rms + 2.0 ** -8 * ref.abs().max().item()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("mode", ["ep", "tp"])
@pytest.mark.timeout(900)
def test_multi_rank_layer_matches_oracle(mode, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), mode, ret), nprocs=world, join=True)
        assert dict(ret) == {r: True for r in range(world)}
