"""-m gpu, needs >= 2 GPUs: expert parallelism with this library's own dispatch / combine kernels
over NVLink peer memory, against the single-process CPU oracle, several steps in a row, at 2, 4
and 8 ranks, with the cross-rank waits as launches of their own and folded into the sort and the
combine kernel (B200MOE_FOLD_WAITS=1).  Peer memory is only touched with plain loads / stores."""

import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from b12x_b200 import synth
from tests.test_gpu_multi import _free_port

pytestmark = pytest.mark.gpu


def _worker(rank: int, world: int, port: int, fold: str, ret: dict):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      B200MOE_FOLD_WAITS=fold, NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    from b12x_b200.moe.distributed import init_process_group
    from b12x_b200.moe.ep_peer import PeerExpertParallelMoE
    from oracle import moe_oracle as O
    init_process_group(dev)
    try:
        tpr = 40
        shp = synth.shape("c1", name="ep", tokens=tpr * world, hidden=512, intermediate=256, experts=8, topk=3)
        full = synth.make_inputs(shp, seed=41)
        layer = PeerExpertParallelMoE.from_global(full, dev, rank, world, tpr)
        ok = True
        for step in range(3):                 # new tokens every step: slots and flags are reused
            g = torch.Generator().manual_seed(100 + step)
            xs = torch.randn(tpr * world, shp.hidden, generator=g).to(torch.bfloat16)
            lgs = torch.randn(tpr * world, shp.experts, generator=g)
            lo = rank * tpr
            x, lg = xs[lo:lo + tpr], lgs[lo:lo + tpr]
            out = layer.forward(x.to(dev), lg.to(dev)).float().cpu()
            torch.cuda.synchronize()
            layer.check_status()
            _, ids, w = O.route_topk(lg, shp.topk)
            a1 = full.w1_global_scale / full.a1_gscale
            a2 = full.w2_global_scale / full.a2_gscale
            ref = O.moe_nvfp4(x, full.w1_fp4, full.w1_blockscale, a1, full.w2_fp4, full.w2_blockscale, a2,
                              full.a1_gscale, full.a2_gscale, ids, w).float()
            # fp32 rows combined in slot order, as on one GPU: the only differences to the CPU oracle
            # are single bf16 roundings (device exp() vs host exp() in the activation)
            same = (out - ref).abs().max().item() <= 2.0 ** -8 * ref.abs().max().item()
            if not same:
                print(f"rank {rank} step {step}: max abs diff {(out - ref).abs().max().item():.4e}, "
                      f"ref max {ref.abs().max().item():.4e}, rows differing "
                      f"{int(((out - ref).abs().amax(dim=1) > 0).sum())}/{out.shape[0]}", flush=True)
            ok = ok and same
        # the same step replayed from a CUDA graph on new tokens: bit-identical to the eager pass
        graph = layer.capture()
        for step in range(2):
            g = torch.Generator().manual_seed(200 + step)
            xs = torch.randn(tpr * world, shp.hidden, generator=g).to(torch.bfloat16)
            lgs = torch.randn(tpr * world, shp.experts, generator=g)
            lo = rank * tpr
            layer.x_stage.copy_(xs[lo:lo + tpr])
            layer.lg_stage.copy_(lgs[lo:lo + tpr])
            graph.replay()
            torch.cuda.synchronize()
            replayed = layer.out.clone()
            layer.graph = None
            eager = layer.forward(layer.x_stage, layer.lg_stage).clone()
            torch.cuda.synchronize()
            layer.check_status()
            if not torch.equal(replayed, eager):
                print(f"rank {rank}: graph replay {step} differs from the eager pass", flush=True)
                ok = False
        ret[rank] = ok
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("fold", ["0", "1"])
@pytest.mark.timeout(900)
def test_peer_memory_expert_parallel_matches_oracle(fold, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), fold, ret), nprocs=world, join=True)
        assert dict(ret) == {r: True for r in range(world)}
