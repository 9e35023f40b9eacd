"""-m gpu, needs >= 2 GPUs: expert parallelism with this library's own dispatch / combine kernels
over NVLink peer memory, against the single-process CPU oracle, several steps in a row, at 2, 4
and 8 ranks, with the cross-rank waits folded into the sort and the combine kernel (the default)
and as launches of their own (B200MOE_FOLD_WAITS=0); rows cross the link quantised (NVFP4 / MXFP8)
or as bf16; the receive regions at worst-case size or sized by a capacity factor whose overflow is
a status word.  Peer memory is only touched with plain loads / stores."""

import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from b12x_b200 import synth
from tests.test_gpu_multi import _free_port

pytestmark = pytest.mark.gpu


def _worker(rank: int, world: int, port: int, fold: str, ret: dict, recipe: str = "nvfp4", payload: str | None = None,
            replica_slots: int = 0):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      B200MOE_FOLD_WAITS=fold, NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    from b12x_b200.moe.distributed import init_process_group
    from b12x_b200.moe.ep_peer import PeerExpertParallelMoE
    from oracle import moe_oracle as O
    from tests.gpu_utils import oracle_call
    init_process_group(dev)
    try:
        tpr = 40
        if recipe == "nvfp4":
            shp = synth.shape("c1", name="ep", tokens=tpr * world, hidden=512, intermediate=256, experts=8, topk=3,
                              zipf_s=1.2 if replica_slots else 0.0)
        else:   # 18 scale bytes per row: the last scale word of a row is half padding
            shp = synth.shape("c5", name="ep_mx", tokens=tpr * world, hidden=576, intermediate=320, experts=8, topk=3)
        full = synth.make_inputs(shp, seed=41)
        layer = PeerExpertParallelMoE.from_global(full, dev, rank, world, tpr, payload=payload,
                                                  replica_slots=replica_slots)
        ok = True
        if replica_slots:
            # the skewed calibration batch must have put copies of hot experts on other ranks, and the
            # planned loads must be flatter than the owners' loads
            plan = layer.replicas
            ok = any(len(x) > 0 for x in plan.extra) and layer.n_local == shp.experts // world + replica_slots
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
            ref = oracle_call(shp, x, full.w1_fp4, full.w1_blockscale, full.w1_global_scale, full.w2_fp4,
                              full.w2_blockscale, full.w2_global_scale, full.a1_gscale, full.a2_gscale, ids, w).float()
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


def _capacity_worker(rank: int, world: int, port: int, ret: dict):
    """A receive region sized by a capacity factor: a balanced step fits and matches the
    worst-case-sized layer bit for bit; a step that sends one rank more than the region holds ends
    with an error status on the sender (rows beyond the region are not sent, nothing hangs)."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    from b12x_b200.moe.distributed import init_process_group
    from b12x_b200.moe.ep_peer import PeerExpertParallelMoE
    init_process_group(dev)
    try:
        tpr = 64
        shp = synth.shape("c1", name="ep", tokens=tpr * world, hidden=512, intermediate=256, experts=8, topk=2)
        full = synth.make_inputs(shp, seed=43)
        wide = PeerExpertParallelMoE.from_global(full, dev, rank, world, tpr)
        tight = PeerExpertParallelMoE.from_global(full, dev, rank, world, tpr, recv_capacity_factor=1.5)
        lo = rank * tpr
        x = full.x[lo:lo + tpr].to(dev)
        lg = full.router_logits[lo:lo + tpr].to(dev)
        a = wide.forward(x, lg).clone()
        b = tight.forward(x, lg).clone()
        torch.cuda.synchronize()
        wide.check_status()
        tight.check_status()
        ok = tight.cap < wide.cap and torch.equal(a, b)
        # every route to the experts of rank 0: rank 0's region overflows on every sender
        lg2 = torch.full_like(lg, -50.0)
        lg2[:, : shp.experts // world] = torch.randn(tpr, shp.experts // world, device=dev)
        tight.forward(x, lg2)
        torch.cuda.synchronize()
        try:
            tight.check_status()
            ok = False
        except RuntimeError as e:
            ok = ok and "rank 0 was sent more rows than its receive capacity" in str(e)
        # the status words are sticky: a later good step does not hide the failed one
        tight.forward(x, lg)
        torch.cuda.synchronize()
        try:
            tight.check_status()
            ok = False
        except RuntimeError:
            pass
        dist.barrier()
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


@pytest.mark.parametrize("recipe,payload", [("w4a8_mx", None), ("nvfp4", "bf16"), ("w4a8_mx", "bf16")])
@pytest.mark.timeout(900)
def test_peer_dispatch_payloads(recipe, payload):
    """MXFP8 payload (K + K/32 bytes per route) and the bf16 payload for both block-scaled recipes;
    the default NVFP4 payload is what the test above runs."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(2, _free_port(), "1", ret, recipe, payload), nprocs=2, join=True)
        assert dict(ret) == {0: True, 1: True}


@pytest.mark.timeout(900)
def test_receive_capacity_factor_and_overflow_status():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_capacity_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
        assert dict(ret) == {0: True, 1: True}


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.timeout(900)
def test_replicated_hot_experts_do_not_change_the_result(world):
    """Spare expert slots filled from a Zipf-skewed calibration batch: routes of the hot experts are
    spread over their holders, and the output still equals the single-process oracle (every holder
    computes the same bytes for a route)."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), "1", ret, "nvfp4", None, 1), nprocs=world, join=True)
        assert dict(ret) == {r: True for r in range(world)}
