"""-m gpu, one GPU: the quantised expert-parallel dispatch against the bf16 one.

A single rank dispatches to itself (world = 1: the "peer" buffers are its own), once with bf16
rows and once with rows quantised by the sender (NVFP4 codes + E4M3 scale bytes, MXFP8 values +
E8M0 scale bytes).  The expert side then runs the layer on the bf16 rows (its own permute +
quantise stage) and on the quantised rows (``permute_packed``): activation codes, scale atoms and
fp32 FC2 rows must be bit-identical, i.e. sending 9K/16 or K + K/32 bytes per route instead of 2K
changes nothing downstream.  Also: a receive region smaller than the routes raises the status word
and sends nothing beyond the region."""

import ctypes as C

import pytest
import torch

from b12x_b200 import synth
from b12x_b200._lib import ext
from b12x_b200.moe import fused_moe
from b12x_b200.moe.fused_moe.stages import StageArena
from tests.gpu_utils import prepare_experts, route_on_gpu

pytestmark = pytest.mark.gpu


def _dispatch(home, x, ti, ex, payload, recv, recv_sf, recv_ids, cap, num_experts, status):
    dev = x.device
    flags = torch.zeros(ext.MAX_RANKS, dtype=torch.int32, device=dev)
    done = torch.zeros(1, dtype=torch.int32, device=dev)
    gs = ex.a1_gscale.reshape(-1).float().contiguous()
    args = ext.EpDispatchArgs(
        x.data_ptr(), ti.data_ptr(), ext.peer_array([recv.data_ptr()]), ext.peer_array([recv_ids.data_ptr()]),
        ext.peer_array([flags.data_ptr()]), done.data_ptr(), None, home.scratch.data_ptr(),
        C.pointer(home.layout), x.stride(0), x.shape[0], ti.shape[1], 1, 0, x.shape[1], num_experts, cap, 1,
        ext.EP_PAYLOADS[payload], 0 if recv_sf is None else int(recv_sf.shape[1]), int(gs.numel()), 0,
        ext.peer_array([0 if recv_sf is None else recv_sf.data_ptr()]), gs.data_ptr(), status.data_ptr())
    rc = ext.load().b200moe_ep_dispatch(C.byref(args), torch.cuda.current_stream(dev).cuda_stream)
    torch.cuda.synchronize()
    assert int(flags[0]) == 1 and int(done[0]) == 0
    return rc


def _setup(recipe):
    dev = torch.device("cuda")
    if recipe == "nvfp4":
        shp = synth.shape("c1", name="pay", tokens=70, hidden=448, intermediate=192, experts=4, topk=3)
    else:
        shp = synth.shape("c5", name="pay_mx", tokens=70, hidden=576, intermediate=320, experts=4, topk=3)
    inp = synth.make_inputs(shp, seed=77, device=dev)
    ex = prepare_experts(inp, dev)
    _, ti, _ = route_on_gpu(inp, dev)
    home = StageArena(shp.tokens, shp.topk, 1, shp.hidden, dev)
    home.sort(ti, torch.zeros(shp.experts, dtype=torch.int32, device=dev))     # every expert lives on rank 0
    return dev, shp, inp, ex, ti, home


@pytest.mark.parametrize("pad", [4, 16])       # scale rows padded to 16 bytes go out 16 bytes at a time
@pytest.mark.parametrize("recipe", ["nvfp4", "w4a8_mx"])
def test_quantised_dispatch_is_bit_identical_to_bf16_dispatch(recipe, pad):
    dev, shp, inp, ex, ti, home = _setup(recipe)
    payload = "nvfp4" if recipe == "nvfp4" else "mxfp8"
    cap = slots = shp.tokens * shp.topk
    row_bytes = shp.hidden // 2 if recipe == "nvfp4" else shp.hidden
    nsf = shp.hidden // (16 if recipe == "nvfp4" else 32)
    status = torch.zeros(16, dtype=torch.int32, device=dev)
    recv_rows = torch.zeros(slots, shp.hidden, dtype=torch.bfloat16, device=dev)
    recv_q = torch.full((slots, row_bytes), 0xFF, dtype=torch.uint8, device=dev)
    recv_sf = torch.full((slots, (nsf + pad - 1) // pad * pad), 0xFF, dtype=torch.uint8, device=dev)
    ids_a = torch.full((slots, 1), -7, dtype=torch.int32, device=dev)
    ids_b = torch.full((slots, 1), -7, dtype=torch.int32, device=dev)
    assert _dispatch(home, inp.x, ti, ex, "bf16", recv_rows, None, ids_a, cap, shp.experts, status) == ext.OK
    assert _dispatch(home, inp.x, ti, ex, payload, recv_q, recv_sf, ids_b, cap, shp.experts, status) == ext.OK
    assert torch.equal(ids_a, ids_b) and int(status[0]) == 0
    # slot j holds route sorted[j]: its local expert id and its row
    routes = home.sorted_route_ids[:slots].long()
    assert torch.equal(ids_a.reshape(-1), ti.reshape(-1)[routes])
    assert torch.equal(recv_rows, inp.x[routes // shp.topk])
    # padding bytes of a scale row are zero, not whatever the buffer held
    assert int(recv_sf[:, nsf:].max().item() if recv_sf.shape[1] > nsf else 0) == 0

    caps = fused_moe.Caps(max_tokens=slots, num_topk=1, device=dev, weight_plan=ex.plan, quant_mode=recipe)
    plan = fused_moe.plan(caps)
    spec = plan.scratch_specs()[0]
    ones = torch.ones(slots, 1, device=dev)
    runs = []
    for packed in (None, (recv_q, recv_sf)):
        scratch = torch.full(spec.shape, 0xEE, dtype=spec.dtype, device=dev)
        a = recv_rows if packed is None else torch.zeros(1, shp.hidden, dtype=torch.bfloat16, device=dev).expand(slots, -1)
        b = fused_moe.bind(plan, scratch=scratch, a=a, experts=ex, topk_weights=ones, topk_ids=ids_a,
                           skip_combine=True, a_packed=packed)
        fused_moe.run(binding=b)
        torch.cuda.synchronize()
        fused_moe.check_device_status(b)
        runs.append(b)
    p, q = runs
    assert torch.equal(p.packed_route_indices, q.packed_route_indices)
    assert torch.equal(p.packed_input[:slots], q.packed_input[:slots])
    assert torch.equal(p.packed_input_scale, q.packed_input_scale)
    assert torch.equal(p.route_output[:slots], q.route_output[:slots])
    assert p.route_output[:slots].abs().max().item() > 0


def test_receive_region_overflow_sets_status_and_sends_nothing_beyond_it():
    dev, shp, inp, ex, ti, home = _setup("nvfp4")
    rows = shp.tokens * shp.topk
    cap = rows - 50
    status = torch.zeros(16, dtype=torch.int32, device=dev)
    recv_q = torch.full((rows, shp.hidden // 2), 0xAB, dtype=torch.uint8, device=dev)
    recv_sf = torch.full((rows, shp.hidden // 16), 0xAB, dtype=torch.uint8, device=dev)
    ids = torch.full((rows, 1), -7, dtype=torch.int32, device=dev)
    assert _dispatch(home, inp.x, ti, ex, "nvfp4", recv_q, recv_sf, ids, cap, shp.experts, status) == ext.OK
    assert status[:2].tolist() == [1, 48]              # 48 + destination rank 0
    assert int((ids[:cap] >= 0).sum()) == cap and int((ids[cap:] != -7).sum()) == 0
    assert bool((recv_q[cap:] == 0xAB).all()) and bool((recv_sf[cap:] == 0xAB).all())
    # without a status word the same call is refused before anything launches
    flags = torch.zeros(ext.MAX_RANKS, dtype=torch.int32, device=dev)
    done = torch.zeros(1, dtype=torch.int32, device=dev)
    gs = ex.a1_gscale.reshape(-1).float().contiguous()
    a = ext.EpDispatchArgs(
        inp.x.data_ptr(), ti.data_ptr(), ext.peer_array([recv_q.data_ptr()]), ext.peer_array([ids.data_ptr()]),
        ext.peer_array([flags.data_ptr()]), done.data_ptr(), None, home.scratch.data_ptr(), C.pointer(home.layout),
        inp.x.stride(0), shp.tokens, shp.topk, 1, 0, shp.hidden, shp.experts, cap, 1, ext.EP_PAYLOADS["nvfp4"],
        int(recv_sf.shape[1]), int(gs.numel()), 0, ext.peer_array([recv_sf.data_ptr()]), gs.data_ptr(), None)
    assert ext.load().b200moe_ep_dispatch(C.byref(a), None) == ext.ECAPACITY
