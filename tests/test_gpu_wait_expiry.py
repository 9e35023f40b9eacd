"""-m gpu: a device-side wait that nobody answers runs out, reports it in the status block and
returns; the context stays usable.  (The failure is a flag that nothing sets -- no GPU fault.)"""

import time

import pytest
import torch

from b12x_b200._lib import ext

pytestmark = pytest.mark.gpu


def test_ep_wait_gives_up_and_names_the_missing_peer():
    lib = ext.load()
    dev = torch.device("cuda")
    flags = torch.zeros(ext.MAX_RANKS, dtype=torch.int32, device=dev)
    flags[0] = 1                                  # rank 0 arrived at step 1, rank 1 never does
    status = torch.zeros(16, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    t0 = time.perf_counter()
    ext.check(lib.b200moe_ep_wait(flags.data_ptr(), 2, 1, None, status.data_ptr(), 200, stream), "ep_wait")
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    st = status.cpu().tolist()
    assert st[0] == 1 and st[1] == 16 + 1, st     # code 16 + missing rank
    assert 0.15 < dt < 2.0, dt
    # the context is alive: a satisfied wait returns at once and leaves a clean status alone
    status.zero_()
    flags[1] = 1
    ext.check(lib.b200moe_ep_wait(flags.data_ptr(), 2, 1, None, status.data_ptr(), 200, stream), "ep_wait")
    torch.cuda.synchronize()
    assert status.cpu().tolist()[0] == 0
    with pytest.raises(ValueError):
        ext.check(lib.b200moe_ep_wait(flags.data_ptr(), 2, 1, None, status.data_ptr(), -5, stream), "ep_wait")


def test_sort_with_folded_wait_gives_up_names_the_peer_and_still_sorts():
    """The expert-side sort of the peer-memory expert parallelism first waits for every peer's
    dispatch flag.  With a flag nobody sets the wait runs out after its limit, the status words name
    the missing rank, and the sort itself still completes (its ids are whatever lies in the buffer)."""
    import ctypes as C

    from oracle import moe_oracle as O

    lib = ext.load()
    dev = torch.device("cuda")
    tokens, topk, experts = 96, 1, 4
    layout = ext.scratch_layout(tokens, topk, experts, 256, 128, "nvfp4", "silu")
    scratch = torch.zeros(int(layout.total_nbytes), dtype=torch.uint8, device=dev)
    ids = torch.randint(0, experts, (tokens, topk), dtype=torch.int32, device=dev)
    flags = torch.zeros(ext.MAX_RANKS, dtype=torch.int32, device=dev)
    flags[0] = 1                                  # rank 1 never flags step 1
    epoch = torch.ones(1, dtype=torch.int32, device=dev)
    status = torch.zeros(16, dtype=torch.int32, device=dev)
    args = ext.SortArgs(ids.data_ptr(), None, scratch.data_ptr(), C.pointer(layout), tokens, topk, experts, 0,
                        flags.data_ptr(), epoch.data_ptr(), status.data_ptr(), 2, 100)
    t0 = time.perf_counter()
    ext.check(lib.b200moe_expert_sort(C.byref(args), torch.cuda.current_stream(dev).cuda_stream), "expert_sort")
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    st = status.cpu().tolist()
    assert st[0] == 1 and st[1] == 16 + 1, st
    assert 0.08 < dt < 2.0, dt
    srt = O.expert_sort(ids.cpu(), experts)
    off = int(layout.sorted_route_ids)
    got = scratch[off: off + tokens * 4].view(torch.int32).cpu()
    assert torch.equal(got, srt.sorted_route_ids)
