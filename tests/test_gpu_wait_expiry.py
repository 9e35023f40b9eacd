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


def test_combine_with_folded_wait_gives_up_names_the_peer_and_still_combines():
    """The expert-parallel combine signals "my FC2 rows are complete", block 0 waits for every peer
    and every other block for the ranks that hold its token's rows.  Here all rows live on rank 0
    (this rank) and rank 1 never signals: the pull completes, block 0's wait for rank 1 runs out after
    its limit, and the status words name rank 1."""
    import ctypes as C

    from b12x_b200.moe.fused_moe.stages import StageArena

    lib = ext.load()
    dev = torch.device("cuda")
    tokens, topk, hidden, world = 8, 2, 64, 2
    cap = tokens * topk
    home = StageArena(tokens, topk, world, hidden, dev)
    ids = torch.randint(0, 4, (tokens, topk), dtype=torch.int32, device=dev)
    home.sort(ids, torch.zeros(4, dtype=torch.int32, device=dev))          # every expert lives on rank 0
    # a stand-in for rank 0's expert arena: slot -> sorted position (identity) and the fp32 FC2 rows
    arena = torch.zeros(4096 + cap * hidden * 4, dtype=torch.uint8, device=dev)
    arena[: world * cap * 4].view(torch.int32).copy_(torch.arange(world * cap, dtype=torch.int32, device=dev))
    rows = torch.randn(cap, hidden, device=dev)
    arena[4096:].view(torch.float32).view(cap, hidden).copy_(rows)
    flags = torch.zeros(ext.MAX_RANKS, dtype=torch.int32, device=dev)
    other = torch.zeros(ext.MAX_RANKS, dtype=torch.int32, device=dev)     # "rank 1's" flag block: it never answers
    epoch = torch.ones(1, dtype=torch.int32, device=dev)
    status = torch.zeros(16, dtype=torch.int32, device=dev)
    w = torch.rand(tokens, topk, device=dev)
    out = torch.zeros(tokens, hidden, dtype=torch.bfloat16, device=dev)
    args = ext.EpCombineArgs(
        w.data_ptr(), out.data_ptr(), ext.peer_array([arena.data_ptr(), arena.data_ptr()]), home.scratch.data_ptr(),
        C.pointer(home.layout), 0, 4096, out.stride(0), tokens, topk, world, 0, hidden, cap, 1.0, 200,
        ext.peer_array([flags.data_ptr(), other.data_ptr()]), flags.data_ptr(), epoch.data_ptr(), status.data_ptr())
    t0 = time.perf_counter()
    ext.check(lib.b200moe_ep_combine(C.byref(args), torch.cuda.current_stream(dev).cuda_stream), "ep_combine")
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert status[:2].tolist() == [1, 16 + 1]
    assert 0.15 < dt < 2.0, dt
    assert int(flags[0]) == 1 and int(other[0]) == 1                      # both ranks were told
    inv = home.inv_perm[: tokens * topk].long().reshape(tokens, topk)
    acc = torch.zeros(tokens, hidden, device=dev)
    for s in range(topk):
        acc = acc + w[:, s:s + 1] * rows[inv[:, s]]
    assert torch.equal(out, acc.to(torch.bfloat16))
