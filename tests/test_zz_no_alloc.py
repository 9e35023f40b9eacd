"""-m gpu: the sort entry point that brings its own scratch (``b200moe_expert_sort_static``).

Some callers cannot give the library a scratch arena: a server that reserved all device memory for
its own pool at start-up, or code that is in the middle of a graph capture.  For them the library
carries a small fixed array on each GPU.  This test calls that entry point straight through the C ABI
and requires the same permutation, bit for bit, as the regular arena-based entry point -- twice in a
row with different inputs, because the built-in array still holds the first call's tables when the
second call starts.  It lives in its own file, collected last."""

import ctypes as C

import pytest
import torch

from b12x_b200._lib import ext
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu


def _arena_sort(ids: torch.Tensor, num_experts: int, emap):
    tokens, topk = ids.shape
    layout = ext.scratch_layout(tokens, topk, num_experts, 64, 64, "w4a16", "silu")
    scratch = torch.full((int(layout.total_nbytes),), 0xFF, dtype=torch.uint8, device="cuda")
    args = ext.SortArgs(ids.data_ptr(), None if emap is None else emap.data_ptr(), scratch.data_ptr(),
                        C.pointer(layout), tokens, topk, num_experts, 0 if emap is None else emap.numel())
    stream = torch.cuda.current_stream().cuda_stream
    ext.check(ext.load().b200moe_expert_sort(C.byref(args), stream), "expert_sort")
    torch.cuda.synchronize()

    def view(name, count):
        off = int(getattr(layout, name))
        return scratch[off:off + 4 * count].view(torch.int32).clone()

    return view("expert_offsets", num_experts + 1), view("sorted_route_ids", tokens * topk), view("inv_perm", tokens * topk)


def _static_sort(ids: torch.Tensor, num_experts: int, emap):
    tokens, topk = ids.shape
    offs = torch.full((num_experts + 1,), -7, dtype=torch.int32, device="cuda")
    srt = torch.full((tokens * topk,), -7, dtype=torch.int32, device="cuda")
    inv = torch.full((tokens * topk,), -7, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    rc = ext.load().b200moe_expert_sort_static(
        ids.data_ptr(), None if emap is None else emap.data_ptr(), 0 if emap is None else emap.numel(),
        tokens, topk, num_experts, offs.data_ptr(), srt.data_ptr(), inv.data_ptr(), stream)
    assert rc == ext.OK, ext.strerror(rc)
    torch.cuda.synchronize()
    return offs, srt, inv


def test_static_sort_matches_arena_sort_on_two_calls_in_a_row():
    lib = ext.load()
    g = torch.Generator().manual_seed(2024)
    cases = [(300, 8, 256, None),
             (77, 4, 40, torch.tensor([(i % 3) - 1 + (i % 5) for i in range(64)], dtype=torch.int32).clamp(-1, 39))]
    for tokens, topk, experts, emap in cases:
        hi = experts if emap is None else emap.numel()
        ids = torch.randint(0, hi, (tokens, topk), generator=g, dtype=torch.int32).cuda()
        emap_d = None if emap is None else emap.cuda()
        ref = _arena_sort(ids, experts, emap_d)
        got = _static_sort(ids, experts, emap_d)
        kept = int(ref[0][-1])
        assert torch.equal(got[0], ref[0])
        assert torch.equal(got[1][:kept], ref[1][:kept])
        assert torch.equal(got[2], ref[2])
        # and against the CPU oracle's canonical sort, not only against the other CUDA entry point
        srt = O.expert_sort(ids.cpu(), experts, emap)
        assert torch.equal(got[0].cpu(), srt.expert_offsets)
        assert torch.equal(got[1][:kept].cpu(), srt.sorted_route_ids) and torch.equal(got[2].cpu(), srt.inv_perm)
    # beyond the fixed maximum: refused with the capacity status, nothing is launched
    dummy = torch.zeros(8, dtype=torch.int32, device="cuda")
    rc = lib.b200moe_expert_sort_static(dummy.data_ptr(), None, 0, 65537, 1, 8, dummy.data_ptr(),
                                        dummy.data_ptr(), dummy.data_ptr(), None)
    assert rc == ext.ECAPACITY
    rc = lib.b200moe_expert_sort_static(dummy.data_ptr(), None, 0, 4, 2, 1025, dummy.data_ptr(),
                                        dummy.data_ptr(), dummy.data_ptr(), None)
    assert rc == ext.ECAPACITY


@pytest.mark.parametrize("tokens,topk,experts,one_expert", [
    (8192, 8, 1024, False),      # both limits at once: 65 536 routes over 1 024 experts
    (65536, 1, 7, True),         # every route to the same expert: one count carries all 65 536
    (1, 1, 1, False),            # the smallest call
])
def test_static_sort_at_its_limits(tokens, topk, experts, one_expert):
    g = torch.Generator().manual_seed(tokens + experts)
    if one_expert:
        ids = torch.full((tokens, topk), 3, dtype=torch.int32)
    else:
        ids = torch.randint(0, experts, (tokens, topk), generator=g, dtype=torch.int32)
    srt = O.expert_sort(ids, experts, None)
    for _ in range(2):       # the built-in array is reused as the previous call left it
        offs, order, inv = _static_sort(ids.cuda(), experts, None)
        assert torch.equal(offs.cpu(), srt.expert_offsets)
        assert torch.equal(order.cpu(), srt.sorted_route_ids)
        assert torch.equal(inv.cpu(), srt.inv_perm)
