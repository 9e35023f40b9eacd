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
