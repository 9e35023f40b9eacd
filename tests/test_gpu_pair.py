"""-m gpu: large NVFP4 batches (several 128-row tiles per expert, odd and even tile counts) against
the CPU oracle.  In-process the library picks the kernel itself (plans that average two or more row
tiles per expert run on the CTA-pair kernels, tcgen05 cta_group::2); `test_both_kernel_families...`
re-runs this file in child processes with B200MOE_PAIR=1 and =0, which forces every case onto the
CTA-pair and onto the single-CTA kernels; with the pair kernels once with the left-over row tile of
an odd-tiled expert on a single-CTA launch of its own (B200MOE_TAIL_SPLIT=1) and once as half of a
pair (=0)."""

import os
import subprocess
import sys

import pytest
import torch

from b12x_b200 import synth
from tests.gpu_utils import run_layer
from tests.test_gpu_parity import _check_mx_layer, _check_nvfp4_layer, _mx, _tiny

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tokens,experts,topk,hidden,inter,act", [
    (700, 4, 2, 512, 256, "silu"),          # 2-3 row tiles per expert, odd and even counts
    (1100, 2, 1, 512, 256, "silu"),         # ~4 tiles per expert
    (600, 2, 2, 640, 192, "silu"),          # K tail (640 = 2.5 k-blocks), half-empty last FC1 tile, FC2 tail
    (520, 2, 2, 256, 128, "swigluoai"),     # clamp + SwiGLU-OAI epilogue
])
def test_pair_kernels_match_oracle(tokens, experts, topk, hidden, inter, act):
    shp = _tiny(tokens=tokens, experts=experts, topk=topk, hidden=hidden, intermediate=inter, activation=act)
    assert tokens * topk >= 256 * experts      # at least two full row tiles per expert on average
    run = run_layer(synth.make_inputs(shp, seed=tokens + hidden), want_fc1=True)
    assert int(run.binding.core_layout.tile_rows) == 128
    _check_nvfp4_layer(run)


@pytest.mark.parametrize("tokens,experts,topk,hidden,inter,act", [
    (700, 4, 2, 512, 256, "silu"),          # 2-3 row tiles per expert
    (600, 2, 2, 320, 192, "swigluoai"),     # K tail (320 = 2.5 k-blocks of 128), half-empty last FC1 tile, FC2 tail
    (1100, 2, 1, 2880, 192, "swigluoai"),   # the GPT-OSS hidden size: 22 k-blocks and a 64-wide tail
])
def test_pair_kernels_w4a8_mx_match_oracle(tokens, experts, topk, hidden, inter, act):
    shp = _mx(tokens=tokens, experts=experts, topk=topk, hidden=hidden, intermediate=inter, activation=act)
    assert tokens * topk >= 256 * experts
    run = run_layer(synth.make_inputs(shp, seed=tokens + hidden), want_fc1=True)
    assert int(run.binding.core_layout.tile_rows) == 128
    _check_mx_layer(run)


def test_pair_single_expert_odd_tile_count():
    shp = _tiny(tokens=300, experts=1, topk=1, hidden=512, intermediate=256)
    inp = synth.make_inputs(shp, seed=31)
    ids = torch.zeros((300, 1), dtype=torch.int32)
    w = torch.rand(300, 1) + 0.5
    _check_nvfp4_layer(run_layer(inp, topk_ids=ids, topk_weights=w))


def test_pair_repeat_runs_bitwise_identical():
    inp = synth.make_inputs(_tiny(tokens=640, experts=2, topk=2, hidden=512, intermediate=256), seed=32)
    a = run_layer(inp, poison=0x00)
    b = run_layer(inp, poison=0xFF)
    assert torch.equal(a.out, b.out) and torch.equal(a.out_f32, b.out_f32)


@pytest.mark.timeout(900)
@pytest.mark.parametrize("forced,split", [("1", "1"), ("1", "0"), ("0", "1")])
def test_both_kernel_families_pass_these_cases(forced, split):
    if os.environ.get("B200MOE_PAIR") is not None:
        pytest.skip("already a child run")
    env = dict(os.environ, B200MOE_PAIR=forced, B200MOE_TAIL_SPLIT=split)
    r = subprocess.run([sys.executable, "-m", "pytest", __file__, "-m", "gpu", "-x", "-q", "-p", "no:cacheprovider"],
                       env=env, capture_output=True, text=True, timeout=800)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
