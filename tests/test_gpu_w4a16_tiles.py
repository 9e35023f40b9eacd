"""-m gpu: W4A16 layers with several 128-row tiles per expert against the CPU oracle.  In-process the
kernel family follows the plan (CTA pairs once it averages two row tiles per expert); the two child
runs repeat this file and the other W4A16 cases with the CTA-pair kernels forced on
(B200MOE_W4A16_PAIR=1: every shape, also experts with one or an odd number of row tiles -- once with
the left-over row tile on a single-CTA launch, B200MOE_TAIL_SPLIT=1, once as half of a pair, =0) and
off (=0: the single-CTA kernel).  The switch is read once per process."""

import os
import subprocess
import sys
from pathlib import Path

import pytest

from b12x_b200 import synth
from tests.gpu_utils import run_layer
from tests.test_gpu_parity import _check_w4a16_layer, _w16

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tokens,experts,topk,hidden,inter,act", [
    (700, 4, 2, 512, 256, "silu"),          # 2-3 row tiles per expert, 4 feature tiles, one code box
    (300, 2, 2, 640, 384, "silu"),          # 6 k-blocks in FC2: a full and a half box of codes
    (260, 1, 1, 320, 192, "silu"),          # 320 output features: the last feature tile is half empty
    (150, 2, 1, 256, 448, "relu2"),         # 7 k-blocks
])
def test_w4a16_multi_tile_matches_oracle(tokens, experts, topk, hidden, inter, act):
    shp = _w16(tokens=tokens, experts=experts, topk=topk, hidden=hidden, intermediate=inter, activation=act)
    _check_w4a16_layer(run_layer(synth.make_inputs(shp, seed=tokens + inter), want_fc1=True))


@pytest.mark.parametrize("tokens,experts,topk,hidden,inter,act", [
    (1100, 4, 2, 512, 256, "silu"),         # 4-5 row tiles per expert: full pairs and a half-empty one
    (640, 1, 1, 256, 192, "silu"),          # exactly five row tiles, one and a half feature tiles
])
def test_w4a16_many_row_tiles_matches_oracle(tokens, experts, topk, hidden, inter, act):
    shp = _w16(tokens=tokens, experts=experts, topk=topk, hidden=hidden, intermediate=inter, activation=act)
    _check_w4a16_layer(run_layer(synth.make_inputs(shp, seed=tokens + inter), want_fc1=True))


@pytest.mark.parametrize("pair,split", [("1", "1"), ("1", "0"), ("0", "1")])
@pytest.mark.timeout(900)
def test_both_kernel_families_pass_the_w4a16_cases(pair, split):
    if os.environ.get("B200MOE_W4A16_CHILD") == "1":
        pytest.skip("already the child run")
    here = Path(__file__).resolve().parent
    env = dict(os.environ, B200MOE_W4A16_PAIR=pair, B200MOE_TAIL_SPLIT=split, B200MOE_W4A16_CHILD="1")
    r = subprocess.run([sys.executable, "-m", "pytest", str(Path(__file__).resolve()),
                        str(here / "test_gpu_parity.py"), str(here / "test_w4a16_sources.py"),
                        "-m", "gpu", "-k", "w4a16", "-x", "-q", "-p", "no:cacheprovider"],
                       env=env, capture_output=True, text=True, timeout=850, cwd=str(here.parent))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
