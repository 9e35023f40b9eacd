"""-m gpu: shapes that leave partial tiles (K and I that are multiples of 64 but not of 128 / 256),
for the nvfp4 recipe, and both tile widths of the grouped GEMM kernel."""

import os
import subprocess
import sys
from pathlib import Path

import pytest

from b12x_b200 import synth
from tests.gpu_utils import run_layer
from tests.test_gpu_parity import _check_nvfp4_layer

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


@pytest.mark.parametrize("tokens,hidden,inter,act", [
    (70, 320, 192, "silu"), (9, 448, 64, "swigluoai"), (130, 192, 320, "relu2"), (40, 576, 448, "silu")])
def test_nvfp4_partial_tiles(tokens, hidden, inter, act):
    shp = synth.shape("c1", name="tail", tokens=tokens, hidden=hidden, intermediate=inter, experts=4, topk=2,
                      activation=act)
    _check_nvfp4_layer(run_layer(synth.make_inputs(shp, seed=hidden + inter)))


def test_narrow_tile_variant_passes_the_parity_suite():
    """The 128-wide, double-buffered tile is selected with B200MOE_TILE_N=128 (read once per process)."""
    env = dict(os.environ, B200MOE_TILE_N="128")
    res = subprocess.run([sys.executable, "-m", "pytest", "-x", "-q", "-m", "gpu", "tests/test_gpu_parity.py",
                          "-k", "nvfp4 or mx or c1"], cwd=ROOT, env=env, capture_output=True, text=True)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
