"""-m gpu: shapes that leave partial tiles (K and I that are multiples of 64 but not of 128 / 256),
for the nvfp4 recipe."""

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
