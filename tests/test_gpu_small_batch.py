"""-m gpu: the small-batch NVFP4 kernels (weights as the 128 tile rows, tokens as columns, experts cut
into 64-row tiles) against the CPU oracle, and against the wide-tile kernels on the same inputs."""

import pytest
import torch

from b12x_b200 import synth
from oracle import moe_oracle as O
from tests.gpu_utils import run_layer
from tests.test_gpu_parity import _check_nvfp4_layer, _tiny

pytestmark = pytest.mark.gpu


def _small(**kw):
    base = dict(hidden=512, intermediate=256, experts=8)
    base.update(kw)
    return _tiny(**base)


@pytest.mark.parametrize("tile_rows", [64, 128])
@pytest.mark.parametrize("tokens", [1, 8, 17, 33, 70, 300])
def test_token_counts_both_tile_heights(tokens, tile_rows):
    """1..300 tokens over 8 experts: tiles of 16, 32 and 64 token columns, several tiles per expert."""
    inp = synth.make_inputs(_small(tokens=tokens), seed=100 + tokens)
    run = run_layer(inp, tile_rows=tile_rows)
    assert int(run.binding.core_layout.tile_rows) == tile_rows
    _check_nvfp4_layer(run)


def test_small_and_wide_kernels_agree():
    """Same inputs through both kernel families: identical activation codes going in, FC1 taps and
    outputs equal up to fp32 summation order."""
    inp = synth.make_inputs(_small(tokens=48, hidden=1024, intermediate=512), seed=7)
    a = run_layer(inp, tile_rows=64)
    b = run_layer(inp, tile_rows=128)
    rows = 48 * 2
    assert torch.equal(a.binding.packed_input.cpu()[:rows], b.binding.packed_input.cpu()[:rows])
    scale = b.fc1[:rows].abs().max().item()
    assert (a.fc1[:rows] - b.fc1[:rows]).abs().max().item() <= 2e-5 * scale
    rms = b.out_f32.square().mean().sqrt().item()
    assert (a.out_f32 - b.out_f32).abs().max().item() <= 1e-2 * rms


def test_swigluoai_with_clamp():
    inp = synth.make_inputs(_small(tokens=20, activation="swigluoai"), seed=21)
    _check_nvfp4_layer(run_layer(inp, tile_rows=64))


def test_relu2_plan_falls_back_to_the_wide_fc1():
    """A non-gated FC1 has no small-batch kernel: FC1 runs on the wide kernel over the 64-row
    tiles, FC2 on the small-batch kernel."""
    inp = synth.make_inputs(_small(tokens=24, activation="relu2", intermediate=384), seed=22)
    _check_nvfp4_layer(run_layer(inp, tile_rows=64))


def test_all_routes_to_one_expert():
    shp = _small(tokens=150, experts=4, topk=1)
    inp = synth.make_inputs(shp, seed=23)
    ids = torch.full((150, 1), 1, dtype=torch.int32)
    w = torch.rand(150, 1) + 0.5
    _check_nvfp4_layer(run_layer(inp, topk_ids=ids, topk_weights=w, tile_rows=64))


def test_expert_map_and_dropped_routes():
    shp = _small(tokens=30, topk=3)
    inp = synth.make_inputs(shp, seed=24)
    local = synth.MoEInputs(shp, inp.x, inp.router_logits, None, inp.w1_fp4[4:], inp.w1_blockscale[4:],
                            inp.w1_global_scale[4:], inp.w2_fp4[4:], inp.w2_blockscale[4:],
                            inp.w2_global_scale[4:], inp.a1_gscale[4:], inp.a2_gscale[4:])
    emap = torch.tensor([-1, -1, -1, -1, 0, 1, 2, 3], dtype=torch.int32)
    _, ids, w = O.route_topk(inp.router_logits, 3)
    run = run_layer(local, topk_ids=ids, topk_weights=w, expert_map=emap, tile_rows=64)
    _check_nvfp4_layer(run, expert_map=emap)


def test_decode_shape_hidden_7168():
    """The headline decode shape at 8 experts: 28 k-blocks, 16 + 28 tiles per expert."""
    shp = synth.shape("c2", tokens=16, experts=8, topk=4, name="c2_e8")
    inp = synth.make_inputs(shp, seed=25)
    run = run_layer(inp, want_fc1=False)
    assert int(run.binding.core_layout.tile_rows) == 64
    _check_nvfp4_layer(run)


def test_output_rows_not_a_multiple_of_256():
    """hidden 640: the last FC2 tile has one full and one empty 128-row sub-tile."""
    inp = synth.make_inputs(_small(tokens=12, hidden=640, intermediate=384 - 128), seed=26)
    _check_nvfp4_layer(run_layer(inp, tile_rows=64))


def test_repeat_runs_bitwise_identical():
    inp = synth.make_inputs(_small(tokens=40), seed=27)
    a = run_layer(inp, poison=0x00, tile_rows=64)
    b = run_layer(inp, poison=0xFF, tile_rows=64)
    assert torch.equal(a.out, b.out) and torch.equal(a.out_f32, b.out_f32)
