"""-m gpu: the benchmark configurations at their own shapes (hidden / intermediate / expert count /
top-k / router / recipe as named; token counts reduced where the CPU oracle would take minutes).

The oracle cannot evaluate a whole full-size layer in reasonable time, so every case checks
(``tests/gpu_utils.sampled_parity``): routing ids bit-exact against the oracle router, the WHOLE
permutation bit-exact, and -- for 48 routes of each of four experts -- activation codes bit-exact
and the fp32 FC2 rows within 1e-2 x RMS; then the weighted combine of the first tokens is
recomputed from the kernels' own FC2 rows and must be bit-equal to the bf16 output."""

from dataclasses import replace

import pytest
import torch

from b12x_b200 import synth
from b12x_b200.moe.distributed import ExpertParallelMoE
from oracle import moe_oracle as O
from tests.gpu_utils import combine_matches, sampled_parity

pytestmark = pytest.mark.gpu


def _run_and_check(shp, *, seed=5, rows_per_expert=48):
    dev = torch.device("cuda")
    inp = synth.make_inputs(shp, seed=seed, device=dev)
    from b12x_b200.moe.distributed import prepare_experts
    layer = ExpertParallelMoE(shp, inp, prepare_experts(inp, dev), dev)
    out = None
    for _ in range(2):       # twice: the scratch arena is reused as it is left
        out = layer.forward(inp.x, inp.router_logits)
    torch.cuda.synchronize()
    layer.check_status()
    # router: bit-exact ids, weights to fp32 round-off
    mode = {"mode": "sigmoid", "route_scale": shp.route_scale} if shp.router == "sigmoid" else {}
    _, ids, w = O.route_topk(inp.router_logits.cpu(), shp.topk, **mode)
    assert torch.equal(layer.topk_ids.cpu(), ids)
    torch.testing.assert_close(layer.topk_weights.cpu(), w, rtol=2e-6, atol=1e-7)
    res = sampled_parity(layer.last_binding, inp, rows_per_expert=rows_per_expert)
    assert res["permutation_ok"], res
    assert res["codes_ok"], res
    assert res["ok"], res
    assert res["rows"] > 0
    assert combine_matches(layer.last_binding, layer.topk_weights, out)
    return res


@pytest.mark.parametrize("tokens", [1, 8, 32, 64])
def test_c2_dsv3_decode_nvfp4_full_shape(tokens):
    """hidden 7168, intermediate 2048, 256 experts, top-8, sigmoid router x 2.5 (64-row expert tiles)."""
    shp = synth.shape("c2", tokens=tokens)
    res = _run_and_check(shp, seed=10 + tokens)
    assert res["permutation_rows"] == tokens * 8


def test_c3_qwen3_w4a16_full_shape():
    """hidden 4096, intermediate 1536, 128 experts, top-8, W4A16; 512 tokens."""
    _run_and_check(synth.shape("c3", tokens=512), seed=21)


@pytest.mark.parametrize("shard", [768, 384, 192])
def test_c3_tensor_parallel_shard_shapes(shard):
    """One rank's share of the Qwen3 shape under 2- / 4- / 8-way tensor parallelism: the
    intermediate dimension is 768 / 384 / 192 (192 = one and a half 128-column tiles)."""
    _run_and_check(replace(synth.shape("c3", tokens=256), intermediate=shard), seed=22 + shard)


def test_c4_mixtral_skewed_nvfp4_full_shape():
    """hidden 4096, intermediate 14336, 8 experts, top-2, Zipf(1.2) routing; 1024 tokens: the hot
    expert holds several row tiles, the cold ones a fraction of one (CTA-pair kernels)."""
    shp = synth.shape("c4", tokens=1024)
    res = _run_and_check(shp, seed=23)
    assert res["permutation_rows"] == 2048


def test_c4_single_cta_kernels_same_shape(monkeypatch):
    """The same shape with too few rows per expert for the CTA-pair kernels (wide single-CTA kernels)."""
    _run_and_check(synth.shape("c4", tokens=768), seed=24)


def test_c5_gptoss_w4a8_mx_full_shape():
    """hidden = intermediate = 2880 (22 k-blocks of 128 and a 64-wide tail), 128 experts, top-4,
    SwiGLU-OAI x MXFP8/MXFP4; 512 tokens."""
    _run_and_check(synth.shape("c5", tokens=512), seed=25)


def test_c5_large_batch_several_tiles_per_expert():
    """The same layer with 4096 tokens: 128 rows per expert on average, partial and full tiles."""
    _run_and_check(synth.shape("c5", tokens=4096), seed=26, rows_per_expert=32)


def test_pipelined_host_step_equals_the_whole_batch_step():
    """``forward_host`` on a large batch copies and computes in token chunks on three streams; the
    result must be the same bytes as one whole-batch step on device-resident inputs."""
    from b12x_b200.moe.distributed import prepare_experts
    dev = torch.device("cuda")
    shp = synth.shape("c4", tokens=4096)
    inp = synth.make_inputs(shp, seed=31, device=dev)
    layer = ExpertParallelMoE(shp, inp, prepare_experts(inp, dev), dev)
    assert layer.host_chunks() == 4
    whole = layer.forward(inp.x, inp.router_logits).clone()
    ids = layer.topk_ids.clone()
    torch.cuda.synchronize()
    x_host = inp.x.cpu().pin_memory()
    lg_host = inp.router_logits.cpu().pin_memory()
    out_host = torch.zeros((shp.tokens, shp.hidden), dtype=torch.bfloat16).pin_memory()
    for _ in range(2):
        layer.forward_host(x_host, lg_host, out_host)
    layer.check_status()
    assert torch.equal(layer.topk_ids, ids)
    assert torch.equal(out_host, whole.cpu())
    # a decode-sized batch is not chunked
    small = synth.shape("c2", tokens=64)
    assert ExpertParallelMoE.host_chunks(type("L", (), {"world": 1, "shape": small})()) == 1


@pytest.mark.parametrize("key", ["c4", "c5", "c3"])
@pytest.mark.timeout(900)
def test_benchmark_configurations_at_full_size(key):
    """The large-batch configurations at the token counts the benchmark times (c4 8192, c5 16384,
    c3 4096 tokens): whole permutation bit-exact, sampled routes against the oracle, and the
    combine of the first tokens recomputed from the kernels' own FC2 rows bit-equal to the output."""
    shp = synth.shape(key)
    res = _run_and_check(shp, seed=40, rows_per_expert=24)
    assert res["permutation_rows"] == shp.tokens * shp.topk
