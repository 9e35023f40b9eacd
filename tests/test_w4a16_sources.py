"""W4A16 over the other two weight sources of the reference (``fp4_e8m0_k32`` and
``compressed_tensors``; b12x/moe/_shared/execution.py:160-183, w4a16/prepare.py:460-465,
1253-1325): the oracle against a fixture made by the reference's own evaluator, the load-time
host logic (CPU), and the CUDA path against the oracle (``-m gpu``)."""

import pytest
import torch

from b12x_b200 import synth
from b12x_b200.moe import fused_moe
from b12x_b200.moe._shared.execution import WeightPreparationTransform as T
from oracle import moe_oracle as O
from tests.helpers import load_golden, t

ACT_API = {"silu": "silu", "relu2": "relu2"}


def _cos(a, b):
    return torch.nn.functional.cosine_similarity(a.flatten().double(), b.flatten().double(), dim=0).item()


def _case(g, tag):
    names = ("x", "w1_fp4", "w1_e8m0", "w2_fp4", "w2_e8m0", "w1_global", "w2_global", "topk_ids",
             "topk_weights", "out_f32")
    d = {n: t(g[f"{tag}_{n}"]) for n in names}
    d["x"] = t(g[f"{tag}_x"], torch.bfloat16)
    return d


@pytest.mark.parametrize("act", ["silu", "relu2"])
def test_oracle_e8m0_source_matches_reference_evaluator(act):
    c = _case(load_golden("tiny_w4a16_e8m0.npz"), act)
    taps = O.MoETaps()
    O.moe_w4a16(c["x"], c["w1_fp4"], c["w1_e8m0"], c["w1_global"], c["w2_fp4"], c["w2_e8m0"],
                c["w2_global"], c["topk_ids"], c["topk_weights"], activation=act, taps=taps,
                scale_format="e8m0_k32")
    ref = c["out_f32"]
    # the reference evaluator keeps fp32 where the kernel (and this oracle) round the intermediate
    # to bf16: relative 2^-9 per element; its own acceptance bar is the cosine
    assert _cos(taps.out_f32, ref) >= (0.9975 if act == "silu" else 0.99)
    assert (taps.out_f32 - ref).abs().max().item() <= 5e-3 * ref.abs().max().item()


def _plan(source, act="silu", e=4, k=256, i=128, modes="w4a16"):
    return fused_moe.plan_weights(quant_modes=modes, source_format=source, activation=act,
                                  params_dtype=torch.bfloat16, num_experts=e, hidden_size=k,
                                  intermediate_size=i)


def test_plan_accepts_the_reference_sources_for_w4a16():
    assert T.EXPAND_E8M0_K32 in _plan("fp4_e8m0_k32").transforms
    assert T.INVERT_GLOBAL_SCALES in _plan("compressed_tensors").transforms
    assert not _plan("modelopt_nvfp4").transforms & {T.EXPAND_E8M0_K32, T.INVERT_GLOBAL_SCALES}
    with pytest.raises(ValueError):
        _plan("compressed_tensors", modes="nvfp4")          # execution.py:172-183: w4a16 only
    with pytest.raises(ValueError):
        _plan("fp4_e8m0_k32", modes=("w4a8_mx", "w4a16"))   # two scale layouts, one allocation


def test_compressed_tensors_inverts_the_global_scales():
    inp = synth.make_inputs(synth.shape("c3", name="ct", tokens=4, hidden=256, intermediate=128, experts=4,
                                        topk=2, activation="silu"), seed=5)
    kw = dict(params_dtype=torch.bfloat16, w1_fp4=inp.w1_fp4, w2_fp4=inp.w2_fp4,
              w1_blockscale=inp.w1_blockscale, w2_blockscale=inp.w2_blockscale)
    mo = fused_moe.prepare_weights(plan=_plan("modelopt_nvfp4"), w1_global_scale=inp.w1_global_scale,
                                   w2_global_scale=inp.w2_global_scale, **kw)
    ct = fused_moe.prepare_weights(plan=_plan("compressed_tensors"),
                                   w1_global_scale=torch.reciprocal(inp.w1_global_scale),
                                   w2_global_scale=torch.reciprocal(inp.w2_global_scale), **kw)
    assert torch.allclose(ct.w1_alphas, mo.w1_alphas, rtol=2e-7, atol=0)
    assert torch.allclose(ct.w2_alphas, mo.w2_alphas, rtol=2e-7, atol=0)
    assert torch.equal(ct.w1_blockscale, mo.w1_blockscale) and torch.equal(ct.w2_blockscale, mo.w2_blockscale)


def test_e8m0_source_scales_are_written_once_per_16():
    c = _case(load_golden("tiny_w4a16_e8m0.npz"), "silu")
    ex = fused_moe.prepare_weights(plan=_plan("fp4_e8m0_k32"), params_dtype=torch.bfloat16,
                                   w1_fp4=c["w1_fp4"], w2_fp4=c["w2_fp4"], w1_blockscale=c["w1_e8m0"],
                                   w2_blockscale=c["w2_e8m0"], w1_global_scale=c["w1_global"],
                                   w2_global_scale=c["w2_global"])
    for sw, grid, rows, cols in ((ex.w1_blockscale, c["w1_e8m0"], 256, 256), (ex.w2_blockscale, c["w2_e8m0"], 256, 128)):
        for e in range(4):
            plain = O.unswizzle_block_scale(sw[e], rows, cols // 16)
            assert torch.equal(plain[:, 0::2], grid[e]) and torch.equal(plain[:, 1::2], grid[e])
    assert torch.equal(ex.w1_alphas, c["w1_global"])
    with pytest.raises(ValueError):
        fused_moe.prepare_weights(plan=_plan("fp4_e8m0_k32"), params_dtype=torch.bfloat16,
                                  w1_fp4=c["w1_fp4"], w2_fp4=c["w2_fp4"], w1_blockscale=c["w1_e8m0"][:, :, :4],
                                  w2_blockscale=c["w2_e8m0"])


# ------------------------------------------------------------------------------------------------
def _run_gpu(plan, kw, x, ids, tw, tokens, topk, hidden, w1_rows):
    dev = torch.device("cuda")
    ex = fused_moe.prepare_weights(plan=plan, params_dtype=torch.bfloat16,
                                   **{n: v.to(dev) for n, v in kw.items()})
    p = fused_moe.plan(fused_moe.Caps(max_tokens=tokens, num_topk=topk, device=dev, weight_plan=plan,
                                      quant_mode="w4a16"))
    spec = p.scratch_specs()[0]
    scratch = torch.full(spec.shape, 0xFF, dtype=spec.dtype, device=dev)
    fc1 = torch.zeros(tokens * topk, w1_rows, device=dev)
    of32 = torch.zeros(tokens, hidden, device=dev)
    b = fused_moe.bind(p, scratch=scratch, a=x.to(dev), experts=ex, topk_weights=tw.to(dev),
                       topk_ids=ids.to(dev), fc1_tap=fc1, output_f32=of32)
    fused_moe.run(binding=b)
    torch.cuda.synchronize()
    fused_moe.check_device_status(b)
    return b, fc1.cpu(), of32.cpu()


@pytest.mark.gpu
@pytest.mark.parametrize("act", ["silu", "relu2"])
def test_gpu_e8m0_source_matches_golden_and_oracle(act):
    c = _case(load_golden("tiny_w4a16_e8m0.npz"), act)
    kw = dict(w1_fp4=c["w1_fp4"], w2_fp4=c["w2_fp4"], w1_blockscale=c["w1_e8m0"], w2_blockscale=c["w2_e8m0"],
              w1_global_scale=c["w1_global"], w2_global_scale=c["w2_global"])
    b, fc1, out = _run_gpu(_plan("fp4_e8m0_k32", act), kw, c["x"], c["topk_ids"], c["topk_weights"], 8, 2, 256,
                           c["w1_fp4"].shape[1])
    taps = O.MoETaps()
    O.moe_w4a16(c["x"], c["w1_fp4"], c["w1_e8m0"], c["w1_global"], c["w2_fp4"], c["w2_e8m0"], c["w2_global"],
                c["topk_ids"], c["topk_weights"], activation=act, taps=taps, scale_format="e8m0_k32")
    rows = taps.fc1.shape[0]
    assert (fc1[:rows] - taps.fc1).abs().max().item() <= 2e-5 * taps.fc1.abs().max().item()
    rms = taps.out_f32.square().mean().sqrt().item()
    assert (out - taps.out_f32).abs().max().item() <= 1e-2 * rms
    assert _cos(out, c["out_f32"]) >= (0.9975 if act == "silu" else 0.99)


@pytest.mark.gpu
@pytest.mark.parametrize("tokens,hidden,inter,act", [(40, 512, 384, "silu"), (130, 256, 256, "relu2"),
                                                     (33, 320, 192, "silu")])
def test_gpu_e8m0_source_layer(tokens, hidden, inter, act):
    shp = synth.shape("c5", name="w16e8", tokens=tokens, hidden=hidden, intermediate=inter, experts=6, topk=2,
                      activation=act)
    inp = synth.make_inputs(shp, seed=tokens)
    g = torch.Generator().manual_seed(tokens)
    ids = torch.stack([torch.randperm(6, generator=g)[:2] for _ in range(tokens)]).to(torch.int32)
    tw = torch.rand(tokens, 2, generator=g)
    g1, g2 = 0.5 + torch.rand(6, generator=g), 0.5 + torch.rand(6, generator=g)
    # widen the scale bytes past what E4M3 could hold (2^-20 .. 2^12), and one block at 0 (2^-127)
    s1 = inp.w1_blockscale.clone()
    s1[:, ::3, :] = s1[:, ::3, :] - 12
    s1[:, 1::5, 1] = s1[:, 1::5, 1] + 10
    s1[0, 0, 0] = 0
    kw = dict(w1_fp4=inp.w1_fp4, w2_fp4=inp.w2_fp4, w1_blockscale=s1, w2_blockscale=inp.w2_blockscale,
              w1_global_scale=g1, w2_global_scale=g2)
    b, fc1, out = _run_gpu(_plan("fp4_e8m0_k32", act, e=6, k=hidden, i=inter), kw, inp.x, ids, tw, tokens, 2,
                           hidden, inp.w1_fp4.shape[1])
    taps = O.MoETaps()
    O.moe_w4a16(inp.x, inp.w1_fp4, s1.view(torch.uint8), g1, inp.w2_fp4, inp.w2_blockscale.view(torch.uint8), g2,
                ids, tw, activation=act, taps=taps, scale_format="e8m0_k32")
    rows = taps.fc1.shape[0]
    assert torch.equal(b.packed_route_indices.cpu()[:rows], taps.sort.sorted_route_ids)
    assert (fc1[:rows] - taps.fc1).abs().max().item() <= 2e-5 * taps.fc1.abs().max().item()
    mid = b.materialized_intermediate.cpu()[:rows].view(torch.bfloat16).float()
    assert (mid != taps.mid).float().mean().item() <= 2e-3
    rms = taps.out_f32.square().mean().sqrt().item()
    assert (out - taps.out_f32).abs().max().item() <= 1e-2 * rms


@pytest.mark.gpu
def test_gpu_compressed_tensors_equals_modelopt_source():
    shp = synth.shape("c3", name="ct", tokens=24, hidden=256, intermediate=128, experts=4, topk=2,
                      activation="silu")
    inp = synth.make_inputs(shp, seed=9)
    g = torch.Generator().manual_seed(9)
    ids = torch.stack([torch.randperm(4, generator=g)[:2] for _ in range(24)]).to(torch.int32)
    tw = torch.rand(24, 2, generator=g)
    base = dict(w1_fp4=inp.w1_fp4, w2_fp4=inp.w2_fp4, w1_blockscale=inp.w1_blockscale,
                w2_blockscale=inp.w2_blockscale)
    # powers of two: the reciprocal round trip is exact, so the two runs must agree bit for bit
    g1 = torch.tensor([0.5, 2.0, 1.0, 0.25])
    g2 = torch.tensor([4.0, 0.125, 1.0, 2.0])
    _, _, out_mo = _run_gpu(_plan("modelopt_nvfp4"), dict(base, w1_global_scale=g1, w2_global_scale=g2),
                            inp.x, ids, tw, 24, 2, 256, 256)
    _, _, out_ct = _run_gpu(_plan("compressed_tensors"),
                            dict(base, w1_global_scale=1 / g1, w2_global_scale=1 / g2),
                            inp.x, ids, tw, 24, 2, 256, 256)
    assert out_mo.abs().max().item() > 0 and torch.equal(out_ct, out_mo)
