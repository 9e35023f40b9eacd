"""The CPU oracle against fixtures produced by the reference library's own torch oracle
(tests/golden/make_golden.py).  Runs without a GPU and without the reference."""

import numpy as np
import torch

from b12x_b200 import synth
from oracle import moe_oracle as O
from tests.helpers import load_golden, sha, t


def _rel(a, b):
    return (a - b).abs().max().item() / max(b.abs().max().item(), 1e-30)


def test_primitives_match_reference():
    g = load_golden("primitives.npz")
    sw = O.swizzle_block_scale(t(g["scale_grid"]))
    assert torch.equal(sw, t(g["scale_swizzled"]))
    for b in range(2):
        assert torch.equal(O.unswizzle_block_scale(sw[b], 200, 14), t(g["scale_grid"])[b])
    assert torch.equal(O.fp4_round(t(g["fp4_in"])), t(g["fp4_out"]))
    r, byte = O.pow2_ceil_ue8m0(t(g["ue8m0_in"]))
    assert torch.equal(r, t(g["ue8m0_rounded"])) and torch.equal(byte, t(g["ue8m0_byte"]))
    _, _, qd = O.quantize_mxfp8_rows(t(g["mxfp8_in"]))
    assert torch.equal(qd, t(g["mxfp8_qdq"]))
    _, _, deq = O.quantize_nvfp4_rows(t(g["nvfp4_rows"]), float(g["nvfp4_rows_gs"]))
    assert torch.equal(deq, t(g["nvfp4_rows_dequant"]))


def test_nvfp4_codes_and_scales_reproduce_dequant():
    g = load_golden("primitives.npz")
    codes, sfb, deq = O.quantize_nvfp4_rows(t(g["nvfp4_rows"]), float(g["nvfp4_rows_gs"]))
    vals = O.fp4_unpack(codes).reshape(5, 4, 16) * O.e4m3_bytes_to_float(sfb).unsqueeze(-1)
    assert torch.equal(vals.reshape(5, 64), deq)


def test_routing_known_answers():
    g = load_golden("primitives.npz")
    lg = t(g["route_logits"])
    _, ids, w = O.route_topk(lg, 4, mode="softmax_topk")
    assert torch.equal(ids, t(g["route_ids"]))
    torch.testing.assert_close(w, t(g["route_weights"]), rtol=1e-6, atol=1e-7)
    _, ids, w = O.route_topk(lg, 4, mode="raw")
    assert torch.equal(ids, t(g["route_raw_ids"])) and torch.equal(w, t(g["route_raw_weights"]))
    _, ids, w = O.route_topk(lg, 4, mode="sigmoid", bias=t(g["sig_bias"]), route_scale=2.5)
    assert torch.equal(ids, t(g["sig_ids"]))
    torch.testing.assert_close(w, t(g["sig_weights"]), rtol=1e-6, atol=1e-7)
    # the reference's own tiny cases (tests/moe/test_sparse_moe_api.py:152-236)
    _, ids, w = O.route_topk(torch.tensor([[10.0, 0.0, -1.0], [0.0, 10.0, -1.0]]), 2)
    assert ids.tolist() == [[0, 1], [1, 0]]
    torch.testing.assert_close(w, torch.softmax(torch.tensor([[10.0, 0.0], [10.0, 0.0]]), dim=-1))
    _, ids, w = O.route_topk(torch.tensor([[0.5, 3.0, -4.0]]), 2, mode="raw")
    assert ids.tolist() == [[1, 0]] and w.tolist() == [[3.0, 0.5]]
    # ties go to the larger index (b12x/moe/_shared/routing.py:39-43)
    _, ids, _ = O.route_topk(torch.tensor([[1.0, 2.0, 2.0, 0.0]]), 2)
    assert ids.tolist() == [[2, 1]]


def _check_nvfp4_case(g, inp, activation):
    a1 = t(g["w1_alphas"])
    a2 = t(g["w2_alphas"])
    ids, tw = t(g["topk_ids"]), t(g["topk_weights"])
    taps = O.MoETaps()
    out = O.moe_nvfp4(inp["x"], inp["w1_fp4"], inp["w1_blockscale"], a1, inp["w2_fp4"],
                      inp["w2_blockscale"], a2, inp["a1_gscale"], inp["a2_gscale"], ids, tw,
                      activation=activation, taps=taps)
    tt, topk = ids.shape
    inv = taps.sort.inv_perm.reshape(tt, topk).long()
    # activation quantisation: exact (element-wise arithmetic only)
    xdq = O.fp4_unpack(taps.act_codes).reshape(tt * topk, -1, 16) * \
        O.e4m3_bytes_to_float(taps.act_scales).unsqueeze(-1)
    assert torch.equal(xdq.reshape(tt * topk, -1)[inv], t(g["x_dequant"]))
    # FC1: same formulas, matrix-matrix instead of matrix-vector products -> fp32 round-off only
    fc1_ref = t(g["fc1"])
    assert _rel(taps.fc1[inv], fc1_ref) < 2e-6
    mid_ref = t(g["mid"])
    flips = (taps.mid[inv] != mid_ref).float().mean().item()
    assert flips < 2e-3, f"bf16 intermediate differs in {flips:.2%} of elements"
    out_f32 = t(g["out_f32"])
    rms = out_f32.square().mean().sqrt().item()
    assert (taps.out_f32 - out_f32).abs().max().item() <= 1e-2 * rms
    # bf16 result: at most one bf16 ulp off where the fp32 sums straddle a rounding boundary
    ref_bf16 = t(g["out_bf16"], torch.bfloat16).float()
    assert (out.float() - ref_bf16).abs().max().item() <= 2 * 2.0 ** -8 * ref_bf16.abs().max().item()
    return taps


def test_c1_nvfp4_silu_matches_reference_oracle():
    g = load_golden("c1_nvfp4_silu.npz")
    inp = synth.make_inputs(synth.shape("c1"), seed=0)
    for n in ("x", "router_logits", "w1_fp4", "w1_blockscale", "w2_fp4", "w2_blockscale", "a1_gscale",
              "a2_gscale", "w1_global_scale", "w2_global_scale"):
        assert sha(getattr(inp, n)) == str(g["sha_" + n]), f"regenerated input {n} differs from the fixture's"
    torch.testing.assert_close(inp.w1_global_scale / inp.a1_gscale, t(g["w1_alphas"]), rtol=0, atol=0)
    _, ids, w = O.route_topk(inp.router_logits, 2)
    assert torch.equal(ids, t(g["topk_ids"]))
    torch.testing.assert_close(w, t(g["topk_weights"]), rtol=1e-6, atol=1e-7)
    d = {k: getattr(inp, k) for k in ("x", "w1_fp4", "w1_blockscale", "w2_fp4", "w2_blockscale",
                                      "a1_gscale", "a2_gscale")}
    _check_nvfp4_case(g, d, "silu")


def _stored_inputs(g):
    d = {k[3:]: t(v) for k, v in g.items() if k.startswith("in_")}
    d["x"] = d["x"].view(torch.bfloat16)
    return d


def test_tiny_nvfp4_silu_and_swigluoai_match_reference_oracle():
    _check_nvfp4_case(load_golden("tiny_nvfp4_silu.npz"), _stored_inputs(load_golden("tiny_nvfp4_silu.npz")), "silu")
    g = load_golden("tiny_nvfp4_swigluoai.npz")
    _check_nvfp4_case(g, _stored_inputs(g), "swigluoai")


def test_tiny_nvfp4_situ_matches_reference_oracle():
    """SiTU (4 tanh(g/4) sigmoid(g) * 25 tanh(u/25)) against ``moe_reference_nvfp4(activation="situ")``
    of the reference (fixture made by tests/golden/make_golden_routing.py)."""
    g = load_golden("tiny_nvfp4_situ.npz")
    inp = _stored_inputs(g)
    a1 = inp["w1_global_scale"] / inp["a1_gscale"]
    a2 = inp["w2_global_scale"] / inp["a2_gscale"]
    ids, tw = t(g["topk_ids"]), t(g["topk_weights"])
    taps = O.MoETaps()
    out = O.moe_nvfp4(inp["x"], inp["w1_fp4"], inp["w1_blockscale"], a1, inp["w2_fp4"], inp["w2_blockscale"], a2,
                      inp["a1_gscale"], inp["a2_gscale"], ids, tw, activation="situ", taps=taps)
    tt, topk = ids.shape
    inv = taps.sort.inv_perm.reshape(tt, topk).long()
    flips = (taps.mid[inv] != t(g["mid"])).float().mean().item()
    assert flips < 2e-3, f"bf16 intermediate differs in {flips:.2%} of elements"
    ref = t(g["out_f32"])
    assert (taps.out_f32 - ref).abs().max().item() <= 1e-2 * ref.square().mean().sqrt().item()
    ref_bf16 = t(g["out_bf16"], torch.bfloat16).float()
    assert (out.float() - ref_bf16).abs().max().item() <= 2 * 2.0 ** -8 * ref_bf16.abs().max().item()


def test_relu2_bit_exact_case():
    g = load_golden("relu2_e1_k128.npz")
    out = O.moe_nvfp4(t(g["x"], torch.bfloat16), t(g["w1_fp4"]), t(g["w1_blockscale"]), t(g["w1_alphas"]),
                      t(g["w2_fp4"]), t(g["w2_blockscale"]), t(g["w2_alphas"]), t(g["a1_gscale"]),
                      t(g["a2_gscale"]), t(g["topk_ids"]), t(g["topk_weights"]), activation="relu2")
    ref = t(g["out_bf16"], torch.bfloat16).float()
    d = (out.float() - ref).abs()
    # K = N = 128: sums are short; allow single-ulp bf16 differences from summation order
    assert d.max().item() <= 2.0 ** -7 * ref.abs().max().item()
    assert (d > 0).float().mean().item() < 1e-2


def test_w4a16_matches_reference_oracle():
    g = load_golden("tiny_w4a16.npz")
    taps = O.MoETaps()
    ids, tw = t(g["topk_ids"]), t(g["topk_weights"])
    out = O.moe_w4a16(t(g["x"], torch.bfloat16), t(g["w1_fp4"]), t(g["w1_blockscale"]), t(g["w1_alphas"]),
                      t(g["w2_fp4"]), t(g["w2_blockscale"]), t(g["w2_alphas"]), ids, tw, taps=taps)
    inv = taps.sort.inv_perm.reshape(ids.shape).long()
    assert _rel(taps.fc1[inv], t(g["fc1"])) < 2e-6
    assert (taps.mid[inv] != t(g["mid"])).float().mean().item() < 2e-3
    # per-route FC2 output, rounded to bf16 by the reference
    down = taps.routed[inv].to(torch.bfloat16).float()
    assert (down != t(g["down_bf16_as_f32"])).float().mean().item() < 5e-3
    ref = t(g["out_bf16"], torch.bfloat16).float()
    # the reference accumulates bf16-rounded contributions in bf16; ours is fp32 + one rounding
    assert (out.float() - ref).abs().max().item() <= 4 * 2.0 ** -8 * ref.abs().max().item()


def test_w4a8_mx_matches_reference_oracle():
    g = load_golden("tiny_w4a8_mx.npz")
    e = t(g["w1_fp4"]).shape[0]
    ones = torch.ones(e)
    out = O.moe_w4a8_mx(t(g["x"], torch.bfloat16), t(g["w1_fp4"]), t(g["w1_e8m0"]), ones, t(g["w2_fp4"]),
                        t(g["w2_e8m0"]), ones, t(g["topk_ids"]), t(g["topk_weights"]))
    ref = t(g["out_f32"])
    rms = ref.square().mean().sqrt().item()
    assert (out - ref).abs().max().item() <= 1e-2 * rms


def test_synth_quantisers_equal_oracle_quantisers():
    gen = torch.Generator().manual_seed(7)
    w = torch.randn(3, 160, 128, generator=gen) * 0.02
    gs = O.per_expert_global_scale(w)
    codes, sw = O.quantize_nvfp4_weight(w, gs)
    for e in range(3):
        c, s, inv_g = synth.quantize_nvfp4_matrix(w[e])
        assert torch.equal(c, codes[e]) and torch.equal(s, sw[e])
        torch.testing.assert_close(inv_g, 1.0 / gs[e], rtol=1e-6, atol=0)
    c2, b2 = O.quantize_mxfp4_weight(w)
    for e in range(3):
        c, b = synth.quantize_mxfp4_matrix(w[e])
        assert torch.equal(c, c2[e]) and torch.equal(b, b2[e])


def test_expert_sort_canonical_order_and_dropped_routes():
    ids = torch.tensor([[3, 1], [1, 0], [7, 3], [1, 9]], dtype=torch.int32)
    s = O.expert_sort(ids, 4)
    assert s.expert_counts.tolist() == [1, 3, 0, 2]
    assert s.expert_offsets.tolist() == [0, 1, 4, 4, 6]
    assert s.sorted_route_ids.tolist() == [3, 1, 2, 6, 0, 5]
    assert s.inv_perm.tolist() == [4, 1, 2, 0, -1, 5, 3, -1]
    assert s.tile_base.tolist() == [0, 1, 2, 2, 3]
    emap = torch.tensor([-1, 0, -1, 1, -1, -1, -1, -1, -1, -1], dtype=torch.int32)
    s = O.expert_sort(ids, 2, emap)
    assert s.sorted_route_ids.tolist() == [1, 2, 6, 0, 5]
