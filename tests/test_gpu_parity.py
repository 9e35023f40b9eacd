"""-m gpu: the CUDA path (through the facade and the C ABI) against the CPU oracle, stage by stage.

Bars: routing ids, permutation, activation codes and scale bytes bit-exact; floating point taps
within the tolerance written next to each check; the layer output (fp32, before the final bf16
rounding) within 1e-2 x output RMS in max-abs."""

import pytest
import torch

from b12x_b200 import synth
from b12x_b200.moe import fused_moe
from oracle import moe_oracle as O
from tests.gpu_utils import oracle_layer, prepare_experts, route_on_gpu, run_layer
from tests.helpers import atoms_to_rows, load_golden, t

pytestmark = pytest.mark.gpu

OUT_TOL = 1e-2     # max-abs error <= OUT_TOL x RMS of the oracle output
FC1_TOL = 2e-5     # FC1 pre-activation: relative to the largest magnitude (fp32 summation order)
FLIP_TOL = 2e-3    # share of re-quantised intermediate bytes allowed to differ


def _tiny(**kw):
    base = dict(name="tiny", tokens=8, hidden=256, intermediate=128, experts=4, topk=2)
    base.update(kw)
    return synth.shape("c1", **base)


@pytest.mark.parametrize("mode,e,k,tokens", [("softmax", 24, 4, 12), ("softmax", 256, 8, 64), ("raw", 8, 2, 5),
                                             ("sigmoid", 256, 8, 33), ("softmax", 1000, 6, 7), ("softmax", 128, 32, 9)])
def test_route_topk_ids_bit_exact(mode, e, k, tokens):
    g = torch.Generator().manual_seed(e * 31 + k)
    lg = torch.randn(tokens, e, generator=g)
    bias = torch.randn(e, generator=g) * 0.1 if mode == "sigmoid" else None
    dev = "cuda"
    tl = torch.empty(tokens, k, device=dev)
    ti = torch.empty(tokens, k, dtype=torch.int32, device=dev)
    tw = torch.empty(tokens, k, device=dev)
    if mode == "sigmoid":
        fused_moe.route_topk(lg.to(dev), tl, ti, tw, renormalize=True, score_func="sigmoid",
                             selection_bias=bias.to(dev), route_scale=2.5)
        _, ids, w = O.route_topk(lg, k, mode="sigmoid", bias=bias, route_scale=2.5)
    else:
        fused_moe.route_topk(lg.to(dev), tl, ti, tw, renormalize=(mode == "softmax"))
        _, ids, w = O.route_topk(lg, k, mode="softmax_topk" if mode == "softmax" else "raw")
    assert torch.equal(ti.cpu(), ids)
    # exp() of the device and of the host differ in the last place; 4 ulp of fp32
    torch.testing.assert_close(tw.cpu(), w, rtol=5e-7, atol=1e-9)


def test_route_topk_golden_and_ties():
    g = load_golden("primitives.npz")
    lg = t(g["route_logits"]).cuda()
    tl = torch.empty(12, 4, device="cuda")
    ti = torch.empty(12, 4, dtype=torch.int32, device="cuda")
    tw = torch.empty(12, 4, device="cuda")
    fused_moe.route_topk(lg, tl, ti, tw, renormalize=True)
    assert torch.equal(ti.cpu(), t(g["route_ids"]))
    torch.testing.assert_close(tw.cpu(), t(g["route_weights"]), rtol=1e-6, atol=1e-8)
    tie = torch.tensor([[1.0, 2.0, 2.0, 0.0], [5.0, 5.0, 5.0, 5.0]], device="cuda")
    ti2 = torch.empty(2, 2, dtype=torch.int32, device="cuda")
    fused_moe.route_topk(tie, torch.empty(2, 2, device="cuda"), ti2, torch.empty(2, 2, device="cuda"), renormalize=True)
    assert ti2.cpu().tolist() == [[2, 1], [3, 2]]
    # bf16 logits are accepted
    fused_moe.route_topk(lg.bfloat16(), tl, ti, tw, renormalize=True)
    _, ids, _ = O.route_topk(t(g["route_logits"]).bfloat16().float(), 4)
    assert torch.equal(ti.cpu(), ids)


def _check_sort(run, taps):
    b, s = run.binding, taps.sort
    rows = s.sorted_route_ids.numel()
    assert torch.equal(b.expert_counts.cpu(), s.expert_counts)
    assert torch.equal(b.expert_offsets.cpu(), s.expert_offsets)
    assert torch.equal(b.expert_tile_base.cpu(), s.tile_base)
    assert torch.equal(b.packed_route_indices.cpu()[:rows], s.sorted_route_ids)
    assert torch.equal(b.inv_perm.cpu(), s.inv_perm)
    return rows


def _check_nvfp4_layer(run, *, expert_map=None, out_tol=OUT_TOL):
    shp = run.inp.shape
    ref, taps = oracle_layer(run.inp, run.topk_ids, run.topk_weights, expert_map)
    # the row-tile tables follow the plan's tile height (64 in small-batch plans)
    taps.sort = O.retile(taps.sort, int(run.binding.core_layout.tile_rows))
    b, s = run.binding, taps.sort
    rows = _check_sort(run, taps)
    if rows == 0:
        assert torch.count_nonzero(run.out_f32) == 0
        return
    assert torch.equal(b.packed_input.cpu()[:rows], taps.act_codes), "activation codes differ"
    sf = b.packed_input_scale.cpu()
    atoms = (shp.hidden + 63) // 64
    for mt in range(int(s.tile_base[-1])):
        r0, nr = int(s.mtile_row0[mt]), int(s.mtile_rows[mt])
        assert torch.equal(atoms_to_rows(sf, mt, atoms, nr, shp.hidden // 16), taps.act_scales[r0:r0 + nr])
    if run.fc1 is not None:
        d = (run.fc1[:rows] - taps.fc1).abs().max().item()
        assert d <= FC1_TOL * taps.fc1.abs().max().item(), f"FC1 tap off by {d}"
    flips = (b.materialized_intermediate.cpu()[:rows] != taps.mid_codes).float().mean().item()
    assert flips <= FLIP_TOL, f"{flips:.3%} of the intermediate code bytes differ"
    rms = taps.out_f32.square().mean().sqrt().item()
    err = (run.out_f32 - taps.out_f32).abs().max().item()
    assert err <= out_tol * rms, f"output max-abs error {err:.3e} > {out_tol} x rms {rms:.3e}"
    # bf16 result: the fp32 sums agree to << 1 bf16 ulp, so the roundings agree up to 1 ulp
    assert (run.out.float() - ref.float()).abs().max().item() <= 2.0 ** -7 * ref.float().abs().max().item()


def test_c1_matches_reference_golden():
    """Benchmark config 1 against the output of the reference library's own oracle."""
    g = load_golden("c1_nvfp4_silu.npz")
    inp = synth.make_inputs(synth.shape("c1"), seed=0)
    run = run_layer(inp)
    assert torch.equal(run.topk_ids, t(g["topk_ids"]))
    torch.testing.assert_close(run.topk_weights, t(g["topk_weights"]), rtol=1e-6, atol=1e-8)
    ref = t(g["out_f32"])
    rms = ref.square().mean().sqrt().item()
    assert (run.out_f32 - ref).abs().max().item() <= OUT_TOL * rms
    inv = run.binding.inv_perm.cpu().reshape(16, 2).long()
    fc1_ref = t(g["fc1"])
    assert (run.fc1[inv] - fc1_ref).abs().max().item() <= FC1_TOL * fc1_ref.abs().max().item()
    _check_nvfp4_layer(run)


@pytest.mark.parametrize("tokens", [1, 8, 127, 129, 300])
def test_nvfp4_silu_token_counts(tokens):
    _check_nvfp4_layer(run_layer(synth.make_inputs(_tiny(tokens=tokens, hidden=512, intermediate=256, experts=8), seed=tokens)))


def test_nvfp4_swigluoai_and_relu2():
    _check_nvfp4_layer(run_layer(synth.make_inputs(_tiny(tokens=40, activation="swigluoai"), seed=11)))
    _check_nvfp4_layer(run_layer(synth.make_inputs(_tiny(tokens=40, activation="relu2", intermediate=384), seed=12)))


def test_nvfp4_golden_swigluoai_inputs():
    g = load_golden("tiny_nvfp4_swigluoai.npz")
    shp = _tiny(activation="swigluoai")
    inp = synth.make_inputs(shp, seed=1)
    assert torch.equal(inp.w1_fp4, t(g["in_w1_fp4"]))
    run = run_layer(inp, topk_ids=t(g["topk_ids"]), topk_weights=t(g["topk_weights"]))
    ref = t(g["out_f32"])
    assert (run.out_f32 - ref).abs().max().item() <= OUT_TOL * ref.square().mean().sqrt().item()


@pytest.mark.parametrize("tile_rows", [64, 128])
def test_nvfp4_situ_against_oracle_and_reference_fixture(tile_rows):
    """The SiTU activation on both kernel families, stage by stage against the oracle, and on the
    fixture's inputs against the output of the reference's own oracle."""
    _check_nvfp4_layer(run_layer(synth.make_inputs(_tiny(tokens=40, activation="situ"), seed=13), tile_rows=tile_rows))
    g = load_golden("tiny_nvfp4_situ.npz")
    inp = synth.make_inputs(synth.shape("c1", name="tiny_situ", tokens=8, hidden=256, intermediate=128, experts=4,
                                        activation="situ"), seed=6)
    assert torch.equal(inp.w1_fp4, t(g["in_w1_fp4"])) and torch.equal(inp.x.view(torch.int16), t(g["in_x"]))
    run = run_layer(inp, topk_ids=t(g["topk_ids"]), topk_weights=t(g["topk_weights"]), tile_rows=tile_rows)
    ref = t(g["out_f32"])
    assert (run.out_f32 - ref).abs().max().item() <= OUT_TOL * ref.square().mean().sqrt().item()


def test_relu2_reference_bit_exact_case():
    """E=1, K=N=128: the reference requires max_abs == 0 between its kernel and its oracle
    (tests/moe/test_tp_moe_relu2_reference.py:240-274)."""
    g = load_golden("relu2_e1_k128.npz")
    shp = synth.shape("c1", name="relu2", tokens=16, hidden=128, intermediate=128, experts=1, topk=1, activation="relu2")
    ones = torch.ones(1)
    inp = synth.MoEInputs(shp, t(g["x"], torch.bfloat16), torch.zeros(16, 1), None, t(g["w1_fp4"]),
                          t(g["w1_blockscale"]), t(g["w1_alphas"]), t(g["w2_fp4"]), t(g["w2_blockscale"]),
                          t(g["w2_alphas"]), ones, ones)
    run = run_layer(inp, topk_ids=t(g["topk_ids"]), topk_weights=t(g["topk_weights"]))
    ref = t(g["out_bf16"], torch.bfloat16).float()
    assert (run.out.float() - ref).abs().max().item() == 0.0


def test_expert_map_drops_non_local_routes():
    shp = _tiny(tokens=50, experts=8, topk=3)
    inp = synth.make_inputs(shp, seed=5)
    # this rank holds global experts 4..7 as local 0..3
    local = synth.MoEInputs(shp, inp.x, inp.router_logits, None, inp.w1_fp4[4:], inp.w1_blockscale[4:],
                            inp.w1_global_scale[4:], inp.w2_fp4[4:], inp.w2_blockscale[4:],
                            inp.w2_global_scale[4:], inp.a1_gscale[4:], inp.a2_gscale[4:])
    emap = torch.tensor([-1, -1, -1, -1, 0, 1, 2, 3], dtype=torch.int32)
    _, ids, w = O.route_topk(inp.router_logits, 3)
    run = run_layer(local, topk_ids=ids, topk_weights=w, expert_map=emap)
    _check_nvfp4_layer(run, expert_map=emap)


def test_all_routes_to_one_expert_and_empty_experts():
    shp = _tiny(tokens=200, experts=4, topk=1)
    inp = synth.make_inputs(shp, seed=6)
    ids = torch.full((200, 1), 2, dtype=torch.int32)
    w = torch.rand(200, 1) + 0.5
    _check_nvfp4_layer(run_layer(inp, topk_ids=ids, topk_weights=w))


def test_zero_tokens_and_capacity_errors():
    shp = _tiny(tokens=4)
    inp = synth.make_inputs(shp, seed=7)
    run = run_layer(inp, max_tokens=16)
    _check_nvfp4_layer(run)
    with pytest.raises(ValueError):
        run.plan.bind(scratch=torch.empty(10, dtype=torch.uint8, device="cuda"), a=inp.x.cuda(),
                      experts=run.experts, topk_weights=run.topk_weights.cuda(), topk_ids=run.topk_ids.cuda())
    big = torch.zeros(17, shp.hidden, dtype=torch.bfloat16, device="cuda")
    spec = run.plan.scratch_specs()[0]
    with pytest.raises(ValueError):
        run.plan.bind(scratch=torch.empty(spec.shape, dtype=torch.uint8, device="cuda"), a=big, experts=run.experts,
                      topk_weights=torch.zeros(17, 2, device="cuda"),
                      topk_ids=torch.zeros(17, 2, dtype=torch.int32, device="cuda"))


def test_repeat_runs_are_bitwise_identical():
    inp = synth.make_inputs(_tiny(tokens=150, hidden=512, experts=8), seed=8)
    a = run_layer(inp, poison=0x00)
    b = run_layer(inp, poison=0xFF)
    assert torch.equal(a.out, b.out) and torch.equal(a.out_f32, b.out_f32)


# ------------------------------------------------------------------------------------------------
# w4a8_mx: MXFP8 activations x MXFP4 weights (kind::mxf8f6f4)
# ------------------------------------------------------------------------------------------------
def _mx(**kw):
    base = dict(name="mx", tokens=24, hidden=256, intermediate=128, experts=4, topk=2, activation="silu")
    base.update(kw)
    return synth.shape("c5", **base)


def _check_mx_layer(run, *, expert_map=None):
    shp = run.inp.shape
    ref, taps = oracle_layer(run.inp, run.topk_ids, run.topk_weights, expert_map)
    b, s = run.binding, taps.sort
    rows = _check_sort(run, taps)
    assert torch.equal(b.packed_input.cpu()[:rows], taps.act_codes), "MXFP8 activation codes differ"
    sf = b.packed_input_scale.cpu()
    atoms = (shp.hidden + 127) // 128
    for mt in range(int(s.tile_base[-1])):
        r0, nr = int(s.mtile_row0[mt]), int(s.mtile_rows[mt])
        assert torch.equal(atoms_to_rows(sf, mt, atoms, nr, shp.hidden // 32), taps.act_scales[r0:r0 + nr])
    d = (run.fc1[:rows] - taps.fc1).abs().max().item()
    assert d <= FC1_TOL * taps.fc1.abs().max().item(), f"FC1 tap off by {d}"
    flips = (b.materialized_intermediate.cpu()[:rows] != taps.mid_codes).float().mean().item()
    assert flips <= FLIP_TOL, f"{flips:.3%} of the intermediate code bytes differ"
    rms = taps.out_f32.square().mean().sqrt().item()
    err = (run.out_f32 - taps.out_f32).abs().max().item()
    assert err <= OUT_TOL * rms, f"output max-abs error {err:.3e} > {OUT_TOL} x rms {rms:.3e}"


@pytest.mark.parametrize("tokens,hidden,inter,act", [
    (24, 256, 128, "silu"), (150, 512, 256, "swigluoai"), (40, 256, 256, "relu2"),
    (33, 320, 192, "swigluoai"),      # K and I with a half tile left over, like hidden 2880
    (1, 384, 128, "silu")])
def test_w4a8_mx_layer(tokens, hidden, inter, act):
    inp = synth.make_inputs(_mx(tokens=tokens, hidden=hidden, intermediate=inter, activation=act), seed=tokens + hidden)
    _check_mx_layer(run_layer(inp))


def test_w4a8_mx_matches_reference_golden():
    g = load_golden("tiny_w4a8_mx.npz")
    shp = _mx(tokens=8)
    inp = synth.make_inputs(shp, seed=4)
    assert torch.equal(inp.w1_fp4, t(g["w1_fp4"])) and torch.equal(inp.w1_blockscale, t(g["w1_e8m0"]))
    run = run_layer(inp, topk_ids=t(g["topk_ids"]), topk_weights=t(g["topk_weights"]))
    ref = t(g["out_f32"])
    assert (run.out_f32 - ref).abs().max().item() <= OUT_TOL * ref.square().mean().sqrt().item()


# ------------------------------------------------------------------------------------------------
# w4a16: BF16 activations x NVFP4 weights expanded to BF16 inside the kernel (kind::f16)
# ------------------------------------------------------------------------------------------------
def _w16(**kw):
    base = dict(name="w16", tokens=24, hidden=256, intermediate=128, experts=4, topk=2, activation="silu")
    base.update(kw)
    return synth.shape("c3", **base)


def _check_w4a16_layer(run, *, expert_map=None, weight_on_input=False):
    ref, taps = oracle_layer(run.inp, run.topk_ids, run.topk_weights, expert_map, weight_on_input)
    b = run.binding
    rows = _check_sort(run, taps)
    d = (run.fc1[:rows] - taps.fc1).abs().max().item()
    assert d <= FC1_TOL * taps.fc1.abs().max().item(), f"FC1 tap off by {d}"
    mid = b.materialized_intermediate.cpu()[:rows].view(torch.bfloat16).float()
    flips = (mid != taps.mid).float().mean().item()
    assert flips <= FLIP_TOL, f"{flips:.3%} of the bf16 intermediate differs"
    assert (mid - taps.mid).abs().max().item() <= 2.0 ** -7 * taps.mid.abs().max().item()
    rms = taps.out_f32.square().mean().sqrt().item()
    err = (run.out_f32 - taps.out_f32).abs().max().item()
    assert err <= OUT_TOL * rms, f"output max-abs error {err:.3e} > {OUT_TOL} x rms {rms:.3e}"


@pytest.mark.parametrize("tokens,hidden,inter,act", [
    (24, 256, 128, "silu"), (200, 512, 384, "silu"), (40, 256, 256, "relu2"),
    (33, 320, 192, "silu"),           # gate half starts mid-way through a scale atom (I % 128 != 0)
    (1, 384, 128, "silu")])
def test_w4a16_layer(tokens, hidden, inter, act):
    inp = synth.make_inputs(_w16(tokens=tokens, hidden=hidden, intermediate=inter, activation=act), seed=tokens + inter)
    _check_w4a16_layer(run_layer(inp))


@pytest.mark.parametrize("tokens,topk,act", [(48, 1, "silu"), (200, 2, "silu"), (40, 2, "relu2")])
def test_w4a16_router_weight_on_input(tokens, topk, act):
    """``Caps.apply_router_weight_on_input`` (W4A16 only, as in the reference): the route's weight
    multiplies FC1's rows before the activation, the combine adds the routes with unit weights."""
    inp = synth.make_inputs(_w16(tokens=tokens, topk=topk, hidden=384, intermediate=256, activation=act), seed=tokens)
    run = run_layer(inp, weight_on_input=True)
    _check_w4a16_layer(run, weight_on_input=True)
    plain = run_layer(inp)
    if topk > 1:                                        # (one renormalised route weighs exactly 1)
        assert not torch.equal(run.out, plain.out)      # the option is not a no-op
    with pytest.raises(NotImplementedError):
        inp4 = synth.make_inputs(synth.shape("c1", name="x", tokens=8, hidden=256, intermediate=128, experts=4, topk=2), seed=1)
        run_layer(inp4, weight_on_input=True)


def test_w4a16_activation_amax_side_channel():
    """``bind(activation_amax=, layer_idx=)`` (W4A16 only, as in the reference): after a run row
    ``layer_idx`` holds, per local expert, max |x| over the rows routed to it and max |h| over its
    BF16 intermediate rows; the maximum is kept across runs; other layers' rows are untouched."""
    dev = torch.device("cuda")
    inp = synth.make_inputs(_w16(tokens=150, topk=2, hidden=384, intermediate=256, experts=6), seed=9, device=dev)
    ex = prepare_experts(inp, dev)
    caps = fused_moe.Caps(max_tokens=150, num_topk=2, device=dev, weight_plan=ex.plan, quant_mode="w4a16",
                          collect_activation_amax=True)
    plan = fused_moe.plan(caps)
    spec = plan.scratch_specs()[0]
    scratch = torch.empty(spec.shape, dtype=spec.dtype, device=dev)
    _, ti, tw = route_on_gpu(inp, dev)
    amax = torch.zeros(3, 6, 2, device=dev)
    amax[0].fill_(7.0)
    b = fused_moe.bind(plan, scratch=scratch, a=inp.x, experts=ex, topk_weights=tw, topk_ids=ti,
                       activation_amax=amax, layer_idx=1)
    fused_moe.run(binding=b)
    torch.cuda.synchronize()
    fused_moe.check_device_status(b)
    ids = ti.cpu().long()
    mid = b.materialized_intermediate.view(torch.bfloat16).float()
    offs = b.expert_offsets.cpu().tolist()
    for e in range(6):
        tok = (ids == e).any(dim=1)
        want_x = inp.x.cpu().float()[tok].abs().max().item() if bool(tok.any()) else 0.0
        want_h = mid[offs[e]:offs[e + 1]].abs().max().item() if offs[e + 1] > offs[e] else 0.0
        assert amax[1, e, 0].item() == want_x and amax[1, e, 1].item() == want_h
    assert bool((amax[0] == 7.0).all()) and bool((amax[2] == 0.0).all())
    # a second run on half-sized inputs cannot lower the record
    before = amax.clone()
    b2 = fused_moe.bind(plan, scratch=scratch, a=(inp.x * 0.5).to(torch.bfloat16), experts=ex, topk_weights=tw,
                        topk_ids=ti, activation_amax=amax, layer_idx=1)
    fused_moe.run(binding=b2)
    torch.cuda.synchronize()
    assert torch.equal(amax, before)
    # W4A16 only
    inp4 = synth.make_inputs(synth.shape("c1", name="x", tokens=8, hidden=256, intermediate=128, experts=4, topk=2), seed=1, device=dev)
    ex4 = prepare_experts(inp4, dev)
    plan4 = fused_moe.plan(fused_moe.Caps(max_tokens=8, num_topk=2, device=dev, weight_plan=ex4.plan, quant_mode="nvfp4"))
    s4 = torch.empty(plan4.scratch_specs()[0].shape, dtype=torch.uint8, device=dev)
    _, ti4, tw4 = route_on_gpu(inp4, dev)
    with pytest.raises(NotImplementedError):
        fused_moe.bind(plan4, scratch=s4, a=inp4.x, experts=ex4, topk_weights=tw4, topk_ids=ti4,
                       activation_amax=torch.zeros(1, 4, 2, device=dev), layer_idx=0)


def test_w4a16_matches_reference_golden():
    g = load_golden("tiny_w4a16.npz")
    inp = synth.make_inputs(_w16(tokens=8), seed=3)
    assert torch.equal(inp.w1_fp4, t(g["w1_fp4"])) and torch.equal(inp.w1_blockscale, t(g["w1_blockscale"]))
    run = run_layer(inp, topk_ids=t(g["topk_ids"]), topk_weights=t(g["topk_weights"]))
    inv = run.binding.inv_perm.cpu().reshape(8, 2).long()
    fc1_ref = t(g["fc1"])
    assert (run.fc1[inv] - fc1_ref).abs().max().item() <= FC1_TOL * fc1_ref.abs().max().item()
    ref = t(g["out_bf16"], torch.bfloat16).float()
    # the reference rounds every route's contribution to bf16 and sums in bf16 (w4a16_reference.py:619-621)
    assert (run.out.float() - ref).abs().max().item() <= 4 * 2.0 ** -8 * ref.abs().max().item()


@pytest.mark.parametrize("tokens,topk,experts,tile_rows", [(4096, 4, 128, 128), (16384, 1, 8, 128), (9000, 2, 37, 128),
                                                           (2048, 8, 256, 64), (65536, 8, 16, 128)])
def test_large_sorts_use_the_multi_cta_path_and_stay_canonical(tokens, topk, experts, tile_rows):
    """From 16 384 routes on the sort runs as three launches over many CTAs: counts, offsets, row
    tiles and the whole permutation must equal the oracle's stable sort bit for bit (ids outside the
    expert range and a route-expert map with holes included)."""
    import ctypes as C

    from b12x_b200._lib import ext
    gen = torch.Generator().manual_seed(tokens + experts)
    ids = torch.randint(-2, experts + 3, (tokens, topk), generator=gen, dtype=torch.int32)
    emap = torch.arange(experts + 3, dtype=torch.int32)
    emap[::5] = -1
    emap[experts:] = -1
    layout = ext.scratch_layout(tokens, topk, experts, 256, 128, "nvfp4", "silu", tile_rows)
    scratch = torch.full((int(layout.total_nbytes),), 0xFF, dtype=torch.uint8, device="cuda")
    for use_map in (False, True):
        args = ext.SortArgs(ids.cuda().data_ptr(), emap.cuda().data_ptr() if use_map else None, scratch.data_ptr(),
                            C.pointer(layout), tokens, topk, experts, emap.numel() if use_map else 0, None, None, None, 0, 0)
        ids_dev = ids.cuda()
        emap_dev = emap.cuda()
        args = ext.SortArgs(ids_dev.data_ptr(), emap_dev.data_ptr() if use_map else None, scratch.data_ptr(),
                            C.pointer(layout), tokens, topk, experts, emap.numel() if use_map else 0, None, None, None, 0, 0)
        ext.check(ext.load().b200moe_expert_sort(C.byref(args), torch.cuda.current_stream().cuda_stream), "sort")
        torch.cuda.synchronize()
        srt = O.expert_sort(ids, experts, emap if use_map else None, tile_rows=int(layout.tile_rows))
        view = lambda name, n: scratch[int(getattr(layout, name)): int(getattr(layout, name)) + 4 * n].view(torch.int32).cpu()
        kept = srt.sorted_route_ids.numel()
        assert torch.equal(view("expert_counts", experts), srt.expert_counts)
        assert torch.equal(view("expert_offsets", experts + 1), srt.expert_offsets)
        assert torch.equal(view("tile_base", experts + 1), srt.tile_base)
        assert torch.equal(view("sorted_route_ids", kept), srt.sorted_route_ids)
        assert torch.equal(view("inv_perm", tokens * topk), srt.inv_perm)
        nt = int(srt.tile_base[-1])
        assert torch.equal(view("mtile_expert", nt), srt.mtile_expert)
        assert torch.equal(view("mtile_row0", nt), srt.mtile_row0)
        assert torch.equal(view("mtile_rows", nt), srt.mtile_rows)
        assert view("status", 16).tolist() == [0] * 16
