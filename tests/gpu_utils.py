"""Run the CUDA layer through the public facade (and so through the C ABI) and hand back the
stage taps next to the oracle's, for the ``-m gpu`` parity tests."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from b12x_b200 import synth
from b12x_b200.moe import fused_moe
from oracle import moe_oracle as O

ACT_API = {"silu": "silu", "relu2": "relu2", "swigluoai": "swigluoai_uninterleave", "situ": "situ"}
SOURCE = {"nvfp4": "modelopt_nvfp4", "w4a16": "modelopt_nvfp4", "w4a8_mx": "fp4_e8m0_k32"}


@dataclass
class LayerRun:
    inp: synth.MoEInputs
    binding: object
    out: torch.Tensor            # bf16 [T, K] (cpu)
    out_f32: torch.Tensor        # f32 [T, K] (cpu)
    fc1: torch.Tensor            # f32 [rows_cap, w1_rows] (cpu)
    topk_ids: torch.Tensor       # cpu
    topk_weights: torch.Tensor   # cpu
    experts: object
    plan: object


def prepare_experts(inp: synth.MoEInputs, dev, *, w13_layout="w13"):
    shp = inp.shape
    wp = fused_moe.plan_weights(
        quant_modes=shp.recipe, source_format=SOURCE[shp.recipe], activation=ACT_API[shp.activation],
        params_dtype=torch.bfloat16, num_experts=inp.w1_fp4.shape[0], hidden_size=shp.hidden,
        intermediate_size=shp.intermediate, w13_layout=w13_layout)
    kw = dict(plan=wp, params_dtype=torch.bfloat16, w1_fp4=inp.w1_fp4.to(dev), w2_fp4=inp.w2_fp4.to(dev),
              w1_blockscale=inp.w1_blockscale.to(dev), w2_blockscale=inp.w2_blockscale.to(dev))
    if shp.recipe == "nvfp4":
        kw.update(w1_global_scale=inp.w1_global_scale.to(dev), w2_global_scale=inp.w2_global_scale.to(dev),
                  a1_gscale=inp.a1_gscale.to(dev), a2_gscale=inp.a2_gscale.to(dev))
    elif shp.recipe == "w4a16":
        kw.update(w1_global_scale=inp.w1_global_scale.to(dev), w2_global_scale=inp.w2_global_scale.to(dev))
    return fused_moe.prepare_weights(**kw)


def route_on_gpu(inp: synth.MoEInputs, dev):
    shp = inp.shape
    t, k = inp.router_logits.shape[0], shp.topk
    tl = torch.empty(t, k, device=dev)
    ti = torch.empty(t, k, dtype=torch.int32, device=dev)
    tw = torch.empty(t, k, device=dev)
    if shp.router == "sigmoid":
        fused_moe.route_topk(inp.router_logits.to(dev), tl, ti, tw, renormalize=True, score_func="sigmoid",
                             route_scale=shp.route_scale)
    else:
        fused_moe.route_topk(inp.router_logits.to(dev), tl, ti, tw, renormalize=True)
    return tl, ti, tw


def run_layer(inp: synth.MoEInputs, *, topk_ids=None, topk_weights=None, expert_map=None, poison=0xFF,
              max_tokens=None, w13_layout="w13", want_fc1=True, tile_rows=None,
              weight_on_input=False) -> LayerRun:
    dev = torch.device("cuda")
    shp = inp.shape
    ex = prepare_experts(inp, dev, w13_layout=w13_layout)
    t = inp.x.shape[0]
    caps = fused_moe.Caps(max_tokens=max_tokens or max(t, 1), num_topk=shp.topk, device=dev,
                          weight_plan=ex.plan, quant_mode=shp.recipe, tile_rows=tile_rows,
                          apply_router_weight_on_input=weight_on_input)
    plan = fused_moe.plan(caps)
    spec = plan.scratch_specs()[0]
    # poison the arena: a kernel that reads something it did not write shows up as garbage
    scratch = torch.full(spec.shape, poison, dtype=spec.dtype, device=dev)
    if topk_ids is None:
        _, ti, tw = route_on_gpu(inp, dev)
    else:
        ti, tw = topk_ids.to(dev), topk_weights.to(dev)
    rows_cap = caps.max_tokens * shp.topk
    fc1 = torch.zeros(rows_cap, inp.w1_fp4.shape[1], device=dev) if want_fc1 else None
    of32 = torch.zeros(t, shp.hidden, device=dev)
    emap = None if expert_map is None else expert_map.to(dev)
    b = fused_moe.bind(plan, scratch=scratch, a=inp.x.to(dev), experts=ex, topk_weights=tw, topk_ids=ti,
                       fc1_tap=fc1, output_f32=of32, route_expert_map=emap)
    out = fused_moe.run(binding=b)
    torch.cuda.synchronize()
    fused_moe.check_device_status(b)
    return LayerRun(inp, b, out.cpu(), of32.cpu(), None if fc1 is None else fc1.cpu(), ti.cpu(), tw.cpu(), ex, plan)


def oracle_layer(inp: synth.MoEInputs, ids, weights, expert_map=None, weight_on_input=False):
    shp = inp.shape
    taps = O.MoETaps()
    if shp.recipe == "nvfp4":
        a1 = inp.w1_global_scale / inp.a1_gscale
        a2 = inp.w2_global_scale / inp.a2_gscale
        out = O.moe_nvfp4(inp.x, inp.w1_fp4, inp.w1_blockscale, a1, inp.w2_fp4, inp.w2_blockscale, a2,
                          inp.a1_gscale, inp.a2_gscale, ids, weights, activation=shp.activation,
                          expert_map=expert_map, taps=taps)
    elif shp.recipe == "w4a16":
        out = O.moe_w4a16(inp.x, inp.w1_fp4, inp.w1_blockscale, inp.w1_global_scale, inp.w2_fp4,
                          inp.w2_blockscale, inp.w2_global_scale, ids, weights, activation=shp.activation,
                          expert_map=expert_map, taps=taps, apply_router_weight_on_input=weight_on_input)
    else:
        ones = torch.ones(inp.w1_fp4.shape[0])
        out = O.moe_w4a8_mx(inp.x, inp.w1_fp4, inp.w1_blockscale, ones, inp.w2_fp4, inp.w2_blockscale, ones,
                            ids, weights, activation=shp.activation, expert_map=expert_map, taps=taps)
    return out, taps


def oracle_call(shp, x, w1, s1, g1, w2, s2, g2, a1, a2, ids, weights, expert_map=None, taps=None):
    """The oracle layer for ``shp.recipe`` on explicit tensors (source-format weights)."""
    if shp.recipe == "nvfp4":
        return O.moe_nvfp4(x, w1, s1, g1 / a1, w2, s2, g2 / a2, a1, a2, ids, weights, activation=shp.activation,
                           expert_map=expert_map, taps=taps)
    if shp.recipe == "w4a16":
        return O.moe_w4a16(x, w1, s1, g1, w2, s2, g2, ids, weights, activation=shp.activation,
                           expert_map=expert_map, taps=taps)
    ones = torch.ones(w1.shape[0])
    return O.moe_w4a8_mx(x, w1, s1, ones, w2, s2, ones, ids, weights, activation=shp.activation,
                         expert_map=expert_map, taps=taps)


def sampled_parity(binding, inp: synth.MoEInputs, *, experts: int = 4, rows_per_expert: int = 48,
                   tolerance: float = 1e-2, a=None) -> dict:
    """Check what the last ``run`` of ``binding`` left in its scratch arena against the CPU oracle.

    Full-size shapes are too large for the oracle as a whole, so: (1) the WHOLE permutation
    (sorted route ids, inverse permutation, per-expert counts) is compared bit for bit with the
    oracle's canonical sort; (2) for up to ``rows_per_expert`` routes of ``experts`` experts (spread
    over the experts that received rows) the oracle evaluates the route from the input row on: the
    activation codes and scale bytes must be bit-identical, the fp32 FC2 rows (alpha applied,
    router weight not) within ``tolerance`` x their RMS.  ``inp`` holds the source-format weights of
    the experts this binding's layer owns (in its local numbering).  ``a`` (anything with
    ``index_select(0, rows)``) stands in for the binding's input rows where the layer received them
    already quantised."""
    b = binding
    shp = inp.shape
    torch.cuda.synchronize(b.device)
    tokens, k = b.topk_ids.shape
    ids = b.topk_ids.cpu()
    emap = None if b.route_expert_map is None else b.route_expert_map.cpu()
    srt = O.expert_sort(ids, b.weight_E, emap, tile_rows=int(b.core_layout.tile_rows))
    kept = int(srt.sorted_route_ids.numel())
    perm_ok = bool(torch.equal(b.packed_route_indices[:kept].cpu(), srt.sorted_route_ids)
                   and torch.equal(b.inv_perm.cpu(), srt.inv_perm)
                   and torch.equal(b.expert_counts.cpu(), srt.expert_counts))
    active = [e for e in range(b.weight_E) if int(srt.expert_counts[e]) > 0]
    res = {"experts": 0, "rows": 0, "permutation_rows": kept, "permutation_ok": perm_ok, "codes_ok": True,
           "max_abs_over_rms": 0.0, "tolerance": tolerance, "ok": perm_ok}
    if not active or experts <= 0:
        return res
    step = max(len(active) // experts, 1)
    chosen = active[::step][:experts]
    pos, local = [], []
    for j, e in enumerate(chosen):
        lo, hi = int(srt.expert_offsets[e]), int(srt.expert_offsets[e + 1])
        n = min(hi - lo, rows_per_expert)
        pos.extend(range(lo, lo + n))
        local.extend([j] * n)
    n = len(pos)
    pos_t = torch.tensor(pos, dtype=torch.int64)
    pos_d = pos_t.to(b.device)
    tok = (srt.sorted_route_ids.to(torch.int64)[pos_t] // k).to(b.device)
    x_sub = (b.a if a is None else a).index_select(0, tok).cpu()
    got = b.route_output.index_select(0, pos_d).cpu()
    sel = torch.tensor(chosen, dtype=torch.int64)
    pick = lambda t: t.index_select(0, sel.to(t.device)).cpu()
    taps = O.MoETaps()
    # the sub-batch is ordered by (expert, position), which the oracle's stable sort keeps
    oracle_call(shp, x_sub, pick(inp.w1_fp4), pick(inp.w1_blockscale), pick(inp.w1_global_scale),
                pick(inp.w2_fp4), pick(inp.w2_blockscale), pick(inp.w2_global_scale), pick(inp.a1_gscale),
                pick(inp.a2_gscale), torch.tensor(local, dtype=torch.int32).reshape(n, 1), torch.ones(n, 1), taps=taps)
    codes_ok = True
    if taps.act_codes is not None:
        codes_ok = bool(torch.equal(b.packed_input.index_select(0, pos_d).cpu(), taps.act_codes))
    ref = taps.routed
    rms = ref.square().mean().sqrt().item()
    ratio = (got - ref).abs().max().item() / max(rms, 1e-30)
    res.update(experts=len(chosen), rows=n, codes_ok=codes_ok, max_abs_over_rms=ratio,
               ok=bool(perm_ok and codes_ok and ratio <= tolerance))
    return res


def combine_matches(binding, topk_weights: torch.Tensor, out_bf16: torch.Tensor, tokens: int = 128) -> bool:
    """The weighted combine of the first ``tokens`` tokens, recomputed on the CPU from the fp32 FC2
    rows the kernels left behind (products and sums in slot order, one bf16 rounding): bit-equal."""
    b = binding
    t = min(tokens, b.tokens)
    k = b.num_topk
    inv = b.inv_perm[: t * k].to(torch.int64)
    rows = b.route_output.index_select(0, inv.clamp(min=0)).cpu().reshape(t, k, -1)
    ok = (inv >= 0).cpu().reshape(t, k, 1)
    w = topk_weights[:t].cpu().float().reshape(t, k, 1)
    acc = torch.zeros(t, rows.shape[-1])
    for s in range(k):
        acc = acc + torch.where(ok[:, s], rows[:, s] * w[:, s], torch.zeros_like(rows[:, s]))
    return bool(torch.equal(acc.to(torch.bfloat16), out_bf16[:t].cpu()))
