"""Run the CUDA layer through the public facade (and so through the C ABI) and hand back the
stage taps next to the oracle's, for the ``-m gpu`` parity tests."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from b12x_b200 import synth
from b12x_b200.moe import fused_moe
from oracle import moe_oracle as O

ACT_API = {"silu": "silu", "relu2": "relu2", "swigluoai": "swigluoai_uninterleave"}
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
              max_tokens=None, w13_layout="w13", want_fc1=True, tile_rows=None) -> LayerRun:
    dev = torch.device("cuda")
    shp = inp.shape
    ex = prepare_experts(inp, dev, w13_layout=w13_layout)
    t = inp.x.shape[0]
    caps = fused_moe.Caps(max_tokens=max_tokens or max(t, 1), num_topk=shp.topk, device=dev,
                          weight_plan=ex.plan, quant_mode=shp.recipe, tile_rows=tile_rows)
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


def oracle_layer(inp: synth.MoEInputs, ids, weights, expert_map=None):
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
                          expert_map=expert_map, taps=taps)
    else:
        ones = torch.ones(inp.w1_fp4.shape[0])
        out = O.moe_w4a8_mx(inp.x, inp.w1_fp4, inp.w1_blockscale, ones, inp.w2_fp4, inp.w2_blockscale, ones,
                            ids, weights, activation=shp.activation, expert_map=expert_map, taps=taps)
    return out, taps
