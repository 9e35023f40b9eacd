"""Generate ``routing_gate.npz`` and ``tiny_nvfp4_situ.npz`` by running the REFERENCE library
(b12x 1.2.6) on seeded inputs.

    python tests/golden/make_golden_routing.py /path/to/b12x

* sigmoid router of the DeepSeek-V3-shaped benchmark: outputs of the reference's own
  ``compute_model_gate_routing`` (benchmarks/benchmark_moe.py:1282-1322) for a gate matrix,
  a selection bias, renormalisation and a route scale of 2.5;
* gate projection + top-k of ``b12x_route_experts_fast`` on CPU tensors
  (b12x/moe/fused_moe/_impl.py:11356-11490 -> ``_select_experts_reference``): fp32 and bf16
  operands, with and without bias, with and without renormalisation;
* the ``situ`` activation through ``moe_reference_nvfp4`` (b12x/moe/_shared/kernels/reference.py:160-172).
"""

from __future__ import annotations

import sys
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parents[1]


def npy(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu()
    return t.view(torch.int16).numpy() if t.dtype == torch.bfloat16 else t.numpy()


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    sys.path.insert(0, str(REPO))
    torch.set_num_threads(8)
    from b12x.moe._shared.kernels import reference as R
    from b12x.moe.fused_moe._impl import (_select_experts_reference, b12x_route_experts_fast,
                                          build_tp_moe_route_binding)
    from benchmarks.benchmark_moe import compute_model_gate_routing

    from b12x_b200 import synth

    g = torch.Generator().manual_seed(11)
    out = {}
    # ---- sigmoid router through the reference benchmark's own function
    t, k, e, topk = 24, 64, 32, 4
    x = torch.randn(t, k, generator=g)
    gw = torch.randn(e, k, generator=g) * 0.3
    bias = torch.randn(e, generator=g) * 0.1
    w = SimpleNamespace(gate_weight=gw, gate_score_func="sigmoid", gate_tid2eid=None, gate_bias=bias,
                        spec=SimpleNamespace(top_k=topk), gate_norm_topk_prob=True, gate_route_scale=2.5)
    ids, wts = compute_model_gate_routing(w, x, seed=0)
    out.update(sig_x=npy(x), sig_gate=npy(gw), sig_bias=npy(bias), sig_ids=npy(ids.to(torch.int32)),
               sig_weights=npy(wts.float()), sig_scores_logits=npy(torch.nn.functional.linear(x, gw)))
    # ---- gate projection + top-k (softmax over the selected logits / raw logits)
    for tag, dt in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        hs = torch.randn(20, 96, generator=g).to(dt)
        gate = (torch.randn(48, 96, generator=g) * 0.25).to(dt)
        gb = (torch.randn(48, generator=g) * 0.5).to(dt)
        for btag, b in (("", None), ("_bias", gb)):
            for rtag, renorm in (("", True), ("_raw", False)):
                rb = build_tp_moe_route_binding(hidden_states=hs, top_k=6, gate_weight=gate, gate_bias=b,
                                                renormalize=renorm)
                r = b12x_route_experts_fast(binding=rb)
                key = f"gate_{tag}{btag}{rtag}"
                out[key + "_ids"] = npy(r.topk_ids.to(torch.int32))
                out[key + "_weights"] = npy(r.topk_weights.float())
                out[key + "_logits"] = npy(r.router_logits)
        out[f"gate_{tag}_hidden"], out[f"gate_{tag}_weight"], out[f"gate_{tag}_gbias"] = npy(hs), npy(gate), npy(gb)
    np.savez_compressed(HERE / "routing_gate.npz", **out)

    # ---- situ activation, NVFP4, all inputs stored
    shp = synth.shape("c1", name="tiny_situ", tokens=8, hidden=256, intermediate=128, experts=4)
    inp = synth.make_inputs(shp, seed=6)
    a1 = (inp.w1_global_scale / inp.a1_gscale).contiguous()
    a2 = (inp.w2_global_scale / inp.a2_gscale).contiguous()
    routing = _select_experts_reference(inp.x.float(), top_k=shp.topk, router_logits=inp.router_logits,
                                        renormalize=True)
    ids, tw = routing.topk_ids.to(torch.int32), routing.topk_weights.float()
    e, k, i = shp.experts, shp.hidden, shp.intermediate
    res = R.moe_reference_nvfp4(inp.x, inp.w1_fp4, inp.w1_blockscale, a1, inp.w2_fp4, inp.w2_blockscale, a2,
                                inp.a1_gscale, inp.a2_gscale, ids, tw, e, k, i, activation="situ")
    tt, topk = ids.shape
    mid = torch.zeros(tt, topk, i)
    acc = torch.zeros(tt, topk, k)
    for ti in range(tt):
        for s in range(topk):
            tr = R.trace_moe_reference_nvfp4_route(
                inp.x, inp.w1_fp4, inp.w1_blockscale, a1, inp.w2_fp4, inp.w2_blockscale, a2, inp.a1_gscale,
                inp.a2_gscale, ids, tw, e, k, i, token_idx=ti, route_idx=s, activation="situ")
            mid[ti, s] = tr.intermediate
            acc[ti, s] = tr.routed_out_accum
    d = dict(topk_ids=npy(ids), topk_weights=npy(tw), out_bf16=npy(res), out_f32=npy(acc.sum(dim=1)), mid=npy(mid),
             routed_accum=npy(acc))
    for n in ("x", "router_logits", "w1_fp4", "w1_blockscale", "w2_fp4", "w2_blockscale", "a1_gscale",
              "a2_gscale", "w1_global_scale", "w2_global_scale"):
        d["in_" + n] = npy(getattr(inp, n))
    np.savez_compressed(HERE / "tiny_nvfp4_situ.npz", **d)
    for f in ("routing_gate.npz", "tiny_nvfp4_situ.npz"):
        print(f, (HERE / f).stat().st_size)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden_routing.py /path/to/b12x")
    main(sys.argv[1])
