"""Generate the golden fixtures in this directory by running the REFERENCE library's own torch
oracle (b12x 1.2.6) on seeded inputs.

Usage (only where a checkout of the reference is available):

    python tests/golden/make_golden.py /path/to/b12x

The fixtures are small ``.npz`` files; tests read them and never need the reference.  Inputs of
the small cases are stored in full; the 16-token NVFP4 case (hidden 1024, 8 experts) stores a
SHA-256 of every input instead, and tests regenerate the inputs with ``b12x_b200.synth``.
"""

from __future__ import annotations

import hashlib
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parents[1]


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.detach().cpu().contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def npy(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy()
    return t.numpy()


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    sys.path.insert(0, str(REPO))
    torch.set_num_threads(8)
    from b12x._lib import intrinsics as RI
    from b12x.moe._shared.kernels import reference as R
    from b12x.moe.fused_moe._impl import _select_experts_reference
    from tests._reference import w4a16_reference as W

    from b12x_b200 import synth

    def prep(shp, seed):
        inp = synth.make_inputs(shp, seed=seed)
        a1 = (inp.w1_global_scale / inp.a1_gscale).contiguous()
        a2 = (inp.w2_global_scale / inp.a2_gscale).contiguous()
        routing = _select_experts_reference(inp.x.float(), top_k=shp.topk,
                                            router_logits=inp.router_logits, renormalize=True)
        ids = routing.topk_ids.to(torch.int32)
        return inp, a1, a2, ids, routing.topk_weights.float()

    def nvfp4_case(shp, seed, activation_ref, store_inputs):
        inp, a1, a2, ids, tw = prep(shp, seed)
        e, k, i = shp.experts, shp.hidden, shp.intermediate
        out = R.moe_reference_nvfp4(inp.x, inp.w1_fp4, inp.w1_blockscale, a1, inp.w2_fp4,
                                    inp.w2_blockscale, a2, inp.a1_gscale, inp.a2_gscale, ids, tw,
                                    e, k, i, activation=activation_ref)
        t, topk = ids.shape
        w1_rows = inp.w1_fp4.shape[1]
        fc1 = torch.zeros(t, topk, w1_rows)
        mid = torch.zeros(t, topk, i)
        xdq = torch.zeros(t, topk, k)
        mdq = torch.zeros(t, topk, i)
        acc = torch.zeros(t, topk, k)
        for ti in range(t):
            for s in range(topk):
                tr = R.trace_moe_reference_nvfp4_route(
                    inp.x, inp.w1_fp4, inp.w1_blockscale, a1, inp.w2_fp4, inp.w2_blockscale, a2,
                    inp.a1_gscale, inp.a2_gscale, ids, tw, e, k, i, token_idx=ti, route_idx=s,
                    activation=activation_ref)
                g_rows, u_rows = R._gated_row_slices(activation_ref, i)
                fc1[ti, s, g_rows] = tr.gate_out
                fc1[ti, s, u_rows] = tr.up_out
                mid[ti, s] = tr.intermediate
                xdq[ti, s] = tr.x_dequant
                mdq[ti, s] = tr.int_dequant
                acc[ti, s] = tr.routed_out_accum
        out_f32 = torch.zeros(t, k)
        for s in range(topk):
            out_f32 += acc[:, s]
        d = dict(topk_ids=npy(ids), topk_weights=npy(tw), out_bf16=npy(out), out_f32=npy(out_f32),
                 fc1=npy(fc1), mid=npy(mid), x_dequant=npy(xdq), mid_dequant=npy(mdq),
                 routed_accum=npy(acc), w1_alphas=npy(a1), w2_alphas=npy(a2))
        names = ("x", "router_logits", "w1_fp4", "w1_blockscale", "w2_fp4", "w2_blockscale",
                 "a1_gscale", "a2_gscale", "w1_global_scale", "w2_global_scale")
        for n in names:
            d["sha_" + n] = np.array(sha(getattr(inp, n)))
            if store_inputs:
                d["in_" + n] = npy(getattr(inp, n))
        return d

    # 1. benchmark config 1: 16 tokens, hidden 1024, I 512, 8 experts, top-2, NVFP4, SwiGLU, seed 0
    np.savez_compressed(HERE / "c1_nvfp4_silu.npz", **nvfp4_case(synth.shape("c1"), 0, "silu", False))

    # 2. small SwiGLU-OAI NVFP4 case with all inputs stored
    tiny = synth.shape("c1", name="tiny", tokens=8, hidden=256, intermediate=128, experts=4)
    np.savez_compressed(HERE / "tiny_nvfp4_swigluoai.npz",
                        **nvfp4_case(synth.shape("c1", name="tiny_oai", tokens=8, hidden=256,
                                                 intermediate=128, experts=4, activation="swigluoai"),
                                     1, "swigluoai_uninterleave", True))
    np.savez_compressed(HERE / "tiny_nvfp4_silu.npz", **nvfp4_case(tiny, 2, "silu", True))

    # 3. the reference's own bit-exact kernel-vs-oracle case generator (E=1, K=N=128, relu2)
    from tests.moe.test_tp_moe_relu2_reference import _make_activation_case
    (x, ids, tw, w1, s1, al1, w2, s2, al2, g1, g2, e, k, n) = _make_activation_case(
        device=torch.device("cpu"), activation="relu2", m=16)
    out = R.moe_reference_nvfp4(x, w1, s1, al1, w2, s2, al2, g1, g2, ids, tw, e, k, n, activation="relu2")
    np.savez_compressed(HERE / "relu2_e1_k128.npz", x=npy(x), topk_ids=npy(ids), topk_weights=npy(tw),
                        w1_fp4=npy(w1), w1_blockscale=npy(s1.view(torch.uint8)), w1_alphas=npy(al1),
                        w2_fp4=npy(w2), w2_blockscale=npy(s2.view(torch.uint8)), w2_alphas=npy(al2),
                        a1_gscale=npy(g1), a2_gscale=npy(g2), out_bf16=npy(out))

    # 4. W4A16 small case (weights rounded to bf16, bf16 intermediate)
    shp = synth.shape("c3", name="tiny_w4a16", tokens=8, hidden=256, intermediate=128, experts=4, topk=2)
    inp, _, _, ids, tw = prep(shp, 3)
    al1, al2 = inp.w1_global_scale, inp.w2_global_scale
    out = W.moe_reference_w4a16(inp.x, inp.w1_fp4, inp.w1_blockscale, al1, inp.w2_fp4, inp.w2_blockscale,
                                al2, ids, tw, shp.experts, shp.hidden, shp.intermediate, activation="silu")
    t, topk = ids.shape
    fc1 = torch.zeros(t, topk, 2 * shp.intermediate)
    mid = torch.zeros(t, topk, shp.intermediate)
    down = torch.zeros(t, topk, shp.hidden)
    for ti in range(t):
        for s in range(topk):
            tr = W.trace_moe_reference_w4a16_route(
                inp.x, inp.w1_fp4, inp.w1_blockscale, al1, inp.w2_fp4, inp.w2_blockscale, al2, ids, tw,
                shp.experts, shp.hidden, shp.intermediate, token_idx=ti, route_idx=s, activation="silu")
            fc1[ti, s, : shp.intermediate] = tr.up_out
            fc1[ti, s, shp.intermediate:] = tr.gate_out
            mid[ti, s] = tr.intermediate
            down[ti, s] = tr.down_out.float()
    np.savez_compressed(HERE / "tiny_w4a16.npz", x=npy(inp.x), router_logits=npy(inp.router_logits),
                        topk_ids=npy(ids), topk_weights=npy(tw), w1_fp4=npy(inp.w1_fp4),
                        w1_blockscale=npy(inp.w1_blockscale), w1_alphas=npy(al1), w2_fp4=npy(inp.w2_fp4),
                        w2_blockscale=npy(inp.w2_blockscale), w2_alphas=npy(al2), out_bf16=npy(out),
                        fc1=npy(fc1), mid=npy(mid), down_bf16_as_f32=npy(down))

    # 5. w4a8_mx small case (MXFP4 source, silu; the reference rejects SwiGLU-OAI here)
    shp = synth.shape("c5", name="tiny_mx", tokens=8, hidden=256, intermediate=128, experts=4, topk=2,
                      activation="silu")
    inp, _, _, ids, tw = prep(shp, 4)
    ones = torch.ones(shp.experts)
    out = R.moe_reference_w4a8_mx(inp.x, inp.w1_fp4, inp.w1_blockscale, None, ones, inp.w2_fp4,
                                  inp.w2_blockscale, None, ones, ids, tw, shp.experts, shp.hidden,
                                  shp.intermediate, activation="silu")
    np.savez_compressed(HERE / "tiny_w4a8_mx.npz", x=npy(inp.x), router_logits=npy(inp.router_logits),
                        topk_ids=npy(ids), topk_weights=npy(tw), w1_fp4=npy(inp.w1_fp4),
                        w1_e8m0=npy(inp.w1_blockscale), w2_fp4=npy(inp.w2_fp4),
                        w2_e8m0=npy(inp.w2_blockscale), out_f32=npy(out))

    # 6. primitives
    g = torch.Generator().manual_seed(5)
    sc = torch.randint(0, 256, (2, 200, 14), generator=g, dtype=torch.uint8)
    sw = RI.swizzle_block_scale(sc)
    ties = torch.tensor([0.0, 0.2, 0.25, 0.26, 0.5, 0.74, 0.75, 1.0, 1.25, 1.26, 1.5, 1.74, 1.75, 2.0,
                         2.5, 2.51, 3.0, 3.49, 3.5, 4.0, 5.0, 5.01, 6.0, 7.5, -0.25, -0.75, -2.5, -5.0, -9.0])
    scales = torch.tensor([0.0, 1.0, 1.0000001, 0.75, 2.0 ** -20, 3.1e-5, 448.0, 0.0022321429, 1e-38])
    r_f, r_b = RI.pow2_ceil_ue8m0_torch(scales)
    xs = torch.randn(6, 128, generator=g) * torch.tensor([1.0, 1e-3, 50.0, 0.0, 3e4, 1e-30]).unsqueeze(1)
    qd = RI.quant_dequant_mxfp8_torch(xs)
    rows = torch.randn(5, 64, generator=g) * 3.0
    deq = torch.stack([R._quantize_vec_to_fp4_dequant(rows[j], 37.5, block_size=16, fp8_e4m3_max=448.0)
                       for j in range(rows.shape[0])])
    # routing known answers (tests/moe/test_sparse_moe_api.py:152-236)
    lg = torch.randn(12, 24, generator=g)
    rt = _select_experts_reference(lg, top_k=4, router_logits=lg, renormalize=True)
    rt_raw = _select_experts_reference(lg, top_k=4, router_logits=lg, renormalize=False)
    # sigmoid scoring as in benchmarks/benchmark_moe.py:1289-1321
    bias = torch.randn(24, generator=g) * 0.1
    scores = torch.sigmoid(lg)
    _, sid = torch.topk(scores + bias, 4, dim=-1)
    sw_ = scores.gather(1, sid)
    sw_ = sw_ / sw_.sum(dim=-1, keepdim=True).clamp_min(1e-20) * 2.5
    np.savez_compressed(
        HERE / "primitives.npz", scale_grid=npy(sc), scale_swizzled=npy(sw), fp4_in=npy(ties),
        fp4_out=npy(RI.fp4_quantize_values_torch(ties)), ue8m0_in=npy(scales), ue8m0_rounded=npy(r_f),
        ue8m0_byte=npy(r_b), mxfp8_in=npy(xs), mxfp8_qdq=npy(qd), nvfp4_rows=npy(rows),
        nvfp4_rows_gs=np.array(37.5, dtype=np.float32), nvfp4_rows_dequant=npy(deq), route_logits=npy(lg),
        route_ids=npy(rt.topk_ids.to(torch.int32)), route_weights=npy(rt.topk_weights),
        route_raw_ids=npy(rt_raw.topk_ids.to(torch.int32)), route_raw_weights=npy(rt_raw.topk_weights),
        sig_bias=npy(bias), sig_ids=npy(sid.to(torch.int32)), sig_weights=npy(sw_))
    for f in sorted(HERE.glob("*.npz")):
        print(f.name, f.stat().st_size)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/b12x")
    main(sys.argv[1])
