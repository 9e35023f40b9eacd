"""Generate ``tiny_w4a16_e8m0.npz``: W4A16 over an ``fp4_e8m0_k32`` source (FP4 codes with plain
E8M0 per-32 block scales and a per-expert global scale), evaluated by the REFERENCE library's own
torch oracle ``moe_reference_w4a16_fp4_e8m0_k32`` (b12x 1.2.6,
b12x/moe/_shared/kernels/reference.py:789-935) on seeded inputs.

    python tests/golden/make_golden_w4a16_sources.py /path/to/b12x

That oracle computes in fp32 without the kernel's bf16 roundings (weights, intermediate); the
tests compare with the tolerance of the reference's own check (tests/moe/test_w4a16_e2e.py:676-765).
"""

from __future__ import annotations

import sys
from pathlib import Path

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
    from b12x.moe._shared.kernels import reference as R

    from b12x_b200 import synth

    out = {}
    for tag, act in (("silu", "silu"), ("relu2", "relu2")):
        shp = synth.shape("c5", name=f"tiny_w4a16_e8m0_{tag}", tokens=8, hidden=256, intermediate=128,
                          experts=4, topk=2, activation=act)
        inp = synth.make_inputs(shp, seed=11 if act == "silu" else 12)
        g = torch.Generator().manual_seed(13)
        ids = torch.stack([torch.randperm(shp.experts, generator=g)[: shp.topk] for _ in range(shp.tokens)])
        ids = ids.to(torch.int32)
        tw = torch.rand(shp.tokens, shp.topk, generator=g)
        g1 = 0.5 + torch.rand(shp.experts, generator=g)
        g2 = 0.5 + torch.rand(shp.experts, generator=g)
        ref = R.moe_reference_w4a16_fp4_e8m0_k32(
            inp.x, inp.w1_fp4, inp.w1_blockscale, g1, inp.w2_fp4, inp.w2_blockscale, g2, ids, tw,
            shp.experts, shp.hidden, shp.intermediate, activation=act, w13_layout="w13")
        for name, val in (("x", inp.x), ("w1_fp4", inp.w1_fp4), ("w1_e8m0", inp.w1_blockscale),
                          ("w2_fp4", inp.w2_fp4), ("w2_e8m0", inp.w2_blockscale), ("w1_global", g1),
                          ("w2_global", g2), ("topk_ids", ids), ("topk_weights", tw), ("out_f32", ref)):
            out[f"{tag}_{name}"] = npy(val)
    np.savez_compressed(HERE / "tiny_w4a16_e8m0.npz", **out)
    print("wrote", HERE / "tiny_w4a16_e8m0.npz")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden_w4a16_sources.py /path/to/b12x")
    main(sys.argv[1])
