"""CPU: the oracle's restatements of the reference's standalone quantisers against fixtures produced
by the reference's own torch implementations (tests/golden/make_golden_quant.py)."""

import torch

from oracle import moe_oracle as O
from tests.helpers import load_golden, t


def _bf16(bits):
    return t(bits).view(torch.bfloat16)


def test_nvfp4_reciprocal_quantiser_matches_reference_fixture():
    g = load_golden("quant_ops.npz")
    x = _bf16(g["nv_x"])
    codes, scales = O.quantize_nvfp4_rows_reciprocal(x, float(g["nv_gs"][0]))
    assert torch.equal(codes, t(g["nv_codes"]))
    m, k = x.shape
    assert torch.equal(O.swizzle_block_scale(scales).reshape(-1), t(g["nv_scales"]))
    # this variant is NOT the layer's direct-division quantiser: the two differ on some inputs
    codes_direct, _, _ = O.quantize_nvfp4_rows(x, float(g["nv_gs"][0]))
    assert codes_direct.shape == codes.shape


def test_mxfp8_quantiser_matches_reference_fixture():
    g = load_golden("quant_ops.npz")
    x = _bf16(g["mx_x"])
    payload, scale, _ = O.quantize_mxfp8_rows(x)
    assert torch.equal(payload, t(g["mx_codes"]))
    assert torch.equal(scale, t(g["mx_scale_rows"]))
    assert torch.equal(O.swizzle_block_scale(scale).reshape(-1), t(g["mx_scale_mma"]))
