"""CPU check of the arithmetic claim behind the W4A16 converter (csrc/grouped_gemm_other.cu): for every
E2M1 code and every finite E4M3 block scale the product is exactly representable in FP16 and in BF16, so
"convert to FP16, multiply in FP16, re-encode as BF16" equals the oracle's "dequantise, hold in BF16"
(tests/_reference/w4a16_reference.py:288-338 of the reference)."""

import torch

from oracle import moe_oracle


def _all_scales():
    b = torch.arange(256, dtype=torch.uint8)
    s = b.view(torch.float8_e4m3fn).float()
    return s[torch.isfinite(s)]


def test_code_times_e4m3_scale_is_exact_in_fp16_and_bf16():
    codes = moe_oracle.fp4_lut()                                           # 16 entries, sign in bit 3
    assert codes.numel() == 16 and torch.equal(codes[:8], torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]))
    assert torch.equal(codes[8:], -codes[:8])
    prod = codes[:, None].double() * _all_scales()[None, :].double()       # exact in f64
    assert torch.equal(prod.half().double(), prod), "FP16 would round a product"
    assert torch.equal(prod.bfloat16().double(), prod), "BF16 would round a product"
    nz = prod[prod != 0].abs()
    assert nz.min().item() >= 2.0 ** -14 and nz.max().item() <= 65504.0     # normal FP16 range
    # the FP16 multiply of the two FP16 factors gives the same value
    got = codes[:, None].half() * _all_scales()[None, :].half()
    assert torch.equal(got.double(), prod)
