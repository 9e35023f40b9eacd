"""-m gpu: the standalone quantiser operators (quantization.nvfp4 / quantization.mxfp8) through the
C ABI, bit for bit against the reference's fixtures and the CPU oracle."""

import pytest
import torch

from b12x_b200.quantization import mxfp8, nvfp4
from oracle import moe_oracle as O
from tests.helpers import load_golden, t

pytestmark = pytest.mark.gpu


def _bf16(bits):
    return t(bits).view(torch.bfloat16)


def test_nvfp4_op_matches_reference_fixture():
    g = load_golden("quant_ops.npz")
    x = _bf16(g["nv_x"]).cuda()
    m, k = x.shape
    plan = nvfp4.plan(m, k)
    outs = nvfp4.allocate_outputs(plan)
    nvfp4.run(plan=plan, x=x, global_scale=t(g["nv_gs"]).cuda(), outputs=outs)
    torch.cuda.synchronize()
    assert torch.equal(outs.packed_a_flat.cpu(), t(g["nv_codes"]).reshape(-1))
    assert torch.equal(outs.scale_flat.cpu(), t(g["nv_scales"]))


@pytest.mark.parametrize("m,k", [(128, 128), (384, 1024), (1024, 7168)])
def test_nvfp4_op_matches_oracle(m, k):
    gen = torch.Generator().manual_seed(m + k)
    x = (torch.randn(m, k, generator=gen) / 3).to(torch.bfloat16)
    gs = (448.0 * 6.0 / x.float().abs().max()).reshape(1)
    plan = nvfp4.plan(m, k)
    outs = nvfp4.allocate_outputs(plan)
    nvfp4.run(plan=plan, x=x.cuda(), global_scale=gs.cuda(), outputs=outs)
    torch.cuda.synchronize()
    codes, scales = O.quantize_nvfp4_rows_reciprocal(x, gs)
    assert torch.equal(outs.packed_a_storage.cpu().reshape(m, k // 2), codes)
    assert torch.equal(outs.scale_flat.cpu(), O.swizzle_block_scale(scales).reshape(-1))


def test_nvfp4_op_argument_errors():
    with pytest.raises(ValueError):
        nvfp4.plan(100, 128)
    plan = nvfp4.plan(128, 128)
    outs = nvfp4.allocate_outputs(plan)
    with pytest.raises(ValueError):
        nvfp4.run(plan=plan, x=torch.zeros(128, 128, device="cuda"), global_scale=torch.ones(1, device="cuda"),
                  outputs=outs)
    with pytest.raises(ValueError):
        nvfp4.run(plan=plan, x=torch.zeros(64, 128, dtype=torch.bfloat16, device="cuda"),
                  global_scale=torch.ones(1, device="cuda"), outputs=outs)


def _run_mxfp8(x):
    m, k = x.shape
    cols = k // 32
    values = torch.empty(m, k, dtype=torch.uint8, device="cuda")
    rows = torch.empty(m, cols, dtype=torch.uint8, device="cuda")
    pad = ((m + 127) // 128 * 128) * ((cols + 3) // 4 * 4)
    mma = torch.zeros(pad, dtype=torch.uint8, device="cuda")
    mxfp8.quantize_rows(x.cuda(), values, rows, mma)
    torch.cuda.synchronize()
    return values.cpu(), rows.cpu(), mma.cpu()


def test_mxfp8_op_matches_reference_fixture():
    g = load_golden("quant_ops.npz")
    values, rows, mma = _run_mxfp8(_bf16(g["mx_x"]))
    assert torch.equal(values, t(g["mx_codes"]))
    assert torch.equal(rows, t(g["mx_scale_rows"]))
    assert torch.equal(mma, t(g["mx_scale_mma"]))


@pytest.mark.parametrize("m,k", [(5, 256), (300, 2880), (64, 8192)])
def test_mxfp8_op_matches_oracle(m, k):
    gen = torch.Generator().manual_seed(m * 7 + k)
    x = (torch.randn(m, k, generator=gen) * 3).to(torch.bfloat16)
    values, rows, mma = _run_mxfp8(x)
    payload, scale, _ = O.quantize_mxfp8_rows(x)
    assert torch.equal(values, payload)
    assert torch.equal(rows, scale)
    assert torch.equal(mma, O.swizzle_block_scale(scale).reshape(-1))
