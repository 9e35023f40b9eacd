"""Generate ``quant_ops.npz``: the standalone activation quantisers of the REFERENCE library
(b12x 1.2.6, torch implementations) on seeded inputs.

    python tests/golden/make_golden_quant.py /path/to/b12x

* NVFP4: ``quantize_grouped_nvfp4_torch`` (b12x/_lib/intrinsics.py:149-193), the oracle the
  reference's own test of ``quantization.nvfp4`` compares with (tests/quantization/test_nvfp4.py);
  scale bytes are stored in the physical order that test recovers.
* MXFP8: ``quantize_grouped_mxfp8_torch`` (b12x/_lib/intrinsics.py:268-312).
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().copy()


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from b12x._lib import intrinsics as RI

    g = torch.Generator().manual_seed(20260720)
    m, k = 256, 256
    x = (torch.randn((m, k), generator=g) / 4).to(torch.bfloat16)
    x[3, 16:32] = 0                                   # an all-zero block
    x[7, 0] = 3.0                                     # a block dominated by one value
    gs = (448.0 * 6.0 / x.float().abs().max()).reshape(1)
    packed, scale_view = RI.quantize_grouped_nvfp4_torch(x.unsqueeze(0), torch.tensor([m], dtype=torch.int32), gs)
    nv_codes = packed.contiguous().view(torch.uint8).reshape(m, k // 2)
    nv_scales = scale_view.permute(5, 2, 4, 0, 1, 3).contiguous().view(torch.uint8).reshape(-1)

    x2 = (torch.randn((133, 160), generator=g) * 2).to(torch.bfloat16)
    x2[5, 32:64] = 0
    payload, mx_view = RI.quantize_grouped_mxfp8_torch(x2.unsqueeze(0), torch.tensor([133], dtype=torch.int32))
    mx_codes = payload.view(torch.uint8).reshape(133, 160)
    mx_swz = mx_view.permute(5, 2, 4, 0, 1, 3).contiguous().view(torch.uint8).reshape(-1)
    blocked = x2.float().reshape(133, 5, 32)
    _, byte = RI.pow2_ceil_ue8m0_torch(blocked.abs().amax(dim=-1) * (1.0 / 448.0))

    np.savez_compressed(HERE / "quant_ops.npz", nv_x=bits(x), nv_gs=gs.numpy(), nv_codes=nv_codes.numpy(),
                        nv_scales=nv_scales.numpy(), mx_x=bits(x2), mx_codes=mx_codes.numpy(),
                        mx_scale_rows=byte.numpy(), mx_scale_mma=mx_swz.numpy())
    print("quant_ops.npz", (HERE / "quant_ops.npz").stat().st_size)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden_quant.py /path/to/b12x")
    main(sys.argv[1])
