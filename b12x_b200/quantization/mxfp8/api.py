"""Public surface of quantization.mxfp8."""

from __future__ import annotations

import torch

from ..._lib import ext


def quantize_rows(source: torch.Tensor, values: torch.Tensor, scale_rows: torch.Tensor,
                  scale_mma: torch.Tensor, *, value_order: str = "linear") -> None:
    """Quantise contiguous BF16 rows ``[M, K]`` (K a multiple of 32) into ``values`` ``[M, K]``
    (E4M3 bytes), ``scale_rows`` ``[M, K/32]`` and ``scale_mma`` (128x4-swizzled,
    ``pad128(M) * pad4(K/32)`` bytes; only the bytes of live rows are written, the caller
    pre-fills the padding).  Runs on the current stream; allocates nothing."""
    if value_order != "linear":
        raise NotImplementedError(f"value_order={value_order!r} is not built (only 'linear')")
    if source.dtype != torch.bfloat16:
        raise TypeError(f"the MXFP8 quantiser takes BF16 input, got {source.dtype}")
    if source.ndim != 2 or not source.is_contiguous():
        raise ValueError("the MXFP8 quantiser takes a contiguous [M, K] input")
    m, k = source.shape
    if k % 32:
        raise ValueError("K must be a multiple of 32")
    if source.device.type != "cuda":
        raise RuntimeError("quantization.mxfp8 runs on CUDA devices only; there is no CPU path")
    cols = k // 32
    pad = ((m + 127) // 128 * 128) * ((cols + 3) // 4 * 4)
    for name, t, n in (("values", values, m * k), ("scale_rows", scale_rows, m * cols), ("scale_mma", scale_mma, pad)):
        if t.element_size() != 1 or t.numel() != n or not t.is_contiguous() or t.device != source.device:
            raise ValueError(f"{name} must be a contiguous 1-byte tensor of {n} elements on the source's device")
    stream = torch.cuda.current_stream(source.device).cuda_stream
    ext.check(ext.load().b200moe_quantize_rows_mxfp8(
        source.data_ptr(), source.stride(0), m, k, values.data_ptr(), scale_rows.data_ptr(),
        scale_mma.data_ptr(), stream), "quantize_rows_mxfp8")


def is_supported(device=None) -> bool:
    """True on sm_100 (B200) with the extension built."""
    from ...moe import fused_moe

    return fused_moe.is_supported(device)
