"""Public surface of quantization.nvfp4 (reference ``b12x/quantization/nvfp4/api.py:24-62`` and
``_impl.py:74-114`` for the output container)."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..._lib import ext

_TILE = 128


@dataclass(frozen=True)
class Plan:
    """A planned (m, k) shape; produced by :func:`plan`."""

    m: int
    k: int


@dataclass
class Outputs:
    """``packed_a_storage`` u8 ``[1, M, K/2]`` (two E2M1 per byte, low nibble = even k) and
    ``scale_storage`` u8 ``[pad128(M) * pad4(K/16)]`` (E4M3 bytes, 128x4-swizzled)."""

    packed_a_storage: torch.Tensor
    scale_storage: torch.Tensor

    @property
    def packed_a_flat(self) -> torch.Tensor:
        return self.packed_a_storage.view(-1)

    @property
    def scale_flat(self) -> torch.Tensor:
        return self.scale_storage.view(-1)


def _validate(m: int, k: int) -> None:
    if m <= 0 or k <= 0:
        raise ValueError(f"M and K must be positive, got M={m}, K={k}")
    if m % _TILE or k % _TILE:
        raise ValueError(f"M and K must be multiples of ({_TILE}, {_TILE}), got M={m}, K={k}")


def plan(m: int, k: int) -> Plan:
    """Fix the quantiser's shape (nothing is compiled here: the kernel takes the shape at launch)."""
    _validate(int(m), int(k))
    return Plan(m=int(m), k=int(k))


def allocate_outputs(plan: Plan, *, device: torch.device | str = "cuda") -> Outputs:
    """Allocate the packed-FP4 + MMA-layout-scale output pair for a plan."""
    _validate(plan.m, plan.k)
    dev = torch.device(device)
    return Outputs(
        packed_a_storage=torch.zeros(1, plan.m, plan.k // 2, dtype=torch.uint8, device=dev),
        scale_storage=torch.zeros(plan.m * (plan.k // 16), dtype=torch.uint8, device=dev))


def run(*, plan: Plan, x: torch.Tensor, global_scale: torch.Tensor, outputs: Outputs) -> None:
    """Quantise ``x`` into ``outputs`` on the current stream (allocation-free, capture safe)."""
    if not isinstance(plan, Plan) or not isinstance(outputs, Outputs):
        raise TypeError("plan / outputs must come from plan() / allocate_outputs()")
    if x.dtype != torch.bfloat16:
        raise ValueError(f"x must have dtype torch.bfloat16, got {x.dtype}")
    if tuple(x.shape) != (plan.m, plan.k) or x.stride(1) != 1:
        raise ValueError(f"x must be a row-contiguous [{plan.m}, {plan.k}] tensor")
    if x.device.type != "cuda":
        raise RuntimeError("quantization.nvfp4 runs on CUDA devices only; there is no CPU path")
    if global_scale.dtype != torch.float32 or global_scale.numel() != 1 or global_scale.device != x.device:
        raise ValueError("global_scale must be one float32 value on x's device")
    if (outputs.packed_a_storage.numel() != plan.m * plan.k // 2
            or outputs.scale_storage.numel() != plan.m * plan.k // 16
            or outputs.packed_a_storage.device != x.device or outputs.scale_storage.device != x.device):
        raise ValueError("outputs do not belong to this plan / device")
    stream = torch.cuda.current_stream(x.device).cuda_stream
    ext.check(ext.load().b200moe_quantize_rows_nvfp4(
        x.data_ptr(), x.stride(0), plan.m, plan.k, global_scale.data_ptr(),
        outputs.packed_a_storage.data_ptr(), outputs.scale_storage.data_ptr(), stream), "quantize_rows_nvfp4")


def is_supported(device=None) -> bool:
    """True on sm_100 (B200) with the extension built."""
    from ...moe import fused_moe

    return fused_moe.is_supported(device)
