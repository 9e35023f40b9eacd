"""Tensor-free vocabulary of the MoE planner: recipes, source formats, the weight plan.

Mirrors the part of the reference's ``b12x/moe/_shared/execution.py`` that the fused_moe facade
exposes (``MoESpec`` :199-259, ``MoEWeightPreparationPlan`` :262-575, source/recipe validation
:157-196, activation metadata ``kernels/activations.py:8-85``).  No torch import: planning code
must be usable without a device.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from enum import Enum

SWIGLUOAI = "swigluoai_uninterleave"
SUPPORTED_ACTIVATIONS = frozenset({"silu", "relu2", SWIGLUOAI})
GATED_ACTIVATIONS = frozenset({"silu", SWIGLUOAI})
# "situ" is part of the reference's activation set; it is not built here.
KNOWN_UNBUILT_ACTIVATIONS = frozenset({"situ"})

QUANT_MODES = frozenset({"nvfp4", "w4a16", "w4a8_mx"})
SOURCE_FORMATS = frozenset({"modelopt_nvfp4", "fp4_e8m0_k32", "compressed_tensors"})
SOURCES_BY_QUANT_MODE = {
    "nvfp4": frozenset({"modelopt_nvfp4"}),
    "w4a8_mx": frozenset({"fp4_e8m0_k32"}),
    "w4a16": frozenset({"modelopt_nvfp4", "fp4_e8m0_k32", "compressed_tensors"}),
}


class WeightStoragePolicy(str, Enum):
    KEEP_SOURCE = "keep_source"        # source tensors are the runtime storage
    TRANSFER_SOURCE = "transfer_source"


class WeightPreparationTransform(str, Enum):
    RUNTIME_ALPHAS = "runtime_alphas"          # alphas = weight global scale / input gscale
    SWIZZLE_MX_SCALES = "swizzle_mx_scales"    # plain E8M0 grids -> 128x4 atoms for tcgen05
    EXPAND_E8M0_K32 = "expand_e8m0_k32"        # w4a16: plain E8M0 K/32 grids -> per-16 atoms
    INVERT_GLOBAL_SCALES = "invert_global_scales"  # compressed-tensors stores 1 / global scale


def normalize_moe_activation(activation: str) -> str:
    activation = str(activation)
    if activation in KNOWN_UNBUILT_ACTIVATIONS:
        raise NotImplementedError(f"activation {activation!r} is not built in this library")
    if activation not in SUPPORTED_ACTIVATIONS:
        raise ValueError(f"unsupported activation {activation!r}")
    return activation


def is_gated_moe_activation(activation: str) -> bool:
    return normalize_moe_activation(activation) in GATED_ACTIVATIONS


def moe_activation_w1_rows(activation: str, n: int) -> int:
    return (2 if is_gated_moe_activation(activation) else 1) * int(n)


def normalize_swiglu_params(activation, limit, alpha, beta):
    """Defaults and validation of the SwiGLU knobs (kernels/activations.py:36-85)."""
    activation = normalize_moe_activation(activation)
    if limit is None:
        limit = 7.0 if activation == SWIGLUOAI else None
    else:
        if activation not in GATED_ACTIVATIONS:
            raise ValueError("swiglu_limit requires a gated MoE activation")
        limit = float(limit)
        if not math.isfinite(limit) or limit <= 0.0:
            raise ValueError(f"swiglu_limit must be positive and finite, got {limit}")
    if activation != SWIGLUOAI:
        if alpha is not None and float(alpha) != 1.0:
            raise ValueError("swiglu_alpha is only configurable for swigluoai_uninterleave")
        if beta is not None and float(beta) != 0.0:
            raise ValueError("swiglu_beta is only configurable for swigluoai_uninterleave")
        return limit, 1.0, 0.0
    alpha = 1.702 if alpha is None else float(alpha)
    beta = 1.0 if beta is None else float(beta)
    if not math.isfinite(alpha) or not math.isfinite(beta):
        raise ValueError("swiglu_alpha and swiglu_beta must be finite")
    return limit, alpha, beta


def validate_moe_source_quant(*, source_format: str, quant_mode: str) -> None:
    quant_mode = str(quant_mode).lower()
    source_format = str(source_format).lower()
    if quant_mode not in QUANT_MODES:
        raise ValueError(f"unsupported quant_mode {quant_mode!r}")
    if source_format not in SOURCE_FORMATS:
        raise ValueError(f"unsupported source_format {source_format!r}")
    if source_format not in SOURCES_BY_QUANT_MODE[quant_mode]:
        raise ValueError(
            f"source_format={source_format!r} is incompatible with quant_mode={quant_mode!r}")


def normalize_w13_layout(activation: str, w13_layout: str) -> str:
    """"w13" = FC1 rows [up; gate]; "w31" / "gate_up" = [gate; up].  SwiGLU-OAI is always
    gate-first (reference _impl.py:1396-1401)."""
    layout = str(w13_layout).lower()
    if layout == "gate_up":
        layout = "w31"
    if layout not in {"w13", "w31"}:
        raise ValueError(f"unsupported W13 layout {w13_layout!r}")
    if activation == SWIGLUOAI:
        return "w31"
    return layout


@dataclass(frozen=True, kw_only=True)
class MoESpec:
    quant_mode: str
    source_format: str
    activation: str
    io_dtype: str
    w13_layout: str = "w13"

    def __post_init__(self) -> None:
        validate_moe_source_quant(source_format=self.source_format, quant_mode=self.quant_mode)
        if self.io_dtype not in {"bfloat16"}:
            raise TypeError(f"unsupported MoE io dtype {self.io_dtype!r} (bfloat16 only)")

    @property
    def activation_block(self) -> int | None:
        return {"nvfp4": 16, "w4a8_mx": 32, "w4a16": None}[self.quant_mode]

    @property
    def weight_block(self) -> int:
        return 32 if self.source_format == "fp4_e8m0_k32" else 16


def make_moe_spec(*, quant_mode, source_format, activation, io_dtype, w13_layout="w13") -> MoESpec:
    activation = normalize_moe_activation(activation)
    return MoESpec(quant_mode=str(quant_mode).lower(), source_format=str(source_format).lower(),
                   activation=activation, io_dtype=str(io_dtype),
                   w13_layout=normalize_w13_layout(activation, w13_layout))


@dataclass(frozen=True, kw_only=True)
class MoEWeightPreparationPlan:
    """Load-time plan: which recipes run on which single weight allocation."""

    specs: tuple[MoESpec, ...]
    num_experts: int
    hidden_size: int
    intermediate_size: int
    transforms: frozenset
    storage_policy: WeightStoragePolicy

    def __post_init__(self) -> None:
        specs = tuple(self.specs)
        if not specs:
            raise ValueError("weight preparation requires at least one MoE spec")
        object.__setattr__(self, "specs", specs)
        for name in ("num_experts", "hidden_size", "intermediate_size"):
            value = int(getattr(self, name))
            if value <= 0:
                raise ValueError(f"{name} must be positive, got {value}")
            object.__setattr__(self, name, value)
        first = specs[0]
        for spec in specs[1:]:
            if (spec.source_format, spec.activation, spec.io_dtype, spec.w13_layout) != (
                    first.source_format, first.activation, first.io_dtype, first.w13_layout):
                raise ValueError("all recipes of one weight plan must share source, activation and dtype")
        object.__setattr__(self, "transforms", frozenset(self.transforms))

    @property
    def quant_modes(self) -> frozenset:
        return frozenset(spec.quant_mode for spec in self.specs)

    @property
    def source_format(self) -> str:
        return self.specs[0].source_format

    @property
    def activation(self) -> str:
        return self.specs[0].activation

    @property
    def io_dtype(self) -> str:
        return self.specs[0].io_dtype

    @property
    def w13_layout(self) -> str:
        return self.specs[0].w13_layout

    @property
    def w1_rows(self) -> int:
        return moe_activation_w1_rows(self.activation, self.intermediate_size)


def plan_moe_weight_preparation(specs, *, num_experts, hidden_size, intermediate_size) -> MoEWeightPreparationPlan:
    """Shape checks per recipe and the list of load-time transforms (reference :718-980)."""
    specs = tuple(specs)
    transforms = set()
    k, n = int(hidden_size), int(intermediate_size)
    for spec in specs:
        if spec.quant_mode == "nvfp4":
            if k % 64 != 0 or n % 64 != 0:
                raise ValueError("nvfp4 requires hidden_size and intermediate_size divisible by 64")
            transforms.add(WeightPreparationTransform.RUNTIME_ALPHAS)
        elif spec.quant_mode == "w4a8_mx":
            if k % 32 != 0 or n % 32 != 0:
                raise ValueError("w4a8_mx requires hidden_size and intermediate_size divisible by 32")
            transforms.add(WeightPreparationTransform.SWIZZLE_MX_SCALES)
        elif spec.quant_mode == "w4a16":
            if k % 64 != 0 or n % 64 != 0:
                raise ValueError("w4a16 requires hidden_size and intermediate_size divisible by 64")
            if spec.source_format == "fp4_e8m0_k32":
                transforms.add(WeightPreparationTransform.EXPAND_E8M0_K32)
            elif spec.source_format == "compressed_tensors":
                transforms.add(WeightPreparationTransform.INVERT_GLOBAL_SCALES)
    both = {WeightPreparationTransform.SWIZZLE_MX_SCALES, WeightPreparationTransform.EXPAND_E8M0_K32}
    if both <= transforms:
        raise ValueError("one weight plan cannot serve both w4a8_mx and w4a16: they need different "
                         "block-scale layouts")
    policy = (WeightStoragePolicy.TRANSFER_SOURCE if transforms & both
              else WeightStoragePolicy.KEEP_SOURCE)
    return MoEWeightPreparationPlan(specs=specs, num_experts=num_experts, hidden_size=k,
                                    intermediate_size=n, transforms=frozenset(transforms),
                                    storage_policy=policy)
