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
SITU = "situ"
SUPPORTED_ACTIVATIONS = frozenset({"silu", SITU, "relu2", SWIGLUOAI})
GATED_ACTIVATIONS = frozenset({"silu", SITU, SWIGLUOAI})

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
        if activation == SITU:
            raise ValueError("swiglu_limit is not part of the situ activation contract")
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
            if spec.activation == SITU:
                raise NotImplementedError("activation='situ' is not supported for W4A16 MoE")
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


# ---------------------------------------------------------------------------------------------
# execution lowering (reference ``MoEExecutionPlan`` :578-653 and ``lower_moe_execution`` :994-1118)
# ---------------------------------------------------------------------------------------------
class MoERegime(str, Enum):
    """Which kernel family a plan runs on B200 (the reference's regimes -- direct / streaming /
    materialized -- describe its SM120 kernels; every regime here materialises the routes with a
    separate sort and walks them with a persistent grid)."""

    SMALL_BATCH = "small_batch_swap_ab"      # 64-row expert tiles, weights as the MMA rows (decode)
    WIDE_TILE = "wide_tile"                  # 128 x 256 tiles, one CTA per tile
    WIDE_TILE_CTA_PAIR = "wide_tile_cta_pair"  # 256 x 256 tiles on CTA pairs (tcgen05 cta_group::2)
    W4A16_CONVERTER = "w4a16_converter"      # bf16 activations, FP4 weights expanded in shared memory


class RouteLayout(str, Enum):
    SORTED_COMPACT_EXPERT = "sorted_compact_expert"   # stable (expert, route id) order, no per-expert padding


class WorkAvailability(str, Enum):
    PRECOMPUTED = "precomputed"


class WorkScheduler(str, Enum):
    PERSISTENT_GRID = "persistent_grid"


class GraphPartition(str, Enum):
    SPLIT_FC1_FC2 = "split_fc1_fc2"          # FC1+activation+requantisation and FC2 are two launches


class GemmEngine(str, Enum):
    TCGEN05_MXF4NVF4 = "tcgen05_mxf4nvf4"    # nvfp4: E2M1 x E2M1, UE4M3 scale per 16
    TCGEN05_MXF8F6F4 = "tcgen05_mxf8f6f4"    # w4a8_mx: E4M3 x E2M1, UE8M0 scale per 32
    TCGEN05_F16 = "tcgen05_f16"              # w4a16: bf16 x bf16 after in-kernel FP4 expansion


class PreparedWeightLayout(str, Enum):
    SOURCE_NATIVE = "source_native"


class OutputReduction(str, Enum):
    ROUTE_BUFFER_TOPK_SUM = "route_buffer_topk_sum"   # fp32 rows per route, fixed-order weighted sum


@dataclass(frozen=True, kw_only=True)
class MoEExecutionPlan:
    """A lowering of :class:`MoESpec` onto one concrete execution regime (same fields as the
    reference's dataclass; the enum values name this library's kernels)."""

    regime: MoERegime
    route_layout: RouteLayout
    work_availability: WorkAvailability
    scheduler: WorkScheduler
    graph_partition: GraphPartition
    gemm_engine: GemmEngine
    weight_layout: PreparedWeightLayout
    reduction: OutputReduction
    tile_m: int | None = None
    tile_n: int | None = None
    route_block_rows: int | None = None

    def __post_init__(self) -> None:
        for name, enum_type in (("regime", MoERegime), ("route_layout", RouteLayout),
                                ("work_availability", WorkAvailability), ("scheduler", WorkScheduler),
                                ("graph_partition", GraphPartition), ("gemm_engine", GemmEngine),
                                ("weight_layout", PreparedWeightLayout), ("reduction", OutputReduction)):
            object.__setattr__(self, name, enum_type(getattr(self, name)))
        for name in ("tile_m", "tile_n", "route_block_rows"):
            value = getattr(self, name)
            if value is not None and int(value) <= 0:
                raise ValueError(f"{name} must be positive, got {value}")

    @property
    def work_is_streamed(self) -> bool:
        return False

    @property
    def grid_addressable(self) -> bool:
        """All compute work is known before the GEMM kernels start (no in-kernel waiting for routes)."""
        return True

    @property
    def uses_explicit_task_queue(self) -> bool:
        return False


def lower_moe_execution(spec: MoESpec, *, routed_rows_capacity: int, num_experts: int, intermediate_size: int,
                        hidden_size: int, tile_rows: int | None = None) -> MoEExecutionPlan:
    """Regime and tile choice for one recipe and capacity -- the host-side statement of what the
    C ABI decides (``b200moe_scratch_nbytes`` for the tile height, the GEMM entry points for the
    kernel family).  ``tile_rows`` overrides the tile height (64 / 128)."""
    rows, e = int(routed_rows_capacity), int(num_experts)
    gated = spec.activation in GATED_ACTIVATIONS
    small_ok = spec.quant_mode == "nvfp4" and intermediate_size % 128 == 0 and hidden_size % 64 == 0
    tm = int(tile_rows) if tile_rows else (64 if (small_ok and rows <= 48 * e) else 128)
    if tm == 64 and not small_ok:
        tm = 128
    if spec.quant_mode == "w4a16":
        regime, engine = MoERegime.W4A16_CONVERTER, GemmEngine.TCGEN05_F16
    elif spec.quant_mode == "w4a8_mx":
        regime, engine = MoERegime.WIDE_TILE, GemmEngine.TCGEN05_MXF8F6F4
    else:
        engine = GemmEngine.TCGEN05_MXF4NVF4
        if tm == 64:
            regime = MoERegime.SMALL_BATCH
        elif gated and rows >= 256 * e:
            regime = MoERegime.WIDE_TILE_CTA_PAIR
        else:
            regime = MoERegime.WIDE_TILE
    return MoEExecutionPlan(
        regime=regime, route_layout=RouteLayout.SORTED_COMPACT_EXPERT,
        work_availability=WorkAvailability.PRECOMPUTED, scheduler=WorkScheduler.PERSISTENT_GRID,
        graph_partition=GraphPartition.SPLIT_FC1_FC2, gemm_engine=engine,
        weight_layout=PreparedWeightLayout.SOURCE_NATIVE, reduction=OutputReduction.ROUTE_BUFFER_TOPK_SUM,
        tile_m=256 if regime is MoERegime.WIDE_TILE_CTA_PAIR else tm,
        tile_n=256, route_block_rows=tm)
