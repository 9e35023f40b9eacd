"""Planner and launch glue of ``moe.fused_moe`` for B200 (sm_100a).

Host-side mirror of the reference's ``b12x/moe/fused_moe/_impl.py``: the same lifecycle
(``plan_weights`` -> ``prepare_weights`` -> ``plan(Caps)`` -> ``bind`` -> ``run``), the same
contracts (one caller-owned uint8 scratch tensor, ``bind`` only creates views, ``run`` launches on
the current stream without allocating or synchronising when ``output`` is given), and the same
exception types.  The work itself is six C-ABI launches into ``libb200moe.so``:
expert sort -> permute+quantise -> grouped FC1+activation -> grouped FC2 -> combine
(plus ``route_topk`` when routing is requested).  There is no other implementation behind this
module: without the extension every call raises.
"""

from __future__ import annotations

import os

import ctypes as C
from collections.abc import Mapping, Sequence
from dataclasses import dataclass, field

import torch

from ..._lib import ext
from ..._lib.scratch import ScratchBufferSpec, scratch_buffer_spec, scratch_tensor
from .._shared.execution import (
    SWIGLUOAI,
    MoEExecutionPlan,
    MoESpec,
    MoEWeightPreparationPlan,
    lower_moe_execution,
    WeightPreparationTransform,
    is_gated_moe_activation,
    make_moe_spec,
    normalize_moe_activation,
    normalize_swiglu_params,
    normalize_w13_layout,
    plan_moe_weight_preparation,
)
from .._shared.routing import route_topk

_ACT_CODE = {"silu": "silu", "relu2": "relu2", SWIGLUOAI: "swigluoai", "situ": "situ"}


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _align_up(v: int, a: int) -> int:
    return (v + a - 1) // a * a


# =============================================================================================
# weights
# =============================================================================================
def plan_b12x_fp4_moe_weights(
    *,
    quant_modes: str | Sequence[str],
    source_format: str,
    activation: str,
    params_dtype: torch.dtype,
    num_experts: int,
    hidden_size: int,
    intermediate_size: int,
    w13_layout: str = "w13",
) -> MoEWeightPreparationPlan:
    """Plan the one canonical weight allocation used by the selected recipes.

    Reference: ``plan_b12x_fp4_moe_weights`` (b12x/moe/fused_moe/_impl.py:4992-5042)."""
    activation = normalize_moe_activation(activation)
    modes = (quant_modes,) if isinstance(quant_modes, str) else tuple(quant_modes)
    if not modes:
        raise ValueError("quant_modes must contain at least one recipe")
    specs = tuple(
        make_moe_spec(quant_mode=m, source_format=source_format, activation=activation,
                      io_dtype=str(params_dtype).removeprefix("torch."), w13_layout=w13_layout)
        for m in modes)
    return plan_moe_weight_preparation(specs, num_experts=num_experts, hidden_size=hidden_size,
                                       intermediate_size=intermediate_size)


@dataclass(frozen=True, kw_only=True)
class B12XFP4ExpertWeights:
    """Sole owner of the expert weights at run time (reference _impl.py:407-581).

    ``w*_fp4`` are the checkpoint tensors themselves (two E2M1 per byte); ``w*_blockscale`` are
    128x4-swizzled scale atoms (E4M3 per 16 for nvfp4 / w4a16, E8M0 per 32 for w4a8_mx, the
    latter produced from the plain checkpoint grids by ``prepare_weights``)."""

    plan: MoEWeightPreparationPlan
    a1_gscale: torch.Tensor
    w1_fp4: torch.Tensor
    w1_blockscale: torch.Tensor
    w1_alphas: torch.Tensor
    a2_gscale: torch.Tensor
    w2_fp4: torch.Tensor
    w2_blockscale: torch.Tensor
    w2_alphas: torch.Tensor
    # nvfp4 with a gated activation: FC1 scales as 128-row atoms in the checkpoint's row order
    # (the caller's own tensor, kept by reference), read by the small-batch kernel
    w1_blockscale_rows: torch.Tensor | None = None

    def __post_init__(self) -> None:
        if not isinstance(self.plan, MoEWeightPreparationPlan):
            raise TypeError("plan must be a MoEWeightPreparationPlan")
        for name in ("a1_gscale", "w1_fp4", "w1_blockscale", "w1_alphas", "a2_gscale", "w2_fp4",
                     "w2_blockscale", "w2_alphas"):
            if not isinstance(getattr(self, name), torch.Tensor):
                raise TypeError(f"{name} must be a torch.Tensor")
        p = self.plan
        if tuple(self.w1_fp4.shape) != (p.num_experts, p.w1_rows, p.hidden_size // 2):
            raise ValueError(
                f"w1_fp4 shape {tuple(self.w1_fp4.shape)} does not match the weight plan "
                f"{(p.num_experts, p.w1_rows, p.hidden_size // 2)}")
        if tuple(self.w2_fp4.shape) != (p.num_experts, p.hidden_size, p.intermediate_size // 2):
            raise ValueError(
                f"w2_fp4 shape {tuple(self.w2_fp4.shape)} does not match the weight plan "
                f"{(p.num_experts, p.hidden_size, p.intermediate_size // 2)}")
        for name in ("w1_fp4", "w2_fp4", "w1_blockscale", "w2_blockscale"):
            if not getattr(self, name).is_contiguous():
                raise ValueError(f"{name} must be contiguous")
        dev = self.w1_fp4.device
        for name in ("a1_gscale", "w1_blockscale", "w1_alphas", "a2_gscale", "w2_fp4", "w2_blockscale",
                     "w2_alphas"):
            if getattr(self, name).device != dev:
                raise ValueError(f"{name} is on {getattr(self, name).device}, w1_fp4 on {dev}")
        for name in ("a1_gscale", "w1_alphas", "a2_gscale", "w2_alphas"):
            t = getattr(self, name)
            if t.dtype != torch.float32 or t.numel() != p.num_experts or not t.is_contiguous():
                raise ValueError(f"{name} must be contiguous float32 with one value per expert")
        # Every tensor a kernel reads is its own byte range: a package whose FC1 and FC2 weights (or a
        # weight and a scale tensor) overlap was assembled from views of the wrong buffer
        ranges = []
        for name in ("w1_fp4", "w2_fp4", "w1_blockscale", "w2_blockscale"):
            t = getattr(self, name)
            lo = t.data_ptr()
            ranges.append((lo, lo + t.numel() * t.element_size(), name))
        ranges.sort()
        for (lo0, hi0, n0), (lo1, _hi1, n1) in zip(ranges[:-1], ranges[1:]):
            if lo1 < hi0 and hi0 > lo0:
                raise ValueError(f"{n0} and {n1} overlap in memory")
        if self.w1_blockscale_rows is not None:
            r = self.w1_blockscale_rows
            want = p.num_experts * _align_up(p.w1_rows, 128) * _align_up(p.hidden_size // 16, 4)
            if r.dtype != torch.uint8 or not r.is_contiguous() or r.numel() != want or r.device != dev:
                raise ValueError("w1_blockscale_rows must be the contiguous 128x4-swizzled FC1 scale atoms")

    # the plan's facts, as the reference's package exposes them (_impl.py:542-564)
    @property
    def source_format(self) -> str:
        return self.plan.source_format

    @property
    def w13_layout(self) -> str:
        return self.plan.w13_layout

    @property
    def activation(self) -> str:
        return self.plan.activation

    @property
    def num_experts(self) -> int:
        return self.plan.num_experts

    @property
    def hidden_size(self) -> int:
        return self.plan.hidden_size

    @property
    def intermediate_size(self) -> int:
        return self.plan.intermediate_size

    def keeps_source(self, source: torch.Tensor) -> bool:
        """True if ``source`` (a tensor handed to ``prepare_weights``) is used where it lies, i.e.
        the caller must keep it alive and unchanged; False if the package holds its own copy (the
        re-laid scale atoms, weights re-homed for tail slack) and the source may be freed."""
        ptr = source.untyped_storage().data_ptr()
        return any(getattr(self, n) is not None and getattr(self, n).untyped_storage().data_ptr() == ptr
                   for n in ("w1_fp4", "w2_fp4", "w1_blockscale", "w2_blockscale", "w1_blockscale_rows"))

    def device_nbytes(self) -> int:
        """Device bytes this package keeps alive, counting each storage once."""
        seen, total = set(), 0
        for n in ("a1_gscale", "w1_fp4", "w1_blockscale", "w1_alphas", "a2_gscale", "w2_fp4", "w2_blockscale",
                  "w2_alphas", "w1_blockscale_rows"):
            t = getattr(self, n)
            if t is None:
                continue
            st = t.untyped_storage()
            if st.data_ptr() not in seen:
                seen.add(st.data_ptr())
                total += st.nbytes()
        return total


def _expert_vector(t: torch.Tensor, num_experts: int, name: str) -> torch.Tensor:
    t = t.to(torch.float32).reshape(-1)
    if t.numel() == 1:
        t = t.expand(num_experts)
    if t.numel() != num_experts:
        raise ValueError(f"{name} must have 1 or {num_experts} elements, got {t.numel()}")
    return t.contiguous()


def _swizzle_scale_grid(grid: torch.Tensor) -> torch.Tensor:
    """[E, rows, cols] bytes -> [E, pad128(rows), pad4(cols)] 128x4-swizzled atoms
    (layout of b12x/_lib/intrinsics.py:62-82)."""
    e, rows, cols = grid.shape
    rp, cp = _align_up(rows, 128), _align_up(cols, 4)
    padded = torch.zeros((e, rp, cp), dtype=torch.uint8, device=grid.device)
    padded[:, :rows, :cols] = grid.view(torch.uint8)
    sw = padded.reshape(e, rp // 128, 4, 32, cp // 4, 4).permute(0, 1, 4, 3, 2, 5).contiguous()
    return sw.reshape(e, rp, cp)


def _unswizzle_scale_grid(sw: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    """Inverse of :func:`_swizzle_scale_grid`: ``[E, padded atoms]`` (or one expert's atoms) ->
    ``[E, rows, cols]`` (``[rows, cols]``) bytes, all experts in one pass."""
    rp, cp = _align_up(rows, 128), _align_up(cols, 4)
    single = sw.numel() == rp * cp and (sw.ndim < 3 or sw.shape[0] != 1)
    e = 1 if single else int(sw.shape[0])
    u = sw.reshape(e, -1)[:, : rp * cp].reshape(e, rp // 128, cp // 4, 32, 4, 4).permute(0, 1, 4, 3, 2, 5)
    out = u.contiguous().reshape(e, rp, cp)[:, :rows, :cols]
    return out[0] if single else out


def _pair_scale_atoms(grid: torch.Tensor, intermediate: int, gate_first: bool) -> torch.Tensor:
    """FC1 scales of a gated activation, re-laid as PAIR atoms.

    ``grid`` is the plain ``[E, 2I, cols]`` byte grid of W13's block scales.  The FC1 kernel works on
    tiles of 64 up rows + 64 gate rows, so the scales of such a tile must form one 128-row atom
    chain: rows are re-ordered to [up 0..63, gate 0..63, up 64..127, gate 64..127, ...] and then
    swizzled.  The weight codes themselves are not touched (the kernel fetches the two 64-row
    halves with separate TMA boxes); this scale tensor is a new allocation of the source's size."""
    e, rows, cols = grid.shape
    i = int(intermediate)
    if rows != 2 * i or i % 64 != 0:
        raise ValueError("gated FC1 needs [E, 2I, cols] scales with I a multiple of 64")
    up, gate = (grid[:, i:], grid[:, :i]) if gate_first else (grid[:, :i], grid[:, i:])
    paired = torch.stack([up.reshape(e, i // 64, 64, cols), gate.reshape(e, i // 64, 64, cols)], dim=2)
    return _swizzle_scale_grid(paired.reshape(e, 2 * i, cols))


def _with_tail_slack(w: torch.Tensor, cols: int) -> torch.Tensor:
    if cols % 128 == 0:
        return w
    flat = torch.empty(w.numel() + 256, dtype=torch.uint8, device=w.device)
    flat[: w.numel()].copy_(w.reshape(-1).view(torch.uint8))
    return flat[: w.numel()].view(w.shape)


def prepare_b12x_fp4_moe_weights(
    *,
    plan: MoEWeightPreparationPlan,
    params_dtype: torch.dtype,
    w1_fp4: torch.Tensor | None = None,
    w2_fp4: torch.Tensor | None = None,
    w1_global_scale: torch.Tensor | None = None,
    w2_global_scale: torch.Tensor | None = None,
    w1_blockscale: torch.Tensor | None = None,
    w2_blockscale: torch.Tensor | None = None,
    a1_gscale: torch.Tensor | None = None,
    a2_gscale: torch.Tensor | None = None,
) -> B12XFP4ExpertWeights:
    """Transfer source tensors into the planner-selected runtime owner.

    Reference: ``prepare_b12x_fp4_moe_weights`` (_impl.py:5045-5365).  For nvfp4 the runtime
    alphas are ``w_global_scale / a_gscale`` (``a*_gscale`` are RECIPROCAL input scales,
    _impl.py:4955-4989); weights and E4M3 scales are used where they lie.  For w4a8_mx the plain
    ``[E, rows, cols/32]`` E8M0 grids are re-laid once into 128x4 atoms."""
    if not isinstance(plan, MoEWeightPreparationPlan):
        raise TypeError("plan must be a MoEWeightPreparationPlan")
    actual = str(params_dtype).removeprefix("torch.")
    if actual != plan.io_dtype:
        raise ValueError(f"params_dtype={actual!r} does not match plan dtype={plan.io_dtype!r}")
    for name, t in (("w1_fp4", w1_fp4), ("w2_fp4", w2_fp4), ("w1_blockscale", w1_blockscale),
                    ("w2_blockscale", w2_blockscale)):
        if not isinstance(t, torch.Tensor):
            raise TypeError(f"{name} is required")
    e = plan.num_experts
    dev = w1_fp4.device
    ones = torch.ones(e, dtype=torch.float32, device=dev)
    a1 = ones if a1_gscale is None else _expert_vector(a1_gscale, e, "a1_gscale").to(dev)
    a2 = ones if a2_gscale is None else _expert_vector(a2_gscale, e, "a2_gscale").to(dev)
    g1 = ones if w1_global_scale is None else _expert_vector(w1_global_scale, e, "w1_global_scale").to(dev)
    g2 = ones if w2_global_scale is None else _expert_vector(w2_global_scale, e, "w2_global_scale").to(dev)
    if WeightPreparationTransform.INVERT_GLOBAL_SCALES in plan.transforms:
        # compressed-tensors keeps the reciprocal of the ModelOpt weight global scale
        # (w4a16/prepare.py:460-465)
        g1, g2 = torch.reciprocal(g1), torch.reciprocal(g2)
    if "nvfp4" in plan.quant_modes:
        if a1_gscale is None or a2_gscale is None or w1_global_scale is None or w2_global_scale is None:
            raise ValueError("nvfp4 needs w*_global_scale and a*_gscale")
        alphas1, alphas2 = torch.div(g1, a1), torch.div(g2, a2)
    else:
        alphas1, alphas2 = g1.clone(), g2.clone()
    s1, s2 = w1_blockscale, w2_blockscale
    s1_rows = None
    if WeightPreparationTransform.SWIZZLE_MX_SCALES in plan.transforms:
        if tuple(s1.shape) != (e, plan.w1_rows, plan.hidden_size // 32):
            raise ValueError("fp4_e8m0_k32 w1_blockscale must be [E, w1_rows, K/32] E8M0 bytes")
        if tuple(s2.shape) != (e, plan.hidden_size, plan.intermediate_size // 32):
            raise ValueError("fp4_e8m0_k32 w2_blockscale must be [E, K, I/32] E8M0 bytes")
        if is_gated_moe_activation(plan.activation):
            s1 = _pair_scale_atoms(s1.view(torch.uint8), plan.intermediate_size, plan.w13_layout == "w31")
        else:
            s1 = _swizzle_scale_grid(s1)
        s2 = _swizzle_scale_grid(s2)
        # the 4-bit unpacking TMA reads whole 128-value groups: a row whose length is not a
        # multiple of 128 values lets the last row's read run 32 bytes past the tensor; re-home
        # such tensors into storage with slack (one-time copy, the source may be freed)
        w1_fp4 = _with_tail_slack(w1_fp4, plan.hidden_size)
        w2_fp4 = _with_tail_slack(w2_fp4, plan.intermediate_size)
    elif WeightPreparationTransform.EXPAND_E8M0_K32 in plan.transforms:
        # w4a16 over an E8M0 K/32 source (w4a16/prepare.py:1289-1325): the kernel's scale stage
        # holds one byte per 16 values, so every per-32 byte is written twice and the kernel is
        # told to decode the bytes as E8M0
        if tuple(s1.shape) != (e, plan.w1_rows, plan.hidden_size // 32):
            raise ValueError("fp4_e8m0_k32 w1_blockscale must be [E, w1_rows, K/32] E8M0 bytes")
        if tuple(s2.shape) != (e, plan.hidden_size, plan.intermediate_size // 32):
            raise ValueError("fp4_e8m0_k32 w2_blockscale must be [E, K, I/32] E8M0 bytes")
        s1 = _swizzle_scale_grid(s1.view(torch.uint8).repeat_interleave(2, dim=-1))
        s2 = _swizzle_scale_grid(s2.view(torch.uint8).repeat_interleave(2, dim=-1))
    else:
        exp1 = (e, _align_up(plan.w1_rows, 128), _align_up(plan.hidden_size // 16, 4))
        exp2 = (e, _align_up(plan.hidden_size, 128), _align_up(plan.intermediate_size // 16, 4))
        if s1.numel() != exp1[0] * exp1[1] * exp1[2] or s2.numel() != exp2[0] * exp2[1] * exp2[2]:
            raise ValueError(
                "modelopt_nvfp4 block scales must be 128x4-swizzled "
                f"{exp1} / {exp2}, got {tuple(s1.shape)} / {tuple(s2.shape)}")
        s1, s2 = s1.view(torch.uint8), s2.view(torch.uint8)
        if ("nvfp4" in plan.quant_modes and is_gated_moe_activation(plan.activation)
                and plan.intermediate_size % 128 == 0):
            s1_rows = s1.contiguous()
        if "nvfp4" in plan.quant_modes and is_gated_moe_activation(plan.activation):
            if "w4a16" in plan.quant_modes:
                raise ValueError("one weight plan cannot serve both nvfp4 and w4a16: they need "
                                 "different FC1 scale layouts")
            rows, cols = plan.w1_rows, plan.hidden_size // 16
            grid = _unswizzle_scale_grid(s1, rows, cols)        # all experts at once
            s1 = _pair_scale_atoms(grid, plan.intermediate_size, plan.w13_layout == "w31")
    return B12XFP4ExpertWeights(
        plan=plan, a1_gscale=a1, w1_fp4=w1_fp4.view(torch.uint8), w1_blockscale=s1.contiguous(),
        w1_alphas=alphas1.contiguous(), a2_gscale=a2, w2_fp4=w2_fp4.view(torch.uint8),
        w2_blockscale=s2.contiguous(), w2_alphas=alphas2.contiguous(), w1_blockscale_rows=s1_rows)


# =============================================================================================
# caps / plan / binding
# =============================================================================================
@dataclass(frozen=True, kw_only=True)
class TPMoEScratchCaps:
    """Capacity and options of one scratch plan (reference _impl.py:747-860, same field names)."""

    max_tokens: int
    num_topk: int
    device: torch.device | str
    weight_plan: MoEWeightPreparationPlan
    quant_mode: str
    core_token_counts: tuple[int, ...] | None = None
    route_num_experts: int | None = None
    route_logits_dtype: torch.dtype | None = None
    apply_router_weight_on_input: bool = False
    swiglu_limit: float | None = None
    swiglu_alpha: float | None = None
    swiglu_beta: float | None = None
    collect_activation_amax: bool = False
    deterministic_output: bool | None = None
    # rows per expert tile: None = chosen from the capacity (64 with the small-batch kernel when
    # the plan averages <= 48 routed rows per expert, else 128); 64 / 128 force it
    tile_rows: int | None = None
    w4a16_block_size_m: int | None = None
    w4a16_fast_math: bool = True
    frozen: bool = True

    def __post_init__(self) -> None:
        object.__setattr__(self, "max_tokens", max(int(self.max_tokens), 1))
        object.__setattr__(self, "num_topk", max(int(self.num_topk), 1))
        dev = torch.device(self.device)
        if dev.type == "cuda" and dev.index is None:
            dev = torch.device("cuda", torch.cuda.current_device() if torch.cuda.is_available() else 0)
        object.__setattr__(self, "device", dev)
        if not isinstance(self.weight_plan, MoEWeightPreparationPlan):
            raise TypeError("weight_plan must be a MoEWeightPreparationPlan")
        mode = str(self.quant_mode).lower()
        if mode not in self.weight_plan.quant_modes:
            raise ValueError(f"quant_mode={mode!r} is absent from the weight plan")
        object.__setattr__(self, "quant_mode", mode)
        if self.core_token_counts is not None:
            object.__setattr__(self, "core_token_counts",
                               tuple(max(int(c), 1) for c in self.core_token_counts))
        if self.route_num_experts is not None:
            object.__setattr__(self, "route_num_experts", max(int(self.route_num_experts), 0))
        limit, alpha, beta = normalize_swiglu_params(self.activation, self.swiglu_limit,
                                                     self.swiglu_alpha, self.swiglu_beta)
        object.__setattr__(self, "swiglu_limit", limit)
        object.__setattr__(self, "swiglu_alpha", alpha)
        object.__setattr__(self, "swiglu_beta", beta)
        if self.apply_router_weight_on_input and str(self.quant_mode).lower() != "w4a16":
            # as the reference: only its W4A16 path takes it (_impl.py:10631-10634)
            raise NotImplementedError("apply_router_weight_on_input is not implemented in b12x_moe_fp4")
        if self.collect_activation_amax and str(self.quant_mode).lower() != "w4a16":
            # as the reference (_impl.py:10601-10604)
            raise NotImplementedError("activation_amax calibration is only supported for W4A16")
        if self.num_topk > 32:
            raise ValueError("num_topk > 32 is not supported")
        if self.tile_rows not in (None, 0, 64, 128):
            raise ValueError("tile_rows must be 64 or 128")

    @property
    def weight_E(self) -> int:
        return self.weight_plan.num_experts

    @property
    def k(self) -> int:
        return self.weight_plan.hidden_size

    @property
    def n(self) -> int:
        return self.weight_plan.intermediate_size

    @property
    def dtype(self) -> torch.dtype:
        return {"bfloat16": torch.bfloat16}[self.weight_plan.io_dtype]

    @property
    def activation(self) -> str:
        return self.weight_plan.activation

    @property
    def source_format(self) -> str:
        return self.weight_plan.source_format

    @property
    def w13_layout(self) -> str:
        return self.weight_plan.w13_layout


@dataclass(frozen=True, kw_only=True)
class TPMoEArenaLayout:
    route_workspace_nbytes: int
    core_workspace_nbytes: int
    total_nbytes: int
    core_token_counts: tuple[int, ...] = ()


@dataclass(frozen=True, kw_only=True)
class TPMoEPlan:
    """Logical launch plan plus the precision-neutral execution descriptors (reference ``TPMoEPlan``
    _impl.py:717-744): ``spec`` is the numeric contract, ``execution`` the regime / tile choice."""

    spec: MoESpec
    execution: MoEExecutionPlan
    implementation: str      # the kernel family: execution.regime.value
    quant_mode: str
    activation: str
    swiglu_limit: float | None = None
    swiglu_alpha: float = 1.0
    swiglu_beta: float = 0.0
    state_E: int
    weight_E: int
    routed_rows: int
    max_rows: int
    k: int
    n: int
    num_topk: int
    device: torch.device
    dtype: torch.dtype
    max_tokens_per_launch: int
    max_m_tiles: int = 0

    @property
    def deterministic_output(self) -> bool:
        return True          # fp32 rows per route, combined in slot order

    @property
    def tile_m(self) -> int:
        return int(self.execution.tile_m)

    @property
    def tile_n(self) -> int:
        return int(self.execution.tile_n)


_ROUTE_ALIGN = 1024


def _route_workspace_nbytes(caps: TPMoEScratchCaps) -> int:
    """Router logits (when a gate GEMM is requested) + top-k logits/ids/weights + the gate kernel's
    arrival counters (laid out by ``TPMoEWorkspace.route_views``)."""
    e = caps.route_num_experts or 0
    if e <= 0:
        return 0
    t, k = caps.max_tokens, caps.num_topk
    return (_align_up(t * e * 4, _ROUTE_ALIGN) + 3 * _align_up(t * k * 4, _ROUTE_ALIGN)
            + _align_up(((t + 3) // 4) * 4, _ROUTE_ALIGN))


def _layout_for(caps: TPMoEScratchCaps) -> ext.ScratchLayout:
    return ext.scratch_layout(caps.max_tokens, caps.num_topk, caps.weight_E, caps.k, caps.n,
                              caps.quant_mode, _ACT_CODE[caps.activation], caps.tile_rows or 0)


def plan_tp_moe_execution(
    *,
    num_tokens: int,
    num_topk: int,
    device: torch.device | str,
    weight_plan: MoEWeightPreparationPlan,
    quant_mode: str,
    swiglu_limit: float | None = None,
    swiglu_alpha: float | None = None,
    swiglu_beta: float | None = None,
    apply_router_weight_on_input: bool = False,
    deterministic_output: bool | None = None,
    tile_rows: int | None = None,
) -> TPMoEPlan:
    """Lower one recipe from an authoritative weight-preparation plan (reference
    ``plan_tp_moe_execution`` _impl.py:5647-5840, same keywords): which kernel family and tile a
    launch over ``num_tokens`` tokens uses.  ``deterministic_output=False`` is accepted: the output
    reduction here is always the deterministic one."""
    if not isinstance(weight_plan, MoEWeightPreparationPlan):
        raise TypeError("weight_plan must be a MoEWeightPreparationPlan")
    mode = str(quant_mode).lower()
    spec = next((sp for sp in weight_plan.specs if sp.quant_mode == mode), None)
    if spec is None:
        raise ValueError(f"quant_mode={mode!r} is absent from the weight plan")
    if apply_router_weight_on_input and mode != "w4a16":
        raise NotImplementedError("apply_router_weight_on_input is not implemented in b12x_moe_fp4")
    limit, alpha, beta = normalize_swiglu_params(weight_plan.activation, swiglu_limit, swiglu_alpha, swiglu_beta)
    t, k_ = max(int(num_tokens), 1), max(int(num_topk), 1)
    rows = t * k_
    ex = lower_moe_execution(spec, routed_rows_capacity=rows, num_experts=weight_plan.num_experts,
                             intermediate_size=weight_plan.intermediate_size, hidden_size=weight_plan.hidden_size,
                             tile_rows=tile_rows)
    dev = torch.device(device)
    tm = int(ex.route_block_rows)
    return TPMoEPlan(
        spec=spec, execution=ex, implementation=ex.regime.value, quant_mode=mode, activation=weight_plan.activation,
        swiglu_limit=limit, swiglu_alpha=alpha, swiglu_beta=beta, state_E=weight_plan.num_experts,
        weight_E=weight_plan.num_experts, routed_rows=rows, max_rows=rows, k=weight_plan.hidden_size,
        n=weight_plan.intermediate_size, num_topk=k_, device=dev,
        dtype={"bfloat16": torch.bfloat16}[weight_plan.io_dtype], max_tokens_per_launch=t,
        max_m_tiles=(rows + tm - 1) // tm + min(weight_plan.num_experts, rows))


def _plan_execution_for_caps(caps: TPMoEScratchCaps) -> TPMoEPlan:
    return plan_tp_moe_execution(
        num_tokens=caps.max_tokens, num_topk=caps.num_topk, device=caps.device, weight_plan=caps.weight_plan,
        quant_mode=caps.quant_mode, swiglu_limit=caps.swiglu_limit, swiglu_alpha=caps.swiglu_alpha,
        swiglu_beta=caps.swiglu_beta, tile_rows=caps.tile_rows or None)


def tp_moe_required_nbytes(caps: TPMoEScratchCaps) -> int:
    """Bytes of scratch ``plan(caps)`` will ask for (reference _impl.py:6781-6783)."""
    return _route_workspace_nbytes(caps) + int(_layout_for(caps).total_nbytes)


@dataclass(frozen=True)
class TPMoEScratchPlan:
    caps: TPMoEScratchCaps
    layout: TPMoEArenaLayout
    launch_plan: TPMoEPlan
    _core_layout: ext.ScratchLayout = field(repr=False)
    _scratch_specs: tuple[ScratchBufferSpec, ...] = ()

    def scratch_specs(self) -> tuple[ScratchBufferSpec, ...]:
        return self._scratch_specs

    def shapes_and_dtypes(self):
        return tuple((spec.shape, spec.dtype) for spec in self._scratch_specs)

    def bind(
        self,
        *,
        scratch: torch.Tensor | Mapping[str, torch.Tensor] | Sequence[torch.Tensor],
        a: torch.Tensor,
        experts: B12XFP4ExpertWeights,
        topk_weights: torch.Tensor,
        topk_ids: torch.Tensor,
        output: torch.Tensor | None = None,
        input_scales_static: bool = False,
        fast_math: bool | None = None,
        unit_scale_contract: bool = False,
        activation_amax: torch.Tensor | None = None,
        layer_idx: int | None = None,
        route_expert_map: torch.Tensor | None = None,
        output_expert_map: torch.Tensor | None = None,
        fc1_tap: torch.Tensor | None = None,
        output_f32: torch.Tensor | None = None,
        output_scale: float = 1.0,
        f32_only: bool = False,
        skip_combine: bool = False,
        sort_wait: tuple | None = None,
        a_packed: tuple | None = None,
    ) -> "TPMoEFP4Binding":
        """Validate the call and map the caller's scratch into kernel-argument views.

        Views only: nothing is allocated, copied or launched (reference
        ``TPMoEScratchPlan.bind`` _impl.py:888-966).  ``route_expert_map`` ([global E] -> local id
        or -1) makes non-local routes inactive, as ``ep_moe`` does in the reference."""
        caps = self.caps
        if not isinstance(experts, B12XFP4ExpertWeights):
            raise TypeError("experts must come from prepare_b12x_fp4_moe_weights")
        if output_expert_map is not None:
            # reference _impl.py:2333-2334: only its trellis full-rotation plans take one
            raise ValueError("output_expert_map requires a full-rotation Trellis plan")
        if activation_amax is not None:
            # reference _impl.py:10601-10604: a W4A16-only calibration side channel,
            # float32 [layers, experts, 2] (FC1 input amax, FC2 input amax), maximum kept across calls
            if caps.quant_mode != "w4a16":
                raise NotImplementedError("activation_amax calibration is only supported for W4A16")
            if (activation_amax.dtype != torch.float32 or activation_amax.ndim != 3 or not activation_amax.is_contiguous()
                    or activation_amax.shape[1] != caps.weight_E or activation_amax.shape[2] != 2
                    or activation_amax.device != caps.device):
                raise ValueError(f"activation_amax must be contiguous float32 [layers, {caps.weight_E}, 2] on {caps.device}")
            if layer_idx is None or not 0 <= int(layer_idx) < activation_amax.shape[0]:
                raise ValueError("activation_amax needs layer_idx inside its first dimension")
        if experts.plan != caps.weight_plan:
            raise ValueError("experts do not match the plan used to size TP MoE scratch")
        if a.ndim != 2 or topk_ids.ndim != 2 or topk_weights.ndim != 2:
            raise ValueError("a, topk_ids and topk_weights must have rank 2")
        tokens = int(a.shape[0])
        if tokens > caps.max_tokens:
            raise ValueError(f"input tokens {tokens} exceed TP MoE scratch capacity {caps.max_tokens}")
        if int(a.shape[1]) != caps.k:
            raise ValueError(f"input hidden size {int(a.shape[1])} does not match TP MoE scratch K={caps.k}")
        if int(topk_ids.shape[1]) != caps.num_topk:
            raise ValueError(f"top-k {int(topk_ids.shape[1])} does not match TP MoE scratch top-k={caps.num_topk}")
        if tuple(topk_ids.shape) != (tokens, caps.num_topk) or tuple(topk_weights.shape) != (tokens, caps.num_topk):
            raise ValueError("topk_ids / topk_weights must be [tokens, top_k]")
        if a.dtype != caps.dtype:
            raise TypeError(f"a must be {caps.dtype}, got {a.dtype}")
        if topk_ids.dtype != torch.int32:
            raise TypeError(f"topk_ids must be int32, got {topk_ids.dtype}")
        if topk_weights.dtype != torch.float32:
            raise TypeError(f"topk_weights must be float32, got {topk_weights.dtype}")
        for name, t in (("a", a), ("topk_ids", topk_ids), ("topk_weights", topk_weights)):
            if t.device != caps.device:
                raise ValueError(f"{name} is on {t.device}, the plan is for {caps.device}")
        if a.stride(1) != 1 or not topk_ids.is_contiguous() or not topk_weights.is_contiguous():
            raise ValueError("a must be row-contiguous; topk_ids / topk_weights contiguous")
        if output is not None:
            if tuple(output.shape) != (tokens, caps.k) or output.dtype != caps.dtype or output.stride(1) != 1:
                raise ValueError("output must be [tokens, K] in the plan dtype, row-contiguous")
        if a_packed is not None:
            # rows that arrive already quantised (the expert side of a quantised dispatch): codes
            # [tokens, K/2 | K] and row-major scale bytes [tokens, stride]; ``a`` is not read
            if caps.quant_mode not in ("nvfp4", "w4a8_mx") or caps.num_topk != 1:
                raise ValueError("a_packed needs an nvfp4 or w4a8_mx plan with top_k = 1")
            q, sf = a_packed
            row_bytes = caps.k // 2 if caps.quant_mode == "nvfp4" else caps.k
            nsf = caps.k // (16 if caps.quant_mode == "nvfp4" else 32)
            if q.dtype != torch.uint8 or sf.dtype != torch.uint8 or not q.is_contiguous() or not sf.is_contiguous():
                raise TypeError("a_packed tensors must be contiguous uint8")
            if tuple(q.shape) != (tokens, row_bytes) or sf.ndim != 2 or sf.shape[0] != tokens:
                raise ValueError(f"a_packed codes must be [tokens, {row_bytes}] with one scale row per token")
            if sf.shape[1] % 4 or sf.shape[1] < nsf:
                raise ValueError(f"a_packed scale rows must hold >= {nsf} bytes, padded to a multiple of 4")
        storage = scratch_tensor(scratch, self._scratch_specs, owner="TP MoE")
        core = storage.narrow(0, self.layout.route_workspace_nbytes, self.layout.core_workspace_nbytes)
        if core.data_ptr() % 32 != 0:
            raise ValueError("scratch must be 32-byte aligned")
        return TPMoEFP4Binding(
            a=a, experts=experts, topk_weights=topk_weights, topk_ids=topk_ids,
            implementation=self.launch_plan.implementation, weight_E=caps.weight_E,
            max_rows=caps.max_tokens * caps.num_topk, k=caps.k, n=caps.n, num_topk=caps.num_topk,
            device=caps.device, dtype=caps.dtype, output=output,
            input_scales_static=bool(input_scales_static), fast_math=fast_math,
            unit_scale_contract=bool(unit_scale_contract and caps.quant_mode == "w4a16"), layer_idx=layer_idx,
            quant_mode=caps.quant_mode, activation=caps.activation, w13_layout=caps.w13_layout,
            swiglu_limit=caps.swiglu_limit, swiglu_alpha=caps.swiglu_alpha,
            swiglu_beta=caps.swiglu_beta, route_expert_map=route_expert_map,
            kernel_workspace=core, core_layout=self._core_layout, fc1_tap=fc1_tap,
            output_f32=output_f32, output_scale=float(output_scale), f32_only=bool(f32_only),
            skip_combine=bool(skip_combine), sort_wait=sort_wait, a_packed=a_packed,
            apply_router_weight_on_input=bool(caps.apply_router_weight_on_input),
            activation_amax=activation_amax)


def plan_tp_moe_scratch(caps: TPMoEScratchCaps) -> TPMoEScratchPlan:
    """Scratch plan for ``caps``: ONE opaque uint8 buffer (reference _impl.py:6786-6863)."""
    if not isinstance(caps, TPMoEScratchCaps):
        raise TypeError("caps must be a TPMoEScratchCaps")
    core = _layout_for(caps)
    route = _route_workspace_nbytes(caps)
    total = route + int(core.total_nbytes)
    layout = TPMoEArenaLayout(route_workspace_nbytes=route, core_workspace_nbytes=int(core.total_nbytes),
                              total_nbytes=total,
                              core_token_counts=caps.core_token_counts or (caps.max_tokens,))
    spec = scratch_buffer_spec("tp_moe.scratch", nbytes=total, device=caps.device)
    return TPMoEScratchPlan(caps, layout, _plan_execution_for_caps(caps), core, (spec,))


def _view(core: torch.Tensor, offset: int, count: int, dtype: torch.dtype) -> torch.Tensor:
    nbytes = count * torch.empty((), dtype=dtype).element_size()
    return core.narrow(0, offset, nbytes).view(dtype)


@dataclass(frozen=True, kw_only=True)
class TPMoEFP4Binding:
    """Caller tensors plus scratch views for one call (reference ``TPMoEFP4Binding``
    _impl.py:969-1056).  The scratch-view properties expose what the kernels left behind; they are
    what the parity tests read."""

    a: torch.Tensor
    experts: B12XFP4ExpertWeights
    topk_weights: torch.Tensor
    topk_ids: torch.Tensor
    implementation: str
    weight_E: int
    max_rows: int
    k: int
    n: int
    num_topk: int
    device: torch.device
    dtype: torch.dtype
    output: torch.Tensor | None = None
    input_scales_static: bool = False
    fast_math: bool | None = None
    unit_scale_contract: bool = False
    layer_idx: int | None = None
    quant_mode: str | None = None
    activation: str = "silu"
    w13_layout: str = "w13"
    deterministic_output: bool = True
    swiglu_limit: float | None = None
    swiglu_alpha: float | None = None
    swiglu_beta: float | None = None
    route_expert_map: torch.Tensor | None = None
    kernel_workspace: torch.Tensor | None = None
    core_layout: ext.ScratchLayout | None = field(default=None, repr=False)
    fc1_tap: torch.Tensor | None = None
    output_f32: torch.Tensor | None = None
    output_scale: float = 1.0
    f32_only: bool = False     # write only ``output_f32`` (un-rounded sums), skip the bf16 output
    skip_combine: bool = False  # stop after FC2: the per-route rows stay in ``route_output``
    # (flags ptr, world, epoch ptr, status ptr): the sort first waits for the peers' flags (the
    # expert side of the peer-memory expert parallelism, whose ids are stored by other ranks)
    sort_wait: tuple | None = None
    # (codes, scale rows): the rows arrive quantised and ``run`` files them instead of quantising ``a``
    a_packed: tuple | None = None
    # w4a16: the router weights multiply FC1's rows (before the activation) instead of the combine's
    apply_router_weight_on_input: bool = False
    # w4a16 calibration: float32 [layers, experts, 2], updated at row ``layer_idx`` by every run
    activation_amax: torch.Tensor | None = None

    # ---- scratch views (valid after run) ----
    def _v(self, name: str, count: int, dtype: torch.dtype) -> torch.Tensor:
        return _view(self.kernel_workspace, int(getattr(self.core_layout, name)), count, dtype)

    @property
    def tokens(self) -> int:
        return int(self.a.shape[0])

    @property
    def status(self) -> torch.Tensor:
        return self._v("status", 16, torch.int32)

    @property
    def expert_counts(self) -> torch.Tensor:
        return self._v("expert_counts", self.weight_E, torch.int32)

    @property
    def expert_offsets(self) -> torch.Tensor:
        return self._v("expert_offsets", self.weight_E + 1, torch.int32)

    @property
    def expert_tile_base(self) -> torch.Tensor:
        return self._v("tile_base", self.weight_E + 1, torch.int32)

    @property
    def packed_route_indices(self) -> torch.Tensor:
        return self._v("sorted_route_ids", self.tokens * self.num_topk, torch.int32)

    @property
    def inv_perm(self) -> torch.Tensor:
        return self._v("inv_perm", self.tokens * self.num_topk, torch.int32)

    @property
    def packed_input(self) -> torch.Tensor:
        row = {"nvfp4": self.k // 2, "w4a8_mx": self.k, "w4a16": self.k * 2}[self.quant_mode]
        return self._v("act_q", self.max_rows * row, torch.uint8).view(self.max_rows, row)

    @property
    def packed_input_scale(self) -> torch.Tensor:
        per = {"nvfp4": 64, "w4a8_mx": 128, "w4a16": 64}[self.quant_mode]
        atoms = (self.k + per - 1) // per
        return self._v("act_sf", self.core_layout.mtile_cap * atoms * 512, torch.uint8)

    @property
    def materialized_intermediate(self) -> torch.Tensor:
        row = {"nvfp4": self.n // 2, "w4a8_mx": self.n, "w4a16": self.n * 2}[self.quant_mode]
        return self._v("mid_q", self.max_rows * row, torch.uint8).view(self.max_rows, row)

    @property
    def intermediate_scale(self) -> torch.Tensor:
        per = {"nvfp4": 64, "w4a8_mx": 128, "w4a16": 64}[self.quant_mode]
        atoms = (self.n + per - 1) // per
        return self._v("mid_sf", self.core_layout.mtile_cap * atoms * 512, torch.uint8)

    @property
    def route_output(self) -> torch.Tensor:
        return self._v("routed", self.max_rows * self.k, torch.float32).view(self.max_rows, self.k)

    def run(self) -> torch.Tensor:
        return b12x_moe_fp4(binding=self)


# =============================================================================================
# run
# =============================================================================================
def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


_NVTX = os.environ.get("B200MOE_NVTX", "0") == "1"
_NEXT_STAGE = {"begin": "expert_sort", "sort": "permute_quant", "quant": "grouped_gemm1_act",
               "gemm1": "grouped_gemm2", "gemm2": "combine"}
_LAST_STAGE = {(True, False): "gemm2", (True, True): "gemm2", (False, False): "combine", (False, True): "combine"}


def b12x_moe_fp4(*, binding: TPMoEFP4Binding, stage_timer=None) -> torch.Tensor:
    """Run the layer for one binding on the current CUDA stream and return ``[tokens, K]``.

    Reference: ``b12x_moe_fp4`` (_impl.py:10446-11012).  With ``binding.output`` set nothing is
    allocated and nothing synchronises, so the call can be captured in a CUDA graph.
    ``stage_timer`` (optional) is called with a stage name at every stage boundary; a benchmark
    uses it to record CUDA events around single kernels."""
    if not isinstance(binding, TPMoEFP4Binding):
        raise TypeError("binding must come from Plan.bind")
    b = binding
    if b.device.type != "cuda":
        raise RuntimeError("moe.fused_moe runs on CUDA devices only; there is no CPU path")
    lib = ext.load()
    tokens = b.tokens
    out = b.output
    if b.skip_combine:
        out = b.route_output
    elif b.f32_only:
        if b.output_f32 is None:
            raise ValueError("f32_only needs output_f32")
        out = b.output_f32
    elif out is None:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("output must be provided during CUDA graph capture")
        out = torch.empty((tokens, b.k), dtype=b.dtype, device=b.device)
    if tokens == 0:
        return out
    ex = b.experts
    L = b.core_layout
    lp = C.pointer(L)
    scratch = b.kernel_workspace.data_ptr()
    stream = _stream_ptr(b.device)
    recipe = ext.RECIPES[b.quant_mode]
    act = ext.ACTIVATIONS[_ACT_CODE[b.activation]]

    timer = stage_timer if stage_timer is not None else (lambda _name: None)
    if _NVTX:
        # B200MOE_NVTX=1: one NVTX range per stage, so that a timeline profiler shows the layer's
        # stages by name (the ranges close at the next stage boundary)
        def mark(name: str) -> None:
            if name != "begin":
                torch.cuda.nvtx.range_pop()
            timer(name)
            if name != _LAST_STAGE[(b.skip_combine, b.f32_only)]:
                torch.cuda.nvtx.range_push("b200moe." + _NEXT_STAGE.get(name, "stage"))
    else:
        mark = timer
    mark("begin")
    emap = b.route_expert_map
    sw = b.sort_wait or (None, 0, None, None)
    sort_args = ext.SortArgs(b.topk_ids.data_ptr(), _ptr(emap), scratch, lp, tokens, b.num_topk,
                             b.weight_E, 0 if emap is None else int(emap.numel()),
                             sw[0], sw[2], sw[3], int(sw[1]), 0)
    ext.check(lib.b200moe_expert_sort(C.byref(sort_args), stream), "expert_sort")
    mark("sort")

    if b.a_packed is not None:
        q, sf = b.a_packed
        pargs = ext.PackedArgs(q.data_ptr(), sf.data_ptr(), scratch, lp, tokens, b.weight_E, b.k,
                               ext.EP_PAYLOADS["nvfp4" if b.quant_mode == "nvfp4" else "mxfp8"],
                               int(sf.shape[1]), 0)
        ext.check(lib.b200moe_permute_packed(C.byref(pargs), stream), "permute_packed")
    elif b.quant_mode in ("nvfp4", "w4a8_mx"):
        qargs = ext.QuantArgs(b.a.data_ptr(), ex.a1_gscale.data_ptr(), scratch, lp, b.a.stride(0),
                              tokens, b.num_topk, b.weight_E, b.k, int(ex.a1_gscale.numel()), 0)
        fn = lib.b200moe_permute_quant_nvfp4 if b.quant_mode == "nvfp4" else lib.b200moe_permute_quant_mxfp8
        ext.check(fn(C.byref(qargs), stream), "permute_quant")
    mark("quant")

    gargs = ext.GemmArgs(
        ex.w1_fp4.data_ptr(), ex.w1_blockscale.data_ptr(), _ptr(ex.w1_blockscale_rows),
        ex.w1_alphas.data_ptr(), ex.w2_fp4.data_ptr(), ex.w2_blockscale.data_ptr(), ex.w2_alphas.data_ptr(),
        ex.a2_gscale.data_ptr(), b.a.data_ptr(), scratch, lp, _ptr(b.fc1_tap), b.a.stride(0),
        tokens, b.num_topk, b.weight_E, b.k, b.n, recipe, act,
        1 if (b.w13_layout == "w31" and is_gated_moe_activation(b.activation)) else 0,
        int(ex.a2_gscale.numel()),
        float(b.swiglu_limit) if b.swiglu_limit is not None else 0.0,
        float(b.swiglu_alpha if b.swiglu_alpha is not None else 1.0),
        float(b.swiglu_beta if b.swiglu_beta is not None else 0.0), 0,
        1 if (b.quant_mode == "w4a16" and ex.plan.source_format == "fp4_e8m0_k32") else 0,
        # router weights into FC1 (every route's rows times its weight before the activation); the
        # combine below then adds the routes with unit weights
        b.topk_weights.data_ptr() if b.apply_router_weight_on_input else None)
    unit = 1 if b.apply_router_weight_on_input else 0
    ext.check(lib.b200moe_grouped_gemm1_act(C.byref(gargs), stream), "grouped_gemm1_act")
    mark("gemm1")
    if b.activation_amax is not None:
        aargs = ext.AmaxArgs(scratch, lp, b.activation_amax.data_ptr(), tokens * b.num_topk, b.weight_E, b.k, b.n,
                             int(b.layer_idx), recipe)
        ext.check(lib.b200moe_activation_amax(C.byref(aargs), stream), "activation_amax")
    ext.check(lib.b200moe_grouped_gemm2(C.byref(gargs), stream), "grouped_gemm2")
    mark("gemm2")

    if b.skip_combine:
        return out
    if not b.f32_only:
        cargs = ext.CombineArgs(b.topk_weights.data_ptr(), out.data_ptr(), scratch, lp, out.stride(0),
                                tokens, b.num_topk, b.k, 0, float(b.output_scale), unit)
        ext.check(lib.b200moe_combine(C.byref(cargs), stream), "combine")
        mark("combine")
    if b.output_f32 is not None:
        targs = ext.CombineArgs(b.topk_weights.data_ptr(), b.output_f32.data_ptr(), scratch, lp,
                                b.output_f32.stride(0), tokens, b.num_topk, b.k, 1,
                                float(b.output_scale), unit)
        ext.check(lib.b200moe_combine(C.byref(targs), stream), "combine(f32 tap)")
        if b.f32_only:
            mark("combine")
    return out


def check_device_status(binding: TPMoEFP4Binding) -> None:
    """Synchronise and raise if a device-side bounded wait ran out during the last run."""
    st = binding.status.cpu()
    if int(st[0]) != 0:
        raise RuntimeError(f"moe.fused_moe kernel gave up waiting (site {int(st[1])}); results are invalid")


# =============================================================================================
# routing and the sparse block (gate -> top-k -> experts)
# =============================================================================================
@dataclass(frozen=True, kw_only=True)
class B12XTopKRouting:
    """Top-k routing selection (reference _impl.py:644-652)."""

    topk_weights: torch.Tensor
    topk_ids: torch.Tensor
    router_logits: torch.Tensor | None = None
    flat_ids: torch.Tensor | None = None
    flat_weights: torch.Tensor | None = None


@dataclass(frozen=True)
class TPMoERouteWorkspace:
    """Views into the route part of a scratch arena: gate logits, top-k outputs, arrival counters."""

    router_logits: torch.Tensor
    topk_logits: torch.Tensor
    topk_ids: torch.Tensor
    topk_weights: torch.Tensor
    counters: torch.Tensor


@dataclass(frozen=True)
class TPMoEWorkspace:
    """The caller-owned scratch of the sparse block: a scratch plan and the ONE uint8 tensor sized by
    it.  It stands where the reference passes its workspace objects as ``scratch`` to
    ``bind_route`` / ``bind_sparse`` (_impl.py:7849-7958); nothing in it is allocated after
    construction."""

    plan: TPMoEScratchPlan
    storage: torch.Tensor

    def __post_init__(self) -> None:
        if not isinstance(self.plan, TPMoEScratchPlan):
            raise TypeError("plan must be a TPMoEScratchPlan")
        scratch_tensor(self.storage, self.plan.scratch_specs(), owner="TP MoE")

    @classmethod
    def allocate(cls, plan: TPMoEScratchPlan) -> "TPMoEWorkspace":
        spec = plan.scratch_specs()[0]
        return cls(plan, torch.empty(spec.shape, dtype=spec.dtype, device=spec.device))

    def route_views(self, tokens: int, num_experts: int, top_k: int,
                    logits_dtype: torch.dtype) -> TPMoERouteWorkspace | None:
        """Route buffers for ``tokens`` tokens carved from the arena, or None when the plan did not
        price them (``Caps.route_num_experts``) or they do not fit."""
        caps = self.plan.caps
        e_cap = caps.route_num_experts or 0
        if e_cap <= 0 or num_experts > e_cap or tokens > caps.max_tokens or top_k > caps.num_topk:
            return None
        if logits_dtype not in (torch.float32, torch.bfloat16):
            return None
        t_cap, k_cap = caps.max_tokens, caps.num_topk
        base = self.storage
        off = 0

        def take(nbytes_cap: int, count: int, dtype: torch.dtype, shape) -> torch.Tensor:
            nonlocal off
            v = _view(base, off, count, dtype).view(shape)
            off += _align_up(nbytes_cap, _ROUTE_ALIGN)
            return v

        logits = take(t_cap * e_cap * 4, tokens * num_experts, logits_dtype, (tokens, num_experts))
        tl = take(t_cap * k_cap * 4, tokens * top_k, torch.float32, (tokens, top_k))
        ti = take(t_cap * k_cap * 4, tokens * top_k, torch.int32, (tokens, top_k))
        tw = take(t_cap * k_cap * 4, tokens * top_k, torch.float32, (tokens, top_k))
        cnt = take(((t_cap + 3) // 4) * 4, (tokens + 3) // 4, torch.int32, ((tokens + 3) // 4,))
        return TPMoERouteWorkspace(logits, tl, ti, tw, cnt)


def _alloc_route_workspace(tokens: int, num_experts: int, top_k: int, device, logits_dtype) -> TPMoERouteWorkspace:
    if torch.cuda.is_current_stream_capturing():
        raise RuntimeError("route buffers must come from caller-owned scratch during CUDA graph capture "
                           "(plan with Caps.route_num_experts and pass the workspace as scratch)")
    return TPMoERouteWorkspace(
        torch.empty((tokens, num_experts), dtype=logits_dtype, device=device),
        torch.empty((tokens, top_k), dtype=torch.float32, device=device),
        torch.empty((tokens, top_k), dtype=torch.int32, device=device),
        torch.empty((tokens, top_k), dtype=torch.float32, device=device),
        torch.empty(((tokens + 3) // 4,), dtype=torch.int32, device=device))


@dataclass(frozen=True, kw_only=True)
class TPMoERouteBinding:
    """Reference ``TPMoERouteBinding`` (_impl.py:1059-1070).  The last four fields are not in the
    reference's binding: they select the sigmoid scoring the reference only has in its benchmark
    (benchmarks/benchmark_moe.py:1282-1322) and the kernel used for the gate projection."""

    hidden_states: torch.Tensor
    top_k: int
    scratch: TPMoEWorkspace | None = None
    gate_weight: torch.Tensor | None = None
    gate_bias: torch.Tensor | None = None
    router_logits: torch.Tensor | None = None
    renormalize: bool = True
    score_func: str = "softmax"          # "softmax" | "sigmoid"
    selection_bias: torch.Tensor | None = None
    route_scale: float = 1.0
    gate_kernel: str = "auto"            # "auto" | "simt" | "tc"

    def run(self) -> B12XTopKRouting:
        return b12x_route_experts_fast(binding=self)


def _check_route_request(hidden_states, top_k, gate_weight, router_logits) -> None:
    if hidden_states.ndim != 2:
        raise ValueError(f"expected hidden_states with rank 2, got shape {tuple(hidden_states.shape)}")
    if int(top_k) <= 0:
        raise ValueError(f"top_k must be positive, got {top_k}")
    if router_logits is not None and gate_weight is not None:
        raise ValueError("pass either router_logits or gate_weight, not both")
    if router_logits is None and gate_weight is None:
        raise ValueError("expected router_logits or gate_weight")


def build_tp_moe_route_binding(
    *,
    scratch: TPMoEWorkspace | None = None,
    hidden_states: torch.Tensor,
    top_k: int,
    gate_weight: torch.Tensor | None = None,
    gate_bias: torch.Tensor | None = None,
    router_logits: torch.Tensor | None = None,
    renormalize: bool = True,
    score_func: str = "softmax",
    selection_bias: torch.Tensor | None = None,
    route_scale: float = 1.0,
    gate_kernel: str = "auto",
) -> TPMoERouteBinding:
    """Reference ``build_tp_moe_route_binding`` (_impl.py:7849-7883)."""
    if scratch is not None and not isinstance(scratch, TPMoEWorkspace):
        raise TypeError("scratch must be a TP MoE scratch object or None")
    _check_route_request(hidden_states, top_k, gate_weight, router_logits)
    if gate_kernel not in ext.GATE_KERNELS:
        raise ValueError(f"unsupported gate_kernel {gate_kernel!r}")
    return TPMoERouteBinding(hidden_states=hidden_states, top_k=int(top_k), scratch=scratch, gate_weight=gate_weight,
                             gate_bias=gate_bias, router_logits=router_logits, renormalize=bool(renormalize),
                             score_func=score_func, selection_bias=selection_bias, route_scale=float(route_scale),
                             gate_kernel=gate_kernel)


_DT_CODE = {torch.float32: 0, torch.bfloat16: 1}


def b12x_route_experts_fast(*, binding: TPMoERouteBinding) -> B12XTopKRouting:
    """Gate projection (optional) and top-k routing (reference ``b12x_route_experts_fast``
    _impl.py:11356-11490).  With ``gate_weight`` the projection and the router are ONE launch
    (``b200moe_gate_route``); with ``router_logits`` only the router runs.  With a workspace as
    ``scratch`` every buffer is a view into it: nothing is allocated and the call can be captured."""
    if not isinstance(binding, TPMoERouteBinding):
        raise TypeError("binding must be a TPMoERouteBinding")
    b = binding
    hs, top_k, gw, gb, logits = b.hidden_states, b.top_k, b.gate_weight, b.gate_bias, b.router_logits
    _check_route_request(hs, top_k, gw, logits)
    if logits is None:
        if gw.ndim != 2:
            raise ValueError(f"expected gate_weight with rank 2, got shape {tuple(gw.shape)}")
        if gw.shape[1] != hs.shape[1]:
            raise ValueError(f"gate_weight hidden-size mismatch: expected {hs.shape[1]}, got {gw.shape[1]}")
        if gb is not None:
            if gb.ndim != 1:
                raise ValueError(f"expected gate_bias with rank 1, got shape {tuple(gb.shape)}")
            if gb.shape[0] != gw.shape[0]:
                raise ValueError(f"gate_bias expert mismatch: expected {gw.shape[0]}, got {gb.shape[0]}")
        num_experts = int(gw.shape[0])
        logits_dtype = torch.result_type(hs, gw)
    else:
        if logits.ndim != 2:
            raise ValueError(f"expected router_logits with rank 2, got shape {tuple(logits.shape)}")
        if logits.shape[0] != hs.shape[0]:
            raise ValueError(f"router_logits batch mismatch: expected {hs.shape[0]}, got {logits.shape[0]}")
        num_experts = int(logits.shape[1])
        logits_dtype = logits.dtype
    if top_k > num_experts:
        raise ValueError(f"top_k={top_k} exceeds num_experts={num_experts}")
    if not hs.is_cuda:
        raise ValueError("route requires CUDA tensors (there is no CPU path)")
    if num_experts > 1024:
        raise ValueError(f"route supports up to 1024 experts, got {num_experts}")
    if b.score_func not in ("softmax", "sigmoid"):
        raise ValueError(f"unsupported score_func {b.score_func!r}")
    tokens = int(hs.shape[0])
    ws = None if b.scratch is None else b.scratch.route_views(tokens, num_experts, top_k, logits_dtype)
    if ws is None:
        ws = _alloc_route_workspace(tokens, num_experts, top_k, hs.device, logits_dtype)
    if logits is not None:
        if not logits.is_contiguous():
            ws.router_logits.copy_(logits)
            logits = ws.router_logits
        route_topk(logits, ws.topk_logits, ws.topk_ids, ws.topk_weights, renormalize=b.renormalize,
                   score_func=b.score_func, selection_bias=b.selection_bias, route_scale=b.route_scale)
    else:
        for name, t in (("hidden_states", hs), ("gate_weight", gw)):
            if t.dtype not in _DT_CODE:
                raise ValueError(f"{name} must be float32 or bfloat16, got {t.dtype}")
        if gb is not None and gb.dtype not in _DT_CODE:
            raise ValueError(f"gate_bias must be float32 or bfloat16, got {gb.dtype}")
        if hs.stride(1) != 1 or not gw.is_contiguous() or (gb is not None and not gb.is_contiguous()):
            raise ValueError("hidden_states must be row-contiguous; gate_weight and gate_bias contiguous")
        if b.score_func == "sigmoid":
            mode = "sigmoid"
        else:
            mode = "softmax_topk" if b.renormalize else "raw"
        sel = b.selection_bias
        if sel is not None:
            if mode != "sigmoid":
                raise ValueError("selection_bias is only used with score_func='sigmoid'")
            if sel.dtype != torch.float32 or sel.numel() != num_experts or not sel.is_contiguous():
                raise ValueError("selection_bias must be contiguous float32 [experts]")
        args = ext.GateRouteArgs(
            hs.data_ptr(), gw.data_ptr(), _ptr(gb), ws.router_logits.data_ptr(), ws.counters.data_ptr(), _ptr(sel),
            ws.topk_logits.data_ptr(), ws.topk_ids.data_ptr(), ws.topk_weights.data_ptr(), None, hs.stride(0),
            tokens, num_experts, int(hs.shape[1]), top_k, _DT_CODE[hs.dtype], _DT_CODE[gw.dtype],
            _DT_CODE[gb.dtype] if gb is not None else 0, ext.ROUTE_MODES[mode], 1 if b.renormalize else 0,
            float(b.route_scale), ext.GATE_KERNELS[b.gate_kernel], 0)
        ext.check(ext.load().b200moe_gate_route(C.byref(args), _stream_ptr(hs.device)), "gate_route")
        logits = ws.router_logits
    return B12XTopKRouting(topk_weights=ws.topk_weights, topk_ids=ws.topk_ids, router_logits=logits,
                           flat_ids=ws.topk_ids.view(-1), flat_weights=ws.topk_weights.view(-1))


@dataclass(frozen=True, kw_only=True)
class TPMoESparseFP4Binding:
    """Route + experts in one binding (reference ``TPMoESparseFP4Binding`` _impl.py:1073-1097)."""

    hidden_states: torch.Tensor
    experts: B12XFP4ExpertWeights
    scratch: TPMoEWorkspace
    routing: B12XTopKRouting | None = None
    top_k: int | None = None
    gate_weight: torch.Tensor | None = None
    gate_bias: torch.Tensor | None = None
    router_logits: torch.Tensor | None = None
    renormalize_topk: bool = True
    routed_scaling_factor: float = 1.0
    output: torch.Tensor | None = None
    return_routing: bool = False
    input_scales_static: bool = False
    fast_math: bool | None = None
    quant_mode: str | None = None
    swiglu_limit: float | None = None
    swiglu_alpha: float | None = None
    swiglu_beta: float | None = None
    activation_amax: torch.Tensor | None = None
    layer_idx: int | None = None
    score_func: str = "softmax"
    selection_bias: torch.Tensor | None = None
    route_scale: float = 1.0

    def run(self):
        return b12x_sparse_moe_fp4(binding=self)


def _select_prepared_quant_mode(experts: B12XFP4ExpertWeights, quant_mode: str | None) -> str:
    modes = experts.plan.quant_modes
    if quant_mode is None:
        if len(modes) != 1:
            raise ValueError(f"quant_mode is required: the experts were prepared for {sorted(modes)}")
        return next(iter(modes))
    mode = str(quant_mode).lower()
    if mode not in modes:
        raise ValueError(f"quant_mode={mode!r} was not prepared (prepared: {sorted(modes)})")
    return mode


def build_tp_moe_sparse_fp4_binding(
    *,
    scratch: TPMoEWorkspace,
    hidden_states: torch.Tensor,
    experts: B12XFP4ExpertWeights,
    routing: B12XTopKRouting | None = None,
    top_k: int | None = None,
    gate_weight: torch.Tensor | None = None,
    gate_bias: torch.Tensor | None = None,
    router_logits: torch.Tensor | None = None,
    renormalize_topk: bool = True,
    routed_scaling_factor: float = 1.0,
    output: torch.Tensor | None = None,
    return_routing: bool = False,
    input_scales_static: bool = False,
    fast_math: bool | None = None,
    quant_mode: str | None = None,
    swiglu_limit: float | None = None,
    swiglu_alpha: float | None = None,
    swiglu_beta: float | None = None,
    activation_amax: torch.Tensor | None = None,
    layer_idx: int | None = None,
    score_func: str = "softmax",
    selection_bias: torch.Tensor | None = None,
    route_scale: float = 1.0,
) -> TPMoESparseFP4Binding:
    """Reference ``build_tp_moe_sparse_fp4_binding`` (_impl.py:7886-7958), same keywords."""
    if not isinstance(scratch, TPMoEWorkspace):
        raise TypeError("scratch must be a TP MoE scratch object")
    if hidden_states.ndim != 2:
        raise ValueError(f"expected hidden_states with rank 2, got shape {tuple(hidden_states.shape)}")
    if not isinstance(experts, B12XFP4ExpertWeights):
        raise TypeError("experts must be a B12XFP4ExpertWeights")
    limit, alpha, beta = normalize_swiglu_params(experts.plan.activation, swiglu_limit, swiglu_alpha, swiglu_beta)
    _select_prepared_quant_mode(experts, quant_mode)
    if routing is not None:
        if top_k is not None or gate_weight is not None or gate_bias is not None or router_logits is not None:
            raise ValueError("routing is mutually exclusive with top_k/gate_weight/gate_bias/router_logits")
    elif top_k is None:
        raise ValueError("top_k is required when routing is not provided")
    return TPMoESparseFP4Binding(
        hidden_states=hidden_states, experts=experts, scratch=scratch, routing=routing,
        top_k=None if top_k is None else int(top_k), gate_weight=gate_weight, gate_bias=gate_bias,
        router_logits=router_logits, renormalize_topk=bool(renormalize_topk),
        routed_scaling_factor=float(routed_scaling_factor), output=output, return_routing=bool(return_routing),
        input_scales_static=bool(input_scales_static), fast_math=fast_math, quant_mode=quant_mode,
        swiglu_limit=limit, swiglu_alpha=alpha, swiglu_beta=beta, activation_amax=activation_amax,
        layer_idx=layer_idx, score_func=score_func, selection_bias=selection_bias, route_scale=float(route_scale))


def _validate_sparse_routing(hidden_states: torch.Tensor, routing: B12XTopKRouting) -> None:
    ids, w = routing.topk_ids, routing.topk_weights
    if ids.ndim != 2 or w.ndim != 2 or ids.shape != w.shape:
        raise ValueError("routing.topk_ids and routing.topk_weights must be matching rank-2 tensors")
    if ids.shape[0] != hidden_states.shape[0]:
        raise ValueError(f"routing batch mismatch: expected {hidden_states.shape[0]}, got {ids.shape[0]}")


def b12x_sparse_moe_fp4(*, binding: TPMoESparseFP4Binding):
    """A fully bound ``gate -> top-k -> routed experts`` block (reference ``b12x_sparse_moe_fp4``
    _impl.py:11493-11575).  ``routed_scaling_factor`` rides in the combine kernel instead of a
    separate in-place multiply.  Returns the output, or ``(output, routing)`` with ``return_routing``."""
    if not isinstance(binding, TPMoESparseFP4Binding):
        raise TypeError("binding must be a TPMoESparseFP4Binding")
    b = binding
    mode = _select_prepared_quant_mode(b.experts, b.quant_mode)
    if b.routing is not None:
        if b.top_k is not None or b.gate_weight is not None or b.gate_bias is not None or b.router_logits is not None:
            raise ValueError("routing is mutually exclusive with top_k/gate_weight/gate_bias/router_logits")
        selected = b.routing
    else:
        if b.top_k is None:
            raise ValueError("top_k is required when routing is not provided")
        selected = b12x_route_experts_fast(binding=build_tp_moe_route_binding(
            scratch=b.scratch, hidden_states=b.hidden_states, top_k=b.top_k, gate_weight=b.gate_weight,
            gate_bias=b.gate_bias, router_logits=b.router_logits, renormalize=b.renormalize_topk,
            score_func=b.score_func, selection_bias=b.selection_bias, route_scale=b.route_scale))
    _validate_sparse_routing(b.hidden_states, selected)
    plan = b.scratch.plan
    if plan.caps.quant_mode != mode:
        raise ValueError(f"the scratch was planned for quant_mode={plan.caps.quant_mode!r}, the call asks for {mode!r}")
    core = plan.bind(scratch=b.scratch.storage, a=b.hidden_states, experts=b.experts,
                     topk_weights=selected.topk_weights, topk_ids=selected.topk_ids, output=b.output,
                     input_scales_static=b.input_scales_static, fast_math=b.fast_math,
                     activation_amax=b.activation_amax, layer_idx=b.layer_idx,
                     output_scale=b.routed_scaling_factor)
    out = b12x_moe_fp4(binding=core)
    if b.return_routing:
        return out, selected
    return out


def clear_tp_moe_caches() -> None:
    """Nothing is cached per shape here (kernels are compiled ahead of time)."""
    return None
