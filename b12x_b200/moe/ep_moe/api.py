"""Public surface of moe.ep_moe (reference ``b12x/moe/ep_moe/api.py:6-54``).

The reference runs this contract on its W4A16 kernel only; here it is the fused layer of
``moe.fused_moe`` with a route-expert map, so every recipe of the weight plan works."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .._shared.execution import MoEWeightPreparationPlan
from ..fused_moe import _impl as F


def _tensor_version(t: torch.Tensor) -> int | None:
    try:
        return int(t._version)
    except RuntimeError:      # tensors made in inference mode have no version counter
        return None


@dataclass(frozen=True)
class ExpertMap:
    """A validated, static global-to-local expert map (reference ``EPExpertMap`` _impl.py:62-83)."""

    tensor: torch.Tensor
    global_num_experts: int
    local_num_experts: int
    device: torch.device
    _data_ptr: int
    _version: int | None

    def validate_static(self) -> None:
        if self.tensor.data_ptr() != self._data_ptr:
            raise RuntimeError("EP expert_map storage changed after preparation")
        version = _tensor_version(self.tensor)
        if self._version is not None and version != self._version:
            raise RuntimeError("EP expert_map was mutated after preparation")
        if self.tensor.device != self.device:
            raise RuntimeError("EP expert_map device changed after preparation")


def prepare_expert_map(expert_map: torch.Tensor, *, local_num_experts: int,
                       global_num_experts: int | None = None,
                       device: torch.device | str | None = None) -> ExpertMap:
    """Validate and freeze one rank's global-to-local expert map: every local id must occur exactly
    once, other entries are -1 (reference ``prepare_ep_expert_map`` _impl.py:86-153; may
    synchronise with the device, so call it before graph capture)."""
    if not isinstance(expert_map, torch.Tensor):
        raise TypeError("expert_map must be a torch.Tensor")
    if expert_map.dtype != torch.int32:
        raise TypeError("expert_map must have dtype torch.int32")
    if expert_map.ndim != 1 or not expert_map.is_contiguous():
        raise ValueError("expert_map must be a contiguous rank-1 tensor")
    if expert_map.device.type == "cuda" and torch.cuda.is_current_stream_capturing():
        raise RuntimeError("EP expert_map must be prepared before CUDA graph capture")
    expected_device = expert_map.device if device is None else torch.device(device)
    if expected_device.type == "cuda" and expected_device.index is None:
        expected_device = torch.device("cuda", expert_map.device.index or 0)
    if expert_map.device != expected_device:
        raise ValueError(f"expert_map must be on {expected_device}, got {expert_map.device}")
    global_e = int(expert_map.numel())
    if global_num_experts is not None and global_e != int(global_num_experts):
        raise ValueError(f"expert_map global expert count mismatch: expected {int(global_num_experts)}, got {global_e}")
    local_e = int(local_num_experts)
    if global_e <= 0:
        raise ValueError("global_num_experts must be positive")
    if local_e <= 0:
        raise ValueError("local_num_experts must be positive")
    if local_e > global_e:
        raise ValueError(f"local_num_experts={local_e} exceeds global_num_experts={global_e}")
    values = expert_map.detach().cpu().tolist()
    invalid = [v for v in values if v < -1 or v >= local_e]
    if invalid:
        raise ValueError("expert_map values must be -1 or valid local expert ids; "
                         f"found {invalid[0]} for local_num_experts={local_e}")
    mapped = sorted(v for v in values if v >= 0)
    if mapped != list(range(local_e)):
        raise ValueError(f"expert_map must map every local expert id exactly once: expected "
                         f"{list(range(local_e))}, got {mapped}")
    return ExpertMap(tensor=expert_map, global_num_experts=global_e, local_num_experts=local_e,
                     device=expected_device, _data_ptr=expert_map.data_ptr(), _version=_tensor_version(expert_map))


@dataclass(frozen=True, kw_only=True)
class Caps:
    """Capacity and weight metadata of one EP rank (reference ``EPMoEScratchCaps`` _impl.py:157-212)."""

    max_tokens: int
    num_topk: int
    global_num_experts: int
    device: torch.device | str
    weight_plan: MoEWeightPreparationPlan
    apply_router_weight_on_input: bool = False
    swiglu_limit: float | None = None
    swiglu_alpha: float | None = None
    swiglu_beta: float | None = None
    quant_mode: str | None = None      # default: the first recipe of the weight plan

    def __post_init__(self) -> None:
        object.__setattr__(self, "global_num_experts", int(self.global_num_experts))
        if not isinstance(self.weight_plan, MoEWeightPreparationPlan):
            raise TypeError("weight_plan must be a MoEWeightPreparationPlan")
        if self.global_num_experts <= 0:
            raise ValueError("global_num_experts must be positive")
        if self.weight_plan.num_experts > self.global_num_experts:
            raise ValueError("local expert count cannot exceed global expert count: "
                             f"local={self.weight_plan.num_experts}, global={self.global_num_experts}")
        if self.apply_router_weight_on_input:
            raise NotImplementedError("apply_router_weight_on_input is not built")
        mode = self.quant_mode or sorted(self.weight_plan.quant_modes)[0]
        object.__setattr__(self, "quant_mode", mode)

    @property
    def local_num_experts(self) -> int:
        return self.weight_plan.num_experts


@dataclass(frozen=True)
class Plan:
    """Scratch plan of one EP rank: the fused layer's plan plus the global expert count."""

    caps: Caps
    inner: F.TPMoEScratchPlan

    def scratch_specs(self):
        return self.inner.scratch_specs()

    def bind(self, *, scratch, a, experts, topk_weights, topk_ids, expert_map: ExpertMap,
             output: torch.Tensor | None = None, **kwargs) -> "Binding":
        if not isinstance(expert_map, ExpertMap):
            raise TypeError("expert_map must come from prepare_expert_map")
        if expert_map.global_num_experts != self.caps.global_num_experts:
            raise ValueError("expert_map does not cover this plan's global experts")
        if expert_map.local_num_experts != self.caps.local_num_experts:
            raise ValueError("expert_map does not match the local weight plan")
        inner = self.inner.bind(scratch=scratch, a=a, experts=experts, topk_weights=topk_weights,
                                topk_ids=topk_ids, output=output, route_expert_map=expert_map.tensor, **kwargs)
        return Binding(inner=inner, expert_map=expert_map)


@dataclass(frozen=True)
class Binding:
    """One allocation-free launch binding (reference ``EPMoEFP4Binding`` _impl.py:453-480)."""

    inner: F.TPMoEFP4Binding
    expert_map: ExpertMap

    def run(self) -> torch.Tensor:
        return run(binding=self)


def plan(caps: Caps) -> Plan:
    """Scratch plan for ``caps`` (reference ``plan_ep_moe_scratch`` _impl.py:363-450)."""
    if not isinstance(caps, Caps):
        raise TypeError("caps must be an ep_moe.Caps")
    inner = F.plan_tp_moe_scratch(F.TPMoEScratchCaps(
        max_tokens=caps.max_tokens, num_topk=caps.num_topk, device=caps.device, weight_plan=caps.weight_plan,
        quant_mode=caps.quant_mode, swiglu_limit=caps.swiglu_limit, swiglu_alpha=caps.swiglu_alpha,
        swiglu_beta=caps.swiglu_beta))
    return Plan(caps=caps, inner=inner)


def bind(plan: Plan, **kwargs) -> Binding:
    """Bind runtime tensors and caller-owned scratch to a plan (views only, capture safe)."""
    return plan.bind(**kwargs)


def run(*, binding: Binding) -> torch.Tensor:
    """Execute one EP rank and return its local partial ``[tokens, K]``: routes whose expert is not
    held here contribute nothing, a token without local routes gives a zero row (reference
    ``b12x_ep_moe_fp4`` _impl.py:483-528).  The caller sums the partials over the EP group."""
    if not isinstance(binding, Binding):
        raise TypeError("binding must be an ep_moe.Binding")
    binding.expert_map.validate_static()
    return F.b12x_moe_fp4(binding=binding.inner)


def is_supported(device=None) -> bool:
    from .. import fused_moe

    return fused_moe.is_supported(device)
