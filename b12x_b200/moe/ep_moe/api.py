"""Public surface of moe.ep_moe (reference ``b12x/moe/ep_moe/api.py:6-54``).

The reference runs this contract on its W4A16 kernel only; here it is the fused layer of
``moe.fused_moe`` with a route-expert map, so every recipe of the weight plan works."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .._shared.execution import MoEWeightPreparationPlan
from ..fused_moe import _impl as F


@dataclass(frozen=True)
class ExpertMap:
    """One rank's frozen global-to-local expert map (the role of the reference's ``EPExpertMap``,
    b12x/moe/ep_moe/_impl.py:62-83).  ``validate_static`` detects a map that was replaced, moved or
    written to since it was prepared: the kernels read it on every call, and a captured graph keeps
    its address."""

    tensor: torch.Tensor
    global_num_experts: int
    local_num_experts: int
    device: torch.device
    _fingerprint: tuple

    @staticmethod
    def _fingerprint_of(t: torch.Tensor) -> tuple:
        try:
            version = int(t._version)
        except RuntimeError:          # inference-mode tensors carry no version counter
            version = None
        return (t.data_ptr(), str(t.device), version)

    def validate_static(self) -> None:
        then, now = self._fingerprint, self._fingerprint_of(self.tensor)
        if now[0] != then[0]:
            raise RuntimeError("EP expert_map storage changed after preparation")
        if now[1] != then[1]:
            raise RuntimeError("EP expert_map device changed after preparation")
        if then[2] is not None and now[2] != then[2]:
            raise RuntimeError("EP expert_map was mutated after preparation")


def prepare_expert_map(expert_map: torch.Tensor, *, local_num_experts: int,
                       global_num_experts: int | None = None,
                       device: torch.device | str | None = None) -> ExpertMap:
    """Check and freeze a rank's expert map: an int32 vector over the GLOBAL experts whose entries
    are a local expert id or -1, every local id used exactly once (a bijection from this rank's
    global experts onto ``range(local_num_experts)``; contract of the reference's
    ``prepare_ep_expert_map``, b12x/moe/ep_moe/_impl.py:86-153).  Reads the map on the host, so it
    must run before CUDA graph capture."""
    if not isinstance(expert_map, torch.Tensor) or expert_map.dtype != torch.int32:
        raise TypeError("expert_map must be a torch.Tensor of dtype torch.int32")
    if expert_map.ndim != 1 or not expert_map.is_contiguous():
        raise ValueError("expert_map must be a contiguous rank-1 tensor")
    if expert_map.is_cuda and torch.cuda.is_current_stream_capturing():
        raise RuntimeError("EP expert_map must be prepared before CUDA graph capture")
    want = expert_map.device if device is None else torch.device(device)
    if want.type == "cuda" and want.index is None:
        want = torch.device("cuda", expert_map.device.index or 0)
    if expert_map.device != want:
        raise ValueError(f"expert_map must be on {want}, got {expert_map.device}")
    n_global, n_local = int(expert_map.numel()), int(local_num_experts)
    if global_num_experts is not None and int(global_num_experts) != n_global:
        raise ValueError(f"expert_map global expert count mismatch: expected {int(global_num_experts)}, got {n_global}")
    if n_global <= 0 or n_local <= 0:
        raise ValueError("global_num_experts and local_num_experts must be positive")
    if n_local > n_global:
        raise ValueError(f"local_num_experts={n_local} exceeds global_num_experts={n_global}")
    host = expert_map.detach().to("cpu", torch.int64)
    out_of_range = host[(host < -1) | (host >= n_local)]
    if out_of_range.numel():
        raise ValueError("expert_map values must be -1 or valid local expert ids; "
                         f"found {int(out_of_range[0])} for local_num_experts={n_local}")
    uses = torch.bincount(host[host >= 0], minlength=n_local)
    if not bool((uses == 1).all()):
        bad = int((uses != 1).nonzero()[0])
        raise ValueError(f"expert_map must map every local expert id exactly once: local id {bad} "
                         f"occurs {int(uses[bad])} times")
    return ExpertMap(tensor=expert_map, global_num_experts=n_global, local_num_experts=n_local, device=want,
                     _fingerprint=ExpertMap._fingerprint_of(expert_map))


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
