"""Public surface of ``moe.fused_moe``: the reference's names (b12x/moe/fused_moe/api.py:6-122)
bound to this library's implementations."""

from __future__ import annotations

import torch

from ..._lib import ext
from .._shared.execution import MoEWeightPreparationPlan as WeightsPlan
from .._shared.routing import route_topk
from ._impl import B12XFP4ExpertWeights as ExpertWeights
from ._impl import B12XTopKRouting as Routing
from ._impl import TPMoEFP4Binding as Binding
from ._impl import TPMoEPlan as ExecutionPlan
from ._impl import TPMoERouteBinding as RouteBinding
from ._impl import TPMoEScratchCaps as Caps
from ._impl import TPMoEScratchPlan as Plan
from ._impl import TPMoESparseFP4Binding as SparseBinding
from ._impl import TPMoEWorkspace as Workspace
from ._impl import b12x_moe_fp4 as run
from ._impl import b12x_route_experts_fast as route
from ._impl import b12x_sparse_moe_fp4 as run_sparse
from ._impl import build_tp_moe_route_binding as bind_route
from ._impl import build_tp_moe_sparse_fp4_binding as bind_sparse
from ._impl import check_device_status
from ._impl import clear_tp_moe_caches as clear_caches
from ._impl import plan_b12x_fp4_moe_weights as plan_weights
from ._impl import plan_tp_moe_execution as plan_execution
from ._impl import plan_tp_moe_scratch as plan
from ._impl import prepare_b12x_fp4_moe_weights as prepare_weights
from ._impl import tp_moe_required_nbytes as required_nbytes


def bind(plan: Plan, **kwargs) -> Binding:
    """Bind runtime tensors and caller-owned scratch to a plan.  Views only, never allocates."""
    return plan.bind(**kwargs)


def is_supported(device=None) -> bool:
    """True on an sm_100 device with the extension built."""
    if not torch.cuda.is_available() or not ext.lib_path().exists():
        return False
    dev = torch.device("cuda" if device is None else device)
    major, _minor = torch.cuda.get_device_capability(dev)
    return major == 10


__all__ = [
    "Caps", "Plan", "ExecutionPlan", "Binding", "SparseBinding", "RouteBinding", "ExpertWeights", "Workspace",
    "Routing", "WeightsPlan", "plan", "required_nbytes", "plan_execution", "plan_weights",
    "prepare_weights", "bind", "bind_sparse", "bind_route", "run", "run_sparse", "route",
    "route_topk", "is_supported", "clear_caches", "check_device_status",
]
