"""Fused MoE layer for B200: route -> sort -> quantise -> FC1 -> activation -> FC2 -> combine.

Same lifecycle as the reference op (b12x/moe/fused_moe/__init__.py:1-39):

    wplan   = fused_moe.plan_weights(quant_modes="nvfp4", source_format="modelopt_nvfp4", ...)
    experts = fused_moe.prepare_weights(plan=wplan, ...)
    plan    = fused_moe.plan(fused_moe.Caps(...))
    spec    = plan.scratch_specs()[0]
    scratch = torch.empty(spec.shape, dtype=spec.dtype, device=spec.device)
    binding = fused_moe.bind(plan, scratch=scratch, a=x, experts=experts,
                             topk_weights=tw, topk_ids=ti)
    out     = fused_moe.run(binding=binding)

Recipes: nvfp4, w4a8_mx, w4a16.  Activations: silu, relu2, swigluoai_uninterleave.
"""

from ..._lib.meta import OpMeta, Provenance, install_lazy_api

META = OpMeta(
    name="fused_moe",
    group="moe",
    api_style="planned",
    entry_points=(
        "Caps", "Plan", "ExecutionPlan", "Binding", "SparseBinding", "RouteBinding", "ExpertWeights",
        "Workspace", "Routing", "WeightsPlan", "plan", "required_nbytes", "plan_execution", "plan_weights",
        "prepare_weights", "bind", "bind_sparse", "bind_route", "run", "run_sparse", "route", "route_topk",
        "is_supported", "clear_caches", "check_device_status",
    ),
    archs=("sm100a",),
    dtypes=("bf16",),
    recipes=("nvfp4", "w4a8_mx", "w4a16"),
    requires=(),
    provenance=Provenance(
        repo="https://github.com/lukealonso/b12x",
        commit="6627d342",
        paths=("b12x/moe/fused_moe/", "b12x/moe/_shared/"),
    ),
    test_path="tests/test_gpu_parity.py",
    notes="C ABI in include/b200moe.h; the FC2-only entry points of the reference "
          "(prepare_fc2_weights, prewarm_fc2, run_fc2) are not part of this operator",
)

install_lazy_api(globals(), META)
