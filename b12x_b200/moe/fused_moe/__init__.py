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

from .api import *  # noqa: F401,F403
from .api import __all__  # noqa: F401
