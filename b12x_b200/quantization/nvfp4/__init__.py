"""BF16 -> NVFP4 row quantiser for B200 (reference: ``b12x/quantization/nvfp4/__init__.py:1-15``).

Quantises a ``[M, K]`` BF16 tensor (M, K multiples of 128, as in the reference) into packed FP4 values
plus E4M3 scales in the 128x4-swizzled MMA layout (scale vector 16).  ``plan(m, k)`` fixes the
shape, ``allocate_outputs`` sizes the output pair, ``run`` launches into the caller's outputs
(allocation-free, capture safe).  There is no bind step: the outputs container is the binding.

    from b12x_b200.quantization import nvfp4

    plan = nvfp4.plan(m=256, k=512)
    outs = nvfp4.allocate_outputs(plan)
    nvfp4.run(plan=plan, x=x_bf16, global_scale=gs, outputs=outs)
"""

from .api import Outputs, Plan, allocate_outputs, is_supported, plan, run

__all__ = ["Outputs", "Plan", "plan", "allocate_outputs", "run", "is_supported"]
