"""Mixture-of-experts operators."""
from . import ep_moe, fused_moe  # noqa: F401
