"""Mixture-of-experts operators."""
from . import fused_moe  # noqa: F401
