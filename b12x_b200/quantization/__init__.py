"""Standalone activation quantisers (the reference's ``b12x.quantization`` ops): the numerics of the
layer's own quantisation stage, offered as operators so that an upstream layer can hand over
pre-quantised activations."""

from . import mxfp8, nvfp4  # noqa: F401

__all__ = ["nvfp4", "mxfp8"]
