"""BF16 -> MXFP8 row quantiser for B200 (reference: ``b12x/quantization/mxfp8/api.py:5-18``,
``b12x/_lib/quant/mxfp8_rows.py:398-434``): E4M3 payload, one UE8M0 scale (power of two, rounded up)
per 32 values, written row-major and in the 128x4-swizzled MMA layout."""

from .api import is_supported, quantize_rows

__all__ = ["quantize_rows", "is_supported"]
