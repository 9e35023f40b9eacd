"""b12x_b200: the ``moe.fused_moe`` operator of b12x, rebuilt for B200 (sm_100a)."""

__version__ = "0.1.0"
