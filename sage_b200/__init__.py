"""sage_b200: the SAGE packed-weight matmul for NVIDIA B200 (sm_100a).

Importing the package does not load the CUDA library; the first operator call does, and
raises if `libsage_b200.so` has not been built (`python -m sage_b200.build`).
"""

from .linear import SAGELinear
from .ops import sage, sage_dequantize, sage_forward, sage_forward_scratch, sage_grouped
from .sphquant import SPHQuantLinear, sph_dequantize, sphquant
from .synthetic import synthetic_sage, synthetic_sphquant

__all__ = [
    "SAGELinear",
    "SPHQuantLinear",
    "sage",
    "sage_dequantize",
    "sage_forward",
    "sage_forward_scratch",
    "sage_grouped",
    "sph_dequantize",
    "sphquant",
    "synthetic_sage",
    "synthetic_sphquant",
]
