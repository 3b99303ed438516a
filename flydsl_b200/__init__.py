"""flydsl_b200: the quantised A8W8 preshuffle GEMM of ROCm/FlyDSL, rebuilt for
NVIDIA B200 (sm_100a) behind the reference's own Python operator surface.

    from flydsl_b200 import compile_preshuffle_gemm, shuffle_weight, pertoken_quant
    from flydsl_b200 import compiler as flyc      # flyc.compile(launch_fn, *args)
"""

from .kernels.gemm.preshuffle_gemm import compile_preshuffle_gemm  # noqa: F401
from .utils import pertoken_quant, shuffle_weight, unshuffle_weight  # noqa: F401
from . import compiler  # noqa: F401

__all__ = ["compile_preshuffle_gemm", "shuffle_weight", "unshuffle_weight", "pertoken_quant", "compiler"]
