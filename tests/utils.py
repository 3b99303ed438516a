"""Same import path as the reference's helper module (``from tests.utils import
pertoken_quant, shuffle_weight``, tests/kernels/test_preshuffle_gemm.py:38),
re-exporting this package's implementations."""

from flydsl_b200.utils import get_dtype_max, pertoken_quant, shuffle_weight, unshuffle_weight  # noqa: F401
