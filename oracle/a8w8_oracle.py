"""CPU oracle for the A8W8 preshuffle GEMM path.  TEST INFRASTRUCTURE ONLY.

This file restates, on the CPU with torch/numpy, what the reference
(ROCm/FlyDSL) defines as the correct result of its quantised preshuffle GEMM.
It exists to check the CUDA kernels; nothing in the shipped package imports
it.  Only the test-suite, the smoke check and the CPU-baseline leg of the
benchmark may call into it.

Parity status: PINNED.  The quantiser, the reference weight layout and the
dequantise-and-matmul check are verified against outputs produced by importing
the reference's own ``tests/utils.py`` (see ``tests/golden/make_golden.py`` and
the fixtures it wrote).  The reference holds no stored golden vectors for this
path; it pins results only relationally (kernel vs. its torch check).

Each function names the reference lines it follows (paths are relative to the
reference project root).
"""

from __future__ import annotations

import math

import numpy as np
import torch

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0
INT8_MAX = 127.0

# ---------------------------------------------------------------------------
# quantiser  (tests/utils.py:29-73)
# ---------------------------------------------------------------------------


def dtype_max(dtype: torch.dtype) -> float:
    """Largest finite value of ``dtype`` (tests/utils.py:21-26)."""
    if dtype.is_floating_point:
        return float(torch.finfo(dtype).max)
    return float(torch.iinfo(dtype).max)


def pertoken_quant(x: torch.Tensor, quant_dtype: torch.dtype = torch.int8, dtypeMax=None, scale=None):
    """Symmetric per-row quantisation (tests/utils.py:29-73).

    scale = max(|row|) / dtypeMax with 0 -> 1; non-finite inputs are scrubbed
    to 0 / +-dtypeMax first; y = (x / scale) cast to ``quant_dtype`` by torch's
    own cast (int8: truncation toward zero; e4m3fn: round-to-nearest-even).
    Returns (y, scale[rows, 1] fp32).
    """
    qmax = dtype_max(quant_dtype) if dtypeMax is None else float(dtypeMax)
    h = torch.nan_to_num(x.to(torch.float32), nan=0.0, posinf=qmax, neginf=-qmax)
    if scale is None:
        hi = h.amax(dim=-1, keepdim=True)
        lo = h.amin(dim=-1, keepdim=True)
        s = torch.maximum(hi, -lo) / qmax
        s = torch.where(s == 0, torch.ones_like(s), s)
    else:
        s = scale
    s = torch.nan_to_num(s, nan=1.0, posinf=1.0, neginf=1.0)
    y = (h / s).to(quant_dtype)
    return y, s.to(torch.float32)


def pertoken_quant_rne_int8(x: torch.Tensor):
    """Bench-input quantiser for the INT8 decode config: scale = amax/127 and
    round-to-nearest before the cast (the benchmark definition asks for
    round-to-nearest; the reference helper above truncates)."""
    h = x.to(torch.float32)
    s = h.abs().amax(dim=-1, keepdim=True) / INT8_MAX
    s = torch.where(s == 0, torch.ones_like(s), s)
    y = torch.round(h / s).clamp_(-127, 127).to(torch.int8)
    return y, s


# ---------------------------------------------------------------------------
# weight layouts
# ---------------------------------------------------------------------------


def shuffle_weight_mfma(x: torch.Tensor, layout=(16, 16)) -> torch.Tensor:
    """The reference's MFMA-oriented weight permutation (tests/utils.py:76-96).

    For a [N, K] matrix of e-byte elements the result, read as a flat array, is
    ordered [N/16][K/BK][BK/Kp][16 rows][Kp elems] with BK = 2*layout[1]
    elements and Kp = 16/e elements.  Same shape and dtype out.
    """
    bn, ik = layout
    bk = ik * 2
    kp = 16 // x.element_size()
    n, k = x.shape[-2], x.shape[-1]
    assert n % bn == 0 and k % bk == 0
    v = x.reshape(-1, n // bn, bn, k // bk, bk // kp, kp)
    return v.permute(0, 1, 3, 4, 2, 5).contiguous().view(*x.shape)


def b200_layout_offsets(n: int, k_bytes: int) -> np.ndarray:
    """Byte offset in the B200 preshuffled image of every byte (row, kbyte).

    Layout: [K_bytes/128 k-blocks][N rows][128 bytes], and inside every group of
    8 consecutive rows (a 1024-byte atom) the eight 16-byte chunks of a row are
    XOR-swizzled with the row index modulo 8 — the 128-byte-swizzle K-major
    shared-memory image that both TMA and the tcgen05 matrix descriptors use.
    This is the replacement for the MFMA layout of tests/utils.py:76-96 /
    kernels/gemm/preshuffle_gemm.py:765-780.
    """
    assert k_bytes % 128 == 0 and n % 8 == 0
    r = np.arange(n, dtype=np.int64)[:, None]
    kb = np.arange(k_bytes, dtype=np.int64)[None, :]
    blk = kb // 128
    chunk = (kb % 128) // 16
    within = kb % 16
    return (blk * n + r) * 128 + ((chunk ^ (r % 8)) * 16) + within


def shuffle_weight_b200(x: torch.Tensor) -> torch.Tensor:
    """CPU statement of the B200 preshuffle (same shape/dtype in and out)."""
    n, k = x.shape[-2], x.shape[-1]
    e = x.element_size()
    flat = x.contiguous().view(torch.uint8).reshape(-1, n * k * e).numpy()
    off = b200_layout_offsets(n, k * e).reshape(-1)
    out = np.empty_like(flat)
    out[:, off] = flat
    return torch.from_numpy(out).view(x.dtype).view(*x.shape)


def unshuffle_weight_b200(x: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`shuffle_weight_b200`."""
    n, k = x.shape[-2], x.shape[-1]
    e = x.element_size()
    flat = x.contiguous().view(torch.uint8).reshape(-1, n * k * e).numpy()
    off = b200_layout_offsets(n, k * e).reshape(-1)
    return torch.from_numpy(flat[:, off].copy()).view(x.dtype).view(*x.shape)


def mfma_to_rowmajor(x: torch.Tensor, layout=(16, 16)) -> torch.Tensor:
    """Inverse of :func:`shuffle_weight_mfma` (used to check the converter that
    accepts weights already shuffled by the reference helper)."""
    bn, ik = layout
    bk = ik * 2
    kp = 16 // x.element_size()
    n, k = x.shape[-2], x.shape[-1]
    v = x.reshape(-1, n // bn, k // bk, bk // kp, bn, kp)
    return v.permute(0, 1, 4, 2, 3, 5).contiguous().view(*x.shape)


# ---------------------------------------------------------------------------
# the reference's correctness definition
# ---------------------------------------------------------------------------


def run_torch(a, b, scale_a, scale_b, bias=None, dtype=torch.float32):
    """Dequantise both operands to fp32 and matmul
    (tests/kernels/test_preshuffle_gemm.py:103-113)."""
    af = a.to(torch.float32)
    bf = b.to(torch.float32)
    if scale_a is not None and scale_b is not None:
        af = af * scale_a.reshape(-1, 1)
        bf = bf * scale_b.reshape(-1, 1)
    c = af @ bf.T
    if bias is not None:
        c = c + bias
    return c.to(dtype)


def int32_acc(a_i8: torch.Tensor, b_i8: torch.Tensor) -> torch.Tensor:
    """Exact int32 accumulators of the INT8 path: what the reference's MFMA
    int32 accumulation holds before scaling
    (kernels/gemm/preshuffle_gemm.py:538,739).  Computed exactly: every partial
    sum is an integer below 2**53, so a float64 matmul is exact (an fp32 matmul
    would not be: |acc| may pass 2**24) and much faster than an integer one."""
    k = a_i8.shape[-1]
    assert k * 128 * 128 < 2**31, "int32 accumulators would overflow"
    acc = a_i8.to(torch.float64) @ b_i8.to(torch.float64).T
    return acc.to(torch.int64).to(torch.int32)


def epilogue(acc, scale_a, scale_b, bias=None, kind="none", out_dtype=torch.bfloat16):
    """Fused epilogue in the reference's operation order
    (kernels/gemm/preshuffle_gemm.py:665-714): float(acc); (v*sa[row])*sb[col];
    + float(bias[col]); relu | silu = v/(1+exp(-v)) | tanh-gelu written with a
    non-positive exponent; round-to-nearest-even cast to the output type."""
    v = acc.to(torch.float32)
    if scale_a is not None:
        v = (v * scale_a.reshape(-1, 1).to(torch.float32)) * scale_b.reshape(1, -1).to(torch.float32)
    if kind != "none":
        v = v + bias.to(torch.float32).reshape(1, -1)
    if kind == "bias_relu":
        v = torch.maximum(v, torch.zeros_like(v))
    elif kind == "bias_silu":
        v = v * (1.0 / (1.0 + torch.exp(-v)))
    elif kind == "bias_gelu":
        y = 0.7978845608 * (v + 0.044715 * (v * v * v))
        e = torch.exp(-2.0 * y.abs())
        num = torch.where(y > 0, torch.full_like(y, 2.0), 2.0 * e)
        v = 0.5 * v * (num * (1.0 / (1.0 + e)))
    return v.to(out_dtype)


def check_allclose(a, b, rtol=1e-2, atol=1e-2) -> float:
    """Fraction of elements outside isclose(rtol, atol)
    (tests/test_common.py:353-394 returns this ratio)."""
    ok = torch.isclose(a, b, rtol=rtol, atol=atol)
    return 1.0 - ok.float().mean().item()


def verify_output(c_out, c_ref, atol=1e-2, rtol=1e-2, logits_diff_threshold=2e-3) -> bool:
    """The reference's pass rule (tests/test_common.py:397-423): pass if fewer
    than 5 % of elements mismatch, else pass if 1 - 2<x,y>/(<x,x>+<y,y>) is at
    most ``logits_diff_threshold``."""
    if check_allclose(c_out, c_ref, rtol=rtol, atol=atol) < 0.05:
        return True
    x, y = c_out.double(), c_ref.double()
    den = (x * x + y * y).sum()
    if den == 0:
        return True
    diff = (1 - 2 * (x * y).sum() / den).item()
    if math.isnan(diff):
        return False
    return diff <= logits_diff_threshold


def strict_mismatches(c_out, c_ref, rtol=1e-2, atol=1e-2) -> int:
    """Number of elements outside the all-element bound the build is held to
    (every element within rtol/atol of the fp32 reference)."""
    return int((~torch.isclose(c_out.float(), c_ref.float(), rtol=rtol, atol=atol)).sum().item())


# ---------------------------------------------------------------------------
# work model  (tests/kernels/test_preshuffle_gemm.py:310-313)
# ---------------------------------------------------------------------------


def gemm_flops(m, n, k):
    return 2 * m * n * k


def gemm_bytes(m, n, k, elem_bytes=1):
    return m * k * elem_bytes + n * k * elem_bytes + 2 * m * n + 4 * (m + n)


# ---------------------------------------------------------------------------
# seeded synthetic inputs for the benchmark configurations
# ---------------------------------------------------------------------------


def make_inputs(m, n, k, in_dtype="fp8", seed=0, weight_scale=1.0, rne_int8=False):
    """Seeded N(0,1) activations [m,k] and weights [n,k] (weights optionally
    scaled), quantised per row.  A CPU generator is used so the oracle and the
    GPU run consume identical bytes.  Returns (a_q, b_q, sa[m], sb[n])."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    a = torch.randn(m, k, generator=g, dtype=torch.float32)
    w = torch.randn(n, k, generator=g, dtype=torch.float32)
    if weight_scale != 1.0:
        w = w * weight_scale
    if in_dtype == "fp8":
        a_q, sa = pertoken_quant(a, quant_dtype=FP8)
        b_q, sb = pertoken_quant(w, quant_dtype=FP8)
    elif in_dtype == "int8":
        q = pertoken_quant_rne_int8 if rne_int8 else (lambda t: pertoken_quant(t, quant_dtype=torch.int8))
        a_q, sa = q(a)
        b_q, sb = q(w)
    else:
        raise ValueError(in_dtype)
    return a_q, b_q, sa.reshape(-1), sb.reshape(-1)
