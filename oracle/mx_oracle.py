"""TEST INFRASTRUCTURE — CPU restatement of the reference's MXFP8 (per-1x32 E8M0
block-scaled E4M3) quantiser and of its dequantise-and-matmul check.  Only
tests, the smoke check and the benchmark's CPU-baseline leg may import this
module; the product never does.

Parity status: PINNED.  ``tests/golden/mx_fp8.npz`` was produced by the
reference's own ``per_1x32_f8_quant`` / ``e8m0_to_f32``
(tests/kernels/utils/gemm_common_utils.py:53-72, 773-790) and the reference
formula of tests/kernels/test_preshuffle_gemm.py:651-654, run on CPU by
``tests/golden/make_golden_mx.py``; ``tests/test_mx_oracle_golden.py`` checks
the functions below against it bit for bit.
"""

from __future__ import annotations

import torch

BLOCK = 32  # elements that share one scale


def f32_to_e8m0(x):
    """Biased power-of-two exponent of x, rounded up when the mantissa is >= 1.5
    (tests/kernels/utils/gemm_common_utils.py:53-60)."""
    u32 = x.contiguous().view(torch.int32)
    exponent = ((u32 >> 23) & 0xFF).to(torch.int32)
    nan_case = exponent == 0xFF
    round_case = ((u32 & 0x400000) > 0) & (((u32 & 0x200000) > 0) | ((u32 & 0x1FFFFF) > 0) | (exponent > 0))
    exponent = torch.where(round_case, exponent + 1, exponent)
    exponent = torch.where(nan_case, torch.full_like(exponent, 0xFF), exponent)
    return (exponent & 0xFF).to(torch.uint8)


def e8m0_to_f32(scale):
    """2 ** (byte - 127); byte 0 is 2 ** -127, byte 255 NaN (gemm_common_utils.py:63-71)."""
    b = scale.view(torch.uint8).to(torch.int32)
    bits = b << 23
    bits = torch.where(b == 0, torch.full_like(bits, 0x00400000), bits)
    bits = torch.where(b == 0xFF, torch.full_like(bits, 0x7F800001), bits)
    return bits.view(torch.float32)


def per_1x32_f8_quant(x):
    """(codes float8_e4m3fn [..., K], scales uint8 E8M0 [..., K/32]) (gemm_common_utils.py:773-790)."""
    fp8_max = float(torch.finfo(torch.float8_e4m3fn).max)
    shape = x.shape
    flat = x.contiguous().view(-1, BLOCK).float()
    max_abs = torch.amax(torch.abs(flat), dim=-1).clamp_min(1e-30)
    scale = f32_to_e8m0(max_abs / fp8_max)
    scale_f32 = e8m0_to_f32(scale).clamp_min(1e-30)
    q = (flat / scale_f32.view(-1, 1)).clamp(-fp8_max, fp8_max).to(torch.float8_e4m3fn)
    return q.view(shape).contiguous(), scale.view(*shape[:-1], shape[-1] // BLOCK).contiguous()


def dequant(codes, scale):
    return codes.float() * e8m0_to_f32(scale).repeat_interleave(BLOCK, dim=-1)


def mx_gemm(a_codes, scale_a, b_codes, scale_b):
    """fp32 [M, N]: dequantise both operands, torch.mm (tests/kernels/test_preshuffle_gemm.py:651-654)."""
    return torch.mm(dequant(a_codes, scale_a), dequant(b_codes, scale_b).T).to(torch.float32)


def scale_image(scale):
    """The scale layout the B200 kernel reads, stated with torch ops: rows padded to
    a multiple of 128, then [K/128][rows/128][32][4][4] bytes with
    byte ((r % 32) * 16 + (r // 32) * 4 + j) of a 512-byte atom holding the scale of
    row r of the 128-row tile for the j-th 32-element block of the 128-element k-block."""
    rows, kb32 = scale.shape
    assert kb32 % 4 == 0
    pad = (-rows) % 128
    s = torch.cat([scale.view(torch.uint8), torch.zeros(pad, kb32, dtype=torch.uint8)]) if pad else scale.view(torch.uint8)
    t = s.view(-1, 4, 32, kb32 // 4, 4)  # [row tile, r // 32, r % 32, k-block, j]
    return t.permute(3, 0, 2, 1, 4).contiguous().view(-1)


def make_inputs(m, n, k, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    a = torch.randn(m, k, generator=g, dtype=torch.float32)
    b = torch.randn(n, k, generator=g, dtype=torch.float32)
    a_q, sa = per_1x32_f8_quant(a)
    b_q, sb = per_1x32_f8_quant(b)
    return a_q, sa, b_q, sb


# ---------------------------------------------------------------------------
# MXFP4: E2M1 codes, two per byte, one E8M0 scale per 32 elements
# (tests/kernels/utils/gemm_common_utils.py:14-50, 162-276, 675-705)
# Parity status: PINNED by tests/golden/mx_fp4.npz (tests/golden/make_golden_mx4.py
# ran the reference's per_1x32_f4_quant / mxfp4_to_f32 / e8m0_to_f32 and the
# reference formula of tests/kernels/test_preshuffle_gemm.py:404-411 on CPU).
# ---------------------------------------------------------------------------
FP4_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)  # magnitudes of codes 0..7; bit 3 is the sign
_FP4_MIDPOINTS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)  # between code c and c + 1


def f32_to_fp4_codes(x):
    """E2M1 code (uint8, 0..15) of every element: round to nearest, ties to the code
    with an even mantissa bit, magnitudes of 6 and above saturate to 6, the sign bit
    (also of -0.0) is kept (gemm_common_utils.py:162-276 with ebits=2, mbits=1)."""
    a = x.float().abs()
    code = torch.zeros_like(a, dtype=torch.int32)
    for c, mid in enumerate(_FP4_MIDPOINTS):
        up = (a > mid) | ((a == mid) & bool(c & 1))  # at a tie the odd code moves up to its even neighbour
        code = code + up.to(torch.int32)
    code = code | (torch.signbit(x.float()).to(torch.int32) << 3)
    return code.to(torch.uint8)


def pack_fp4(codes):
    """Two codes per byte, the even element in the low nibble (gemm_common_utils.py:142-149)."""
    assert codes.shape[-1] % 2 == 0
    return (codes[..., 1::2] << 4 | codes[..., 0::2]).contiguous()


def mxfp4_to_f32(packed):
    """fp32 value of every E2M1 code of a packed tensor [..., K/2] -> [..., K] (gemm_common_utils.py:23-50)."""
    b = packed.view(torch.uint8)
    codes = torch.stack([b & 0xF, b >> 4], dim=-1).flatten(-2)
    table = torch.tensor(FP4_VALUES + tuple(-v for v in FP4_VALUES), dtype=torch.float32)
    return table[codes.long()]


def per_1x32_f4_quant(x):
    """(packed codes uint8 [..., K/2], scales uint8 E8M0 [..., K/32]): scale = E8M0 of
    blockmax / 4 (4 = the largest power of two E2M1 holds), codes = x / scale rounded
    to E2M1 (gemm_common_utils.py:675-705)."""
    shape = x.shape
    flat = x.contiguous().view(-1, BLOCK).float()
    max_abs = torch.amax(torch.abs(flat), dim=-1)
    scale = f32_to_e8m0(max_abs / 4.0)
    y = flat / e8m0_to_f32(scale).view(-1, 1)
    codes = f32_to_fp4_codes(y).view(*shape)
    return pack_fp4(codes), scale.view(*shape[:-1], shape[-1] // BLOCK).contiguous()


def dequant_fp4(packed, scale):
    return mxfp4_to_f32(packed) * e8m0_to_f32(scale).repeat_interleave(BLOCK, dim=-1)


def mx4_gemm(a_packed, scale_a, b_packed, scale_b):
    """fp32 [M, N]: dequantise both operands, torch.mm (tests/kernels/test_preshuffle_gemm.py:404-411)."""
    return torch.mm(dequant_fp4(a_packed, scale_a), dequant_fp4(b_packed, scale_b).T).to(torch.float32)


def make_inputs_fp4(m, n, k, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    a = torch.randn(m, k, generator=g, dtype=torch.float32)
    b = torch.randn(n, k, generator=g, dtype=torch.float32)
    a_q, sa = per_1x32_f4_quant(a)
    b_q, sb = per_1x32_f4_quant(b)
    return a_q, sa, b_q, sb


# ---------------------------------------------------------------------------
# MXFP6 (E2M3) activations, and the byte containers of the mixed kinds
# (tests/kernels/utils/gemm_common_utils.py:708-770; reference formula of
# tests/kernels/test_preshuffle_gemm.py:530-538)
# Parity status: PINNED by tests/golden/mx_fp6.npz (tests/golden/make_golden_mx6.py ran the
# reference's per_1x32_f6_quant / pack_fp6_e2m3 / fp6_e2m3_to_f32 and the A6W4 formula on CPU).
# ---------------------------------------------------------------------------
def _fp6_magnitudes():
    v = []
    for c in range(32):
        e, m = (c >> 3) & 3, c & 7
        v.append(m / 8.0 if e == 0 else (2.0 ** (e - 1)) * (1.0 + m / 8.0))
    return v


FP6_VALUES = tuple(_fp6_magnitudes())  # magnitudes of codes 0..31; bit 5 is the sign


def f32_to_fp6_codes(x):
    """E2M3 code (uint8, low 6 bits) of every element: round to nearest, ties to the code with an
    even mantissa bit, magnitudes of 7.5 and above saturate, sign kept (gemm_common_utils.py:162-276
    with ebits=2, mbits=3)."""
    a = x.float().abs()
    code = torch.zeros_like(a, dtype=torch.int32)
    for c in range(31):
        mid = (FP6_VALUES[c] + FP6_VALUES[c + 1]) / 2.0
        code = code + ((a > mid) | ((a == mid) & bool(c & 1))).to(torch.int32)
    code = code | (torch.signbit(x.float()).to(torch.int32) << 5)
    return code.to(torch.uint8)


def fp6_to_f32(codes):
    table = torch.tensor(FP6_VALUES + tuple(-v for v in FP6_VALUES), dtype=torch.float32)
    return table[(codes & 0x3F).long()]


def pack_fp6(codes):
    """Four 6-bit codes -> three bytes, little-endian bit stream (gemm_common_utils.py:708-721)."""
    g = codes.to(torch.int32).unflatten(-1, (-1, 4)) & 0x3F
    e0, e1, e2, e3 = g.unbind(dim=-1)
    out = torch.stack([((e1 & 3) << 6) | e0, ((e2 & 15) << 4) | (e1 >> 2), (e3 << 2) | (e2 >> 4)], dim=-1).to(torch.uint8)
    return out.reshape(*codes.shape[:-1], codes.shape[-1] // 4 * 3).contiguous()


def per_1x32_f6_quant(x):
    """(a_pad uint8 [M, K]: per 32 elements 24 bytes of packed codes + 8 zero bytes, scales uint8
    [M, K/32], codes uint8 [M, K]) (gemm_common_utils.py:744-770)."""
    m, k = x.shape
    flat = x.contiguous().view(-1, BLOCK).float()
    scale = f32_to_e8m0(torch.amax(torch.abs(flat), dim=-1) / 4.0)  # 4 = the largest power of two below 7.5
    codes = f32_to_fp6_codes(flat / e8m0_to_f32(scale).view(-1, 1)).view(m, k)
    a_pad = torch.zeros(m, k // BLOCK, BLOCK, dtype=torch.uint8)
    a_pad[:, :, :24] = pack_fp6(codes).view(m, k // BLOCK, 24)
    return a_pad.view(m, k), scale.view(m, k // BLOCK), codes


def fp6_containers(codes):
    """6-bit codes [.., K] -> byte containers [.., K]: every 16 codes become 12 packed bytes + 4 zero bytes."""
    g = pack_fp6(codes).unflatten(-1, (-1, 12))
    return torch.cat([g, torch.zeros(*g.shape[:-1], 4, dtype=torch.uint8)], dim=-1).flatten(-2).contiguous()


def fp4_containers(packed):
    """packed 4-bit codes [.., K/2] -> byte containers [.., K]: every 16 codes (8 bytes) + 8 zero bytes."""
    g = packed.view(torch.uint8).unflatten(-1, (-1, 8))
    return torch.cat([g, torch.zeros_like(g)], dim=-1).flatten(-2).contiguous()


def a6w4_gemm(a_codes, scale_a, b_packed, scale_b):
    """fp32 [M, N] of MXFP6 activations x MXFP4 weights (tests/kernels/test_preshuffle_gemm.py:530-538)."""
    a = fp6_to_f32(a_codes) * e8m0_to_f32(scale_a).repeat_interleave(BLOCK, dim=-1)
    return torch.mm(a, dequant_fp4(b_packed, scale_b).T).to(torch.float32)


def a8w4_gemm(a_fp8, scale_a, b_packed, scale_b):
    return torch.mm(dequant(a_fp8, scale_a), dequant_fp4(b_packed, scale_b).T).to(torch.float32)
