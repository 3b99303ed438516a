"""MXFP8 x MXFP8 preshuffle GEMM (E4M3 codes, one E8M0 scale per 32 elements of
K on both operands): the B200 counterpart of the reference's block-scaled GEMM
``kernels/gemm/mxfp4_preshuffle.py`` in its a_dtype = b_dtype = "fp8"
configuration, with the call shape its tests use
(tests/kernels/test_preshuffle_gemm.py:48-81, 602-700):

    launch = compile_mxfp8_preshuffle_gemm(N=N, K=K, out_dtype="bf16")
    a_q, sa = per_1x32_f8_quant(a)                  # codes [M, K], scales uint8 [M, K/32]
    w_q, sw = per_1x32_f8_quant(w)
    launch(c, a_q, shuffle_weight(w_q), shuffle_scale(sa), shuffle_scale(sw), bias, M, N, stream)

``shuffle_weight`` is the one of the per-channel-scaled GEMM (same weight
image); ``shuffle_scale`` plays the role of the reference's ``shuffle_scale_w4``
and writes the scale image the tensor core's block-scaled instruction wants
(see include/flyb200.h).  The multiply runs as
``tcgen05.mma.kind::mxf8f6f4.block_scale`` with the scale factors in TMEM.
"""

from __future__ import annotations

import torch

from ... import _lib
from .preshuffle_gemm import _stream_handle

_TORCH_OUT = {"bf16": torch.bfloat16, "fp16": torch.float16, "f16": torch.float16}
FP8_MAX = 448.0


def per_1x32_f8_quant(x: torch.Tensor):
    """Per-1x32 MXFP8 quantiser, torch ops on the tensor's device: (codes
    float8_e4m3fn [..., K], E8M0 scales uint8 [..., K/32]); same arithmetic as the
    reference helper (tests/kernels/utils/gemm_common_utils.py:53-72, 773-790)."""
    shape = x.shape
    if shape[-1] % 32 != 0:
        raise ValueError("K must be a multiple of 32")
    flat = x.contiguous().view(-1, 32).float()
    max_abs = torch.amax(torch.abs(flat), dim=-1).clamp_min(1e-30)
    u32 = (max_abs / FP8_MAX).view(torch.int32)
    exponent = (u32 >> 23) & 0xFF
    round_case = ((u32 & 0x400000) > 0) & (((u32 & 0x200000) > 0) | ((u32 & 0x1FFFFF) > 0) | (exponent > 0))
    exponent = torch.where(round_case, exponent + 1, exponent)
    exponent = torch.where(((u32 >> 23) & 0xFF) == 0xFF, torch.full_like(exponent, 0xFF), exponent) & 0xFF
    bits = exponent << 23
    bits = torch.where(exponent == 0, torch.full_like(bits, 0x00400000), bits)
    bits = torch.where(exponent == 0xFF, torch.full_like(bits, 0x7F800001), bits)
    scale_f32 = bits.view(torch.float32).clamp_min(1e-30)
    q = (flat / scale_f32.view(-1, 1)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.view(shape).contiguous(), exponent.to(torch.uint8).view(*shape[:-1], shape[-1] // 32).contiguous()


def shuffle_scale(scale: torch.Tensor) -> torch.Tensor:
    """E8M0 scales [rows, K/32] (uint8) -> the B200 scale image (1-D uint8,
    ``flyb200_mx_scale_image_bytes(rows, K)`` bytes, rows padded to whole 128-row tiles)."""
    if scale.dim() != 2 or scale.element_size() != 1:
        raise ValueError("scale must be a 2-D one-byte tensor [rows, K/32]")
    rows, kb32 = scale.shape
    if kb32 % 4 != 0:
        raise ValueError("K must be a multiple of 128")
    if not scale.is_cuda:
        raise ValueError("scale must be a CUDA tensor")
    lib = _lib.load()
    src = scale.contiguous().view(torch.uint8)
    out = torch.empty(int(lib.flyb200_mx_scale_image_bytes(rows, kb32 * 32)), dtype=torch.uint8, device=scale.device)
    with torch.cuda.device(scale.device):
        _lib.check(
            lib.flyb200_mx_scale_image(out.data_ptr(), src.data_ptr(), rows, kb32 * 32,
                                       torch.cuda.current_stream(scale.device).cuda_stream),
            "mx_scale_image",
        )
    return out


class MxFp8Gemm:
    """The callable returned by :func:`compile_mxfp8_preshuffle_gemm`."""

    def __init__(self, N, K, out_dtype):
        self.N, self.K, self.out_dtype = int(N), int(K), out_dtype
        self._out = _lib.OUT_FP16 if _TORCH_OUT[out_dtype] == torch.float16 else _lib.OUT_BF16

    def __call__(self, arg_c, arg_a, arg_b, arg_scale_a, arg_scale_b, arg_bias, i32_m, i32_n, stream=None):
        M, n_rt = int(i32_m), int(i32_n)
        if n_rt != self.N:
            raise ValueError(f"N passed at call time ({n_rt}) differs from the N the launcher was built for ({self.N})")
        if M < 0:
            raise ValueError("M must be non-negative")
        lib = _lib.load()
        need = (
            ("c", arg_c, M * self.N), ("a", arg_a, M * self.K), ("b", arg_b, self.N * self.K),
            ("scale_a", arg_scale_a, int(lib.flyb200_mx_scale_image_bytes(max(M, 1), self.K))),
            ("scale_b", arg_scale_b, int(lib.flyb200_mx_scale_image_bytes(self.N, self.K))),
        )
        for name, t, n in need:
            if not isinstance(t, torch.Tensor) or not t.is_cuda or not t.is_contiguous():
                raise ValueError(f"{name} must be a contiguous CUDA tensor")
            if t.numel() < n:
                raise ValueError(f"{name} holds {t.numel()} elements, the launch needs {n}")
        if arg_c.dtype != _TORCH_OUT[self.out_dtype]:
            raise ValueError(f"c must be {_TORCH_OUT[self.out_dtype]}, got {arg_c.dtype}")
        for name, t in (("a", arg_a), ("b", arg_b), ("scale_a", arg_scale_a), ("scale_b", arg_scale_b)):
            if t.element_size() != 1:
                raise ValueError(f"{name} must be a one-byte tensor")
        if arg_bias is not None and arg_bias.numel() != 0:
            raise ValueError("the MXFP8 GEMM has no bias epilogue")
        if M == 0:
            return None
        with torch.cuda.device(arg_c.device):
            _lib.check(
                lib.flyb200_gemm_mxfp8(arg_c.data_ptr(), arg_a.data_ptr(), arg_b.data_ptr(), arg_scale_a.data_ptr(),
                                       arg_scale_b.data_ptr(), M, self.N, self.K, self._out, _stream_handle(stream) or None),
                "gemm_mxfp8",
            )
        return None


def compile_mxfp8_preshuffle_gemm(*, N, K, tile_m=128, tile_n=128, tile_k=256, out_dtype="bf16", a_dtype="fp8", b_dtype="fp8"):
    """Builder.  ``tile_*`` are accepted as hints (the kernel works on 128x128 tiles
    and 128-element k-blocks).  Only the fp8 x fp8 configuration is built; the
    reference's fp4 / fp6 operand types raise ``ValueError``."""
    if a_dtype != "fp8" or b_dtype != "fp8":
        raise ValueError(f"only a_dtype = b_dtype = 'fp8' is built for B200, got {a_dtype!r} x {b_dtype!r}")
    if out_dtype not in _TORCH_OUT:
        raise ValueError(f"out_dtype must be 'bf16' or 'fp16', got {out_dtype!r}")
    if int(K) % 128 != 0 or int(N) % 128 != 0:
        raise ValueError(f"MXFP8 GEMM needs N % 128 == 0 and K % 128 == 0, got N={N}, K={K}")
    return MxFp8Gemm(N, K, out_dtype)


__all__ = ["compile_mxfp8_preshuffle_gemm", "per_1x32_f8_quant", "shuffle_scale"]
