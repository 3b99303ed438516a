"""MXFP4 x MXFP4 preshuffle GEMM (E2M1 codes, two per byte, one E8M0 scale per 32
elements of K on both operands): the B200 counterpart of the reference's
``kernels/gemm/mxfp4_preshuffle.py`` in its a_dtype = b_dtype = "fp4"
configuration, with the call shape its tests use
(tests/kernels/test_preshuffle_gemm.py:343-466):

    launch = compile_mxfp4_preshuffle_gemm(N=N, K=K, out_dtype="bf16")
    a_q, sa = per_1x32_f4_quant(a)                 # packed codes [M, K/2] uint8, scales uint8 [M, K/32]
    w_q, sw = per_1x32_f4_quant(w)
    launch(c, a_q, shuffle_weight_w4(w_q), shuffle_scale_w4(sa), shuffle_scale_w4(sw), bias, M, N, stream)

``shuffle_weight_w4`` writes the same weight image as ``shuffle_weight`` (the
packed codes are just bytes: a 128-byte swizzled row holds 256 elements) and
``shuffle_scale_w4`` the scale image of the MXFP8 GEMM.  The multiply runs as
``tcgen05.mma.kind::mxf4.block_scale.scale_vec::2X`` with the scale factors in
TMEM.

The mixed configurations - MXFP6 (E2M3) or MXFP8 activations with MXFP4 weights,
``a_dtype="fp6"`` / ``"fp8"`` (tests/kernels/test_preshuffle_gemm.py:472-587) - run as
``tcgen05.mma.kind::mxf8f6f4.block_scale``, which takes sub-byte codes only in
byte-sized containers (16 codes per 16 bytes, the unused bytes padding).  The
launcher converts the reference's activation layout on every call and wants the
weights as ``shuffle_weight_w4(w_q, ..., for_a_dtype="fp6")`` (containers, one
byte per code); a packed 4-bit image is expanded on first sight and cached by
address.  The weight stream of these kinds therefore has FP8's size: the memory
saving of 4-bit weights comes with ``a_dtype="fp4"`` only.
"""

from __future__ import annotations

import torch

from ... import _lib
from ...utils import shuffle_weight
from .mxfp8_preshuffle import shuffle_scale
from .preshuffle_gemm import _stream_handle

_TORCH_OUT = {"bf16": torch.bfloat16, "fp16": torch.float16, "f16": torch.float16}
_FP4_MIDPOINTS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)  # between E2M1 code c and c + 1
_FP4_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def _e8m0_of(x: torch.Tensor) -> torch.Tensor:
    """Biased exponent byte of a non-negative fp32 tensor, rounded up when the mantissa is 1.5 or more
    (the reference's f32_to_e8m0, tests/kernels/utils/gemm_common_utils.py:53-60), as int32."""
    u32 = x.contiguous().view(torch.int32)
    exponent = (u32 >> 23) & 0xFF
    round_case = ((u32 & 0x400000) > 0) & (((u32 & 0x200000) > 0) | ((u32 & 0x1FFFFF) > 0) | (exponent > 0))
    rounded = torch.where(round_case, exponent + 1, exponent)
    return torch.where(exponent == 0xFF, torch.full_like(exponent, 0xFF), rounded) & 0xFF


def per_1x32_f4_quant(x: torch.Tensor):
    """Per-1x32 MXFP4 quantiser, torch ops on the tensor's device: (packed E2M1 codes
    uint8 [..., K/2], E8M0 scales uint8 [..., K/32]).  Scale = E8M0 of blockmax / 4, codes =
    x / scale rounded to nearest (ties to the even code, magnitudes >= 6 saturate), the even
    element in the low nibble - the arithmetic of the reference helper
    (tests/kernels/utils/gemm_common_utils.py:675-705)."""
    shape = x.shape
    if shape[-1] % 32 != 0:
        raise ValueError("K must be a multiple of 32")
    flat = x.contiguous().view(-1, 32).float()
    exponent = _e8m0_of(torch.amax(torch.abs(flat), dim=-1) / 4.0)
    bits = exponent << 23
    bits = torch.where(exponent == 0, torch.full_like(bits, 0x00400000), bits)
    bits = torch.where(exponent == 0xFF, torch.full_like(bits, 0x7F800001), bits)
    y = flat / bits.view(torch.float32).view(-1, 1)
    mag = y.abs()
    code = torch.zeros_like(mag, dtype=torch.int32)
    for c, mid in enumerate(_FP4_MIDPOINTS):
        code += ((mag > mid) | ((mag == mid) & bool(c & 1))).to(torch.int32)
    code |= torch.signbit(y).to(torch.int32) << 3
    code = code.view(*shape).to(torch.uint8)
    packed = (code[..., 1::2] << 4 | code[..., 0::2]).contiguous()
    return packed, exponent.to(torch.uint8).view(*shape[:-1], shape[-1] // 32).contiguous()


def mxfp4_to_f32(packed: torch.Tensor) -> torch.Tensor:
    """fp32 value of every code of a packed tensor [..., K/2] -> [..., K]."""
    b = packed.view(torch.uint8)
    codes = torch.stack([b & 0xF, b >> 4], dim=-1).flatten(-2)
    table = torch.tensor(_FP4_VALUES + tuple(-v for v in _FP4_VALUES), dtype=torch.float32, device=packed.device)
    return table[codes.long()]


def fp4_containers(packed: torch.Tensor) -> torch.Tensor:
    """Packed 4-bit codes [N, K/2] -> byte containers [N, K] for the mixed kinds: every 16 codes
    (8 bytes) are followed by 8 bytes of padding."""
    g = packed.view(torch.uint8).unflatten(-1, (-1, 8))
    return torch.cat([g, torch.zeros_like(g)], dim=-1).flatten(-2).contiguous()


def fp6_containers_from_padded(a_pad: torch.Tensor) -> torch.Tensor:
    """The reference's activation layout for MXFP6 (per 32 elements 24 bytes of packed codes + 8 zero
    bytes, tests/kernels/utils/gemm_common_utils.py:744-770) -> byte containers [M, K]: every 16
    codes (12 bytes) followed by 4 bytes of padding."""
    m, k = a_pad.shape
    v = a_pad.view(torch.uint8).view(m, k // 32, 32)
    out = torch.zeros(m, k // 32, 2, 16, dtype=torch.uint8, device=a_pad.device)
    out[:, :, 0, :12] = v[:, :, 0:12]
    out[:, :, 1, :12] = v[:, :, 12:24]
    return out.view(m, k)


def pack_fp6_e2m3(codes: torch.Tensor) -> torch.Tensor:
    """Four 6-bit codes -> three bytes, little-endian bit stream (gemm_common_utils.py:708-721)."""
    g = codes.to(torch.int32).unflatten(-1, (-1, 4)) & 0x3F
    e0, e1, e2, e3 = g.unbind(dim=-1)
    out = torch.stack([((e1 & 3) << 6) | e0, ((e2 & 15) << 4) | (e1 >> 2), (e3 << 2) | (e2 >> 4)], dim=-1).to(torch.uint8)
    return out.reshape(*codes.shape[:-1], codes.shape[-1] // 4 * 3).contiguous()


_FP6_VALUES = tuple((c & 7) / 8.0 if ((c >> 3) & 3) == 0 else (2.0 ** (((c >> 3) & 3) - 1)) * (1.0 + (c & 7) / 8.0)
                    for c in range(32))


def fp6_e2m3_to_f32(codes: torch.Tensor) -> torch.Tensor:
    table = torch.tensor(_FP6_VALUES + tuple(-v for v in _FP6_VALUES), dtype=torch.float32, device=codes.device)
    return table[(codes & 0x3F).long()]


def per_1x32_f6_quant(x: torch.Tensor):
    """Per-1x32 MXFP6 (E2M3) quantiser of an activation matrix [M, K], torch ops on the tensor's
    device; returns what the reference helper returns (gemm_common_utils.py:744-770): the padded
    packed codes uint8 [M, K] (per 32 elements 24 bytes + 8 zero bytes), the E8M0 scales uint8
    [M, K/32], and the unpacked codes uint8 [M, K]."""
    if x.dim() != 2 or x.shape[-1] % 32 != 0:
        raise ValueError("x must be [M, K] with K a multiple of 32")
    m, k = x.shape
    flat = x.contiguous().view(-1, 32).float()
    exponent = _e8m0_of(torch.amax(torch.abs(flat), dim=-1) / 4.0)
    bits = exponent << 23
    bits = torch.where(exponent == 0, torch.full_like(bits, 0x00400000), bits)
    bits = torch.where(exponent == 0xFF, torch.full_like(bits, 0x7F800001), bits)
    y = flat / bits.view(torch.float32).view(-1, 1)
    mag = y.abs()
    code = torch.zeros_like(mag, dtype=torch.int32)
    for c in range(31):
        mid = (_FP6_VALUES[c] + _FP6_VALUES[c + 1]) / 2.0
        code += ((mag > mid) | ((mag == mid) & bool(c & 1))).to(torch.int32)
    code |= torch.signbit(y).to(torch.int32) << 5
    codes = code.view(m, k).to(torch.uint8)
    a_pad = torch.zeros(m, k // 32, 32, dtype=torch.uint8, device=x.device)
    a_pad[:, :, :24] = pack_fp6_e2m3(codes).view(m, k // 32, 24)
    return a_pad.view(m, k), exponent.to(torch.uint8).view(m, k // 32).contiguous(), codes


def shuffle_weight_w4(src: torch.Tensor, NLane: int = 16, gate_up: bool = False, moe_gemm: bool = False, *,
                      for_a_dtype: str = "fp4") -> torch.Tensor:
    """Packed weight codes [N, K/2] -> the B200 weight image.  Signature of the reference helper
    (tests/kernels/utils/gemm_common_utils.py:607-642); ``NLane`` describes the MFMA lane layout
    there and is ignored, the MoE forms are not built.  ``for_a_dtype`` (not in the reference):
    "fp4" gives the image of the packed codes (N * K/2 bytes, for the fp4 x fp4 GEMM); "fp6" or
    "fp8" the image of the codes in byte containers (N * K bytes) that the mixed kinds read."""
    if gate_up or moe_gemm:
        raise NotImplementedError("the mixture-of-experts forms of the FP4 weight shuffle are not built")
    if src.dim() != 2 or src.element_size() != 1:
        raise ValueError("src must be the packed code matrix [N, K/2] (one byte per two codes)")
    if for_a_dtype not in ("fp4", "fp6", "fp8"):
        raise ValueError(f"for_a_dtype must be 'fp4', 'fp6' or 'fp8', got {for_a_dtype!r}")
    if for_a_dtype == "fp4":
        return shuffle_weight(src.view(torch.uint8))
    return shuffle_weight(fp4_containers(src))


def shuffle_scale_w4(src: torch.Tensor, experts_cnt: int = 1, gate_up: bool = False) -> torch.Tensor:
    """E8M0 scales [rows, K/32] -> the B200 scale image (signature of the reference helper,
    tests/kernels/utils/gemm_common_utils.py:645-672; one expert only)."""
    if experts_cnt != 1 or gate_up:
        raise NotImplementedError("the mixture-of-experts forms of the scale shuffle are not built")
    return shuffle_scale(src)


_FORMATS = {"fp8": 0, "fp6": 3, "fp4": 5}  # FLYB200_MXFMT_E4M3 / E2M3 / E2M1


class MxMixedGemm:
    """The callable returned by :func:`compile_mxfp4_preshuffle_gemm` for ``a_dtype`` "fp6" or "fp8"
    with ``b_dtype="fp4"``: same call shape; activations in the reference's layout for that dtype."""

    def __init__(self, N, K, out_dtype, a_dtype):
        self.N, self.K, self.out_dtype, self.a_dtype = int(N), int(K), out_dtype, a_dtype
        self._out = _lib.OUT_FP16 if _TORCH_OUT[out_dtype] == torch.float16 else _lib.OUT_BF16
        self._expanded: dict = {}  # (data_ptr, numel) of a packed weight image -> its container image

    def prepare_weights(self, b_packed_image: torch.Tensor) -> torch.Tensor:
        """Container image of a packed 4-bit weight image (what ``shuffle_weight_w4(w_q)`` returns
        without ``for_a_dtype``): un-shuffle, expand, shuffle again.  Cached by address; call
        :meth:`forget` when the weights at that address change."""
        from ...utils import unshuffle_weight

        key = (b_packed_image.data_ptr(), b_packed_image.numel())
        img = self._expanded.get(key)
        if img is None:
            rows = unshuffle_weight(b_packed_image.view(torch.uint8).view(self.N, self.K // 2))
            img = shuffle_weight(fp4_containers(rows)).view(-1)
            self._expanded[key] = img
        return img

    def forget(self, b_packed_image: torch.Tensor) -> None:
        self._expanded.pop((b_packed_image.data_ptr(), b_packed_image.numel()), None)

    def __call__(self, arg_c, arg_a, arg_b, arg_scale_a, arg_scale_b, arg_bias, i32_m, i32_n, stream=None):
        M, n_rt = int(i32_m), int(i32_n)
        if n_rt != self.N:
            raise ValueError(f"N passed at call time ({n_rt}) differs from the N the launcher was built for ({self.N})")
        if M < 0:
            raise ValueError("M must be non-negative")
        lib = _lib.load()
        for name, t in (("c", arg_c), ("a", arg_a), ("b", arg_b), ("scale_a", arg_scale_a), ("scale_b", arg_scale_b)):
            if not isinstance(t, torch.Tensor) or not t.is_cuda or not t.is_contiguous():
                raise ValueError(f"{name} must be a contiguous CUDA tensor")
        if arg_c.dtype != _TORCH_OUT[self.out_dtype]:
            raise ValueError(f"c must be {_TORCH_OUT[self.out_dtype]}, got {arg_c.dtype}")
        if arg_c.numel() < M * self.N or arg_a.numel() < M * self.K or arg_a.element_size() != 1:
            raise ValueError("c or a is smaller than the launch needs (a: one byte per code)")
        if arg_scale_a.numel() < int(lib.flyb200_mx_scale_image_bytes(max(M, 1), self.K)) or \
                arg_scale_b.numel() < int(lib.flyb200_mx_scale_image_bytes(self.N, self.K)):
            raise ValueError("a scale image is smaller than the launch needs")
        if arg_bias is not None and arg_bias.numel() != 0:
            raise ValueError("the block-scaled GEMMs have no bias epilogue")
        if arg_b.numel() == self.N * self.K:
            w = arg_b
        elif arg_b.numel() == self.N * self.K // 2:
            w = self.prepare_weights(arg_b)
        else:
            raise ValueError(f"b holds {arg_b.numel()} bytes: neither the container image ({self.N * self.K}) nor the packed one")
        if M == 0:
            return None
        s = _stream_handle(stream)
        with torch.cuda.device(arg_c.device):
            a = arg_a.view(torch.uint8).view(-1)[: M * self.K].view(M, self.K)
            if self.a_dtype == "fp6":
                ext = torch.cuda.ExternalStream(s, device=arg_c.device) if s else torch.cuda.default_stream(arg_c.device)
                with torch.cuda.stream(ext):  # the conversion runs on the launch stream, ahead of the GEMM
                    a = fp6_containers_from_padded(a)
            _lib.check(
                lib.flyb200_gemm_mx_mixed(arg_c.data_ptr(), a.data_ptr(), w.data_ptr(), arg_scale_a.data_ptr(),
                                          arg_scale_b.data_ptr(), M, self.N, self.K, _FORMATS[self.a_dtype], _FORMATS["fp4"],
                                          self._out, s or None),
                "gemm_mx_mixed",
            )
            if self.a_dtype == "fp6":
                a.record_stream(ext)  # the temporary must outlive the kernel that reads it
        return None


class MxFp4Gemm:
    """The callable returned by :func:`compile_mxfp4_preshuffle_gemm`."""

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
            ("c", arg_c, M * self.N), ("a", arg_a, M * self.K // 2), ("b", arg_b, self.N * self.K // 2),
            ("scale_a", arg_scale_a, int(lib.flyb200_mx_scale_image_bytes(max(M, 1), self.K))),
            ("scale_b", arg_scale_b, int(lib.flyb200_mx_scale_image_bytes(self.N, self.K))),
        )  # fmt: skip
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
            raise ValueError("the MXFP4 GEMM has no bias epilogue")
        if M == 0:
            return None
        with torch.cuda.device(arg_c.device):
            _lib.check(
                lib.flyb200_gemm_mxfp4(arg_c.data_ptr(), arg_a.data_ptr(), arg_b.data_ptr(), arg_scale_a.data_ptr(),
                                       arg_scale_b.data_ptr(), M, self.N, self.K, self._out, _stream_handle(stream) or None),
                "gemm_mxfp4",
            )
        return None


def compile_mxfp4_preshuffle_gemm(*, N, K, tile_m=128, tile_n=128, tile_k=256, out_dtype="bf16", a_dtype="fp4", b_dtype="fp4"):
    """Builder for 4-bit weights: ``a_dtype`` "fp4" (both operands packed, ``kind::mxf4``), or
    "fp6" / "fp8" (mixed, ``kind::mxf8f6f4`` on byte containers).  ``tile_*`` are accepted as
    hints.  fp8 x fp8 is ``compile_mxfp8_preshuffle_gemm``."""
    if b_dtype != "fp4" or a_dtype not in ("fp4", "fp6", "fp8"):
        raise ValueError(f"a_dtype must be 'fp4', 'fp6' or 'fp8' and b_dtype 'fp4' here, got {a_dtype!r} x {b_dtype!r}")
    if out_dtype not in _TORCH_OUT:
        raise ValueError(f"out_dtype must be 'bf16' or 'fp16', got {out_dtype!r}")
    if int(K) % 256 != 0 or int(N) % 128 != 0:
        raise ValueError(f"MXFP4 GEMM needs N % 128 == 0 and K % 256 == 0, got N={N}, K={K}")
    if a_dtype == "fp4":
        return MxFp4Gemm(N, K, out_dtype)
    return MxMixedGemm(N, K, out_dtype, a_dtype)


__all__ = ["compile_mxfp4_preshuffle_gemm", "per_1x32_f4_quant", "mxfp4_to_f32", "shuffle_weight_w4", "shuffle_scale_w4",
           "per_1x32_f6_quant", "fp6_e2m3_to_f32", "pack_fp6_e2m3", "fp4_containers", "fp6_containers_from_padded"]
