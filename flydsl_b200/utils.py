"""Host-side helpers of the operator surface: the per-token quantiser and the
weight preshuffle, with the names, arguments and results of the reference's
``tests/utils.py`` (pertoken_quant :29-73, shuffle_weight :76-96).

``pertoken_quant`` is input preparation and runs as torch ops on whatever
device its argument lives on.  ``shuffle_weight`` keeps the reference's call
but writes the B200 weight image — [K*e/128][N][128 B], 128-byte swizzled, the
shared-memory form TMA and tcgen05 consume — instead of the MFMA one; for CUDA
tensors it runs the library's permutation kernel.
"""

from __future__ import annotations

import torch

from . import _lib

_FP8_TYPES = tuple(getattr(torch, n) for n in ("float8_e4m3fn", "float8_e4m3fnuz", "float8_e5m2") if hasattr(torch, n))


def get_dtype_max(dtype: torch.dtype) -> float:
    return torch.finfo(dtype).max if dtype.is_floating_point else torch.iinfo(dtype).max


_X_DTYPES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def _kernel_can_quantise(x, scale, x_scale, scale_dtype, quant_dtype, dtypeMax) -> bool:
    if not (isinstance(x, torch.Tensor) and x.is_cuda and x.is_contiguous() and x.dim() >= 1):
        return False
    if scale is not None or x_scale is not None or dtypeMax is not None or scale_dtype != torch.float32:
        return False
    if x.dtype not in _X_DTYPES or quant_dtype not in (torch.int8, getattr(torch, "float8_e4m3fn", None)):
        return False
    k = x.shape[-1]
    return k > 0 and k % (4 if x.dtype == torch.float32 else 8) == 0 and x.data_ptr() % 16 == 0 and x.numel() < 2**31


def pertoken_quant_kernel(x: torch.Tensor, quant_dtype=torch.int8):
    """The quantiser as ONE CUDA kernel (row maximum, scale and conversion
    fused; the torch statement below launches about ten element-wise kernels
    and materialises fp32 temporaries).  Bit-identical to :func:`pertoken_quant`
    evaluated by torch on the same GPU tensor."""
    lib = _lib.load()
    k = x.shape[-1]
    rows = x.numel() // k
    y = torch.empty(x.shape, dtype=quant_dtype, device=x.device)
    s = torch.empty(*x.shape[:-1], 1, dtype=torch.float32, device=x.device)
    qd = _lib.DT_INT8 if quant_dtype == torch.int8 else _lib.DT_FP8
    with torch.cuda.device(x.device):
        rc = lib.flyb200_pertoken_quant(
            y.data_ptr(), s.data_ptr(), x.data_ptr(), rows, k, _X_DTYPES[x.dtype], qd, _stream_ptr(x.device)
        )
    _lib.check(rc, "pertoken_quant")
    return y, s


def pertoken_quant(
    x, scale=None, x_scale=None, scale_dtype=torch.float32, quant_dtype=torch.int8, dtypeMax=None, use_kernel=None
):
    """Symmetric per-row quantisation: returns ``(y, y_scale)`` with
    ``y = (x / s).to(quant_dtype)`` and ``s = rowmax(|x|) / dtypeMax`` (shape
    [..., 1]); all-zero rows get scale 1; NaN -> 0 and +-Inf -> +-dtypeMax before
    the reduction; ``x_scale`` is an optional smoothing factor multiplied in
    first; ``scale`` supplies the scales instead of computing them.  The cast is
    torch's (int8 truncates toward zero, float8 rounds to nearest even).

    CUDA tensors in the common form (no explicit scale, smoothing factor or
    dtypeMax) go through the fused kernel (:func:`pertoken_quant_kernel`);
    ``use_kernel=False`` forces the torch statement, ``use_kernel=True`` raises
    if the kernel cannot take the arguments."""
    can = _kernel_can_quantise(x, scale, x_scale, scale_dtype, quant_dtype, dtypeMax)
    if use_kernel and not can:
        raise ValueError("the fused quantiser needs a contiguous CUDA fp32/fp16/bf16 tensor and default options")
    if can and use_kernel is not False:
        return pertoken_quant_kernel(x, quant_dtype)
    h = x.to(torch.float32)
    if x_scale is not None:
        h = h * x_scale
    qmax = float(get_dtype_max(quant_dtype) if dtypeMax is None else dtypeMax)
    h = torch.nan_to_num(h, nan=0.0, posinf=qmax, neginf=-qmax)
    if scale is None:
        amax = torch.maximum(h.amax(dim=-1, keepdim=True), h.amin(dim=-1, keepdim=True).neg())
        s = amax / qmax
        s.masked_fill_(s == 0, 1.0)
    else:
        s = scale
    s = torch.nan_to_num(s, nan=1.0, posinf=1.0, neginf=1.0)
    return (h / s).to(quant_dtype), s.to(scale_dtype)


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _permute_on_host(x2: torch.Tensor, inverse: bool) -> torch.Tensor:
    """The same byte permutation for a tensor that lives in host memory (e.g. a
    checkpoint being prepared before upload): chunk (n, blk, c) of 16 bytes goes
    to image position ((blk*N + n)*8 + (c ^ (n & 7)))."""
    n, kb = x2.shape
    v = x2.view(n, kb // 128, 8, 16)
    c = torch.arange(8).view(1, 8) ^ (torch.arange(n).view(n, 1) & 7)  # [n, 8]: image chunk of source chunk
    idx = c.view(n, 1, 8, 1).expand(n, kb // 128, 8, 16)
    if inverse:
        img = x2.view(kb // 128, n, 8, 16).permute(1, 0, 2, 3)
        return torch.gather(img, 2, idx).reshape(n, kb)
    out = torch.empty_like(v)
    out.scatter_(2, idx, v)
    return out.permute(1, 0, 2, 3).reshape(n, kb)


def _as_bytes_3d(x: torch.Tensor):
    if x.dim() < 2:
        raise ValueError("shuffle_weight expects a tensor of at least two dimensions [..., N, K]")
    n, k = x.shape[-2], x.shape[-1]
    e = x.element_size()
    xb = x.contiguous().view(torch.uint8).view(-1, n, k * e)
    return xb, n, k, e


def shuffle_weight(x: torch.Tensor, layout=(16, 16), use_int4=False, src_layout: str = "row_major") -> torch.Tensor:
    """Preshuffle weights ``[..., N, K]`` for the B200 GEMM; same shape and dtype
    out, ``.is_shuffled = True`` set on the result (as the reference does).

    ``layout`` is accepted for call compatibility; only the reference default
    (16, 16) is meaningful and the B200 image does not depend on it.
    ``use_int4`` (packed int4 weights) is not supported.  ``src_layout="mfma"``
    converts weights that were already permuted by the reference helper.
    Requires N % 16 == 0 and K * element_size % 128 == 0 (ValueError otherwise).
    """
    if use_int4:
        raise NotImplementedError("int4 weights are outside the A8W8 path")
    if tuple(layout) != (16, 16):
        raise ValueError(f"only layout=(16, 16) is supported, got {layout!r}")
    if src_layout not in ("row_major", "mfma"):
        raise ValueError(f"src_layout must be 'row_major' or 'mfma', got {src_layout!r}")
    xb, n, k, e = _as_bytes_3d(x)
    if n % 16 != 0 or (k * e) % 128 != 0 or e not in (1, 2):
        raise ValueError(
            f"cannot preshuffle [N={n}, K={k}] of {e}-byte elements: need N % 16 == 0 and K*elem_bytes % 128 == 0"
        )
    if x.is_cuda:
        lib = _lib.load()
        out = torch.empty_like(xb)
        src = _lib.SRC_ROW_MAJOR if src_layout == "row_major" else _lib.SRC_MFMA_16x16
        with torch.cuda.device(x.device):
            stream = _stream_ptr(x.device)
            for i in range(xb.shape[0]):
                _lib.check(
                    lib.flyb200_shuffle_weight(out[i].data_ptr(), xb[i].data_ptr(), n, k, e, src, stream),
                    "shuffle_weight",
                )
    else:
        if src_layout == "mfma":
            v = xb.view(-1, n // 16, (k * e) // 16, 16, 16).permute(0, 1, 3, 2, 4).reshape(-1, n, k * e)
        else:
            v = xb
        out = torch.stack([_permute_on_host(v[i], inverse=False) for i in range(v.shape[0])])
    out = out.view(x.dtype).view(*x.shape)
    out.is_shuffled = True
    return out


def unshuffle_weight(x: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`shuffle_weight`: the row-major ``[..., N, K]`` weights."""
    xb, n, k, e = _as_bytes_3d(x)
    if n % 16 != 0 or (k * e) % 128 != 0 or e not in (1, 2):
        raise ValueError(f"[N={n}, K={k}] of {e}-byte elements is not a B200 weight image")
    if x.is_cuda:
        lib = _lib.load()
        out = torch.empty_like(xb)
        with torch.cuda.device(x.device):
            stream = _stream_ptr(x.device)
            for i in range(xb.shape[0]):
                _lib.check(
                    lib.flyb200_unshuffle_weight(out[i].data_ptr(), xb[i].data_ptr(), n, k, e, stream),
                    "unshuffle_weight",
                )
    else:
        out = torch.stack([_permute_on_host(xb[i], inverse=True) for i in range(xb.shape[0])])
    return out.view(x.dtype).view(*x.shape)
