"""ctypes binding of libflyb200.so (the C ABI in include/flyb200.h).

There is no fallback: if the library cannot be loaded every operator of this
package raises.
"""

from __future__ import annotations

import ctypes
import threading

from . import build as _build

OK = 0
E_BAD_ARG, E_BAD_ALIGN, E_CUDA, E_TIMEOUT, E_UNSUPPORTED, E_SMEM_ALIGN, E_WORKSPACE, E_SCRATCH_LIMIT = range(1, 9)

DT_FP8, DT_INT8, DT_FP16, DT_BF16 = range(4)
OUT_BF16, OUT_FP16, OUT_F32 = range(3)
EPI_NONE, EPI_BIAS, EPI_BIAS_RELU, EPI_BIAS_SILU, EPI_BIAS_GELU = range(5)
SRC_ROW_MAJOR, SRC_MFMA_16x16 = range(2)

IN_DTYPES = {"fp8": DT_FP8, "int8": DT_INT8, "fp16": DT_FP16, "bf16": DT_BF16}
OUT_DTYPES = {"bf16": OUT_BF16, "fp16": OUT_FP16}
EPILOGUES = {
    "none": EPI_NONE,
    "bias": EPI_BIAS,
    "bias_relu": EPI_BIAS_RELU,
    "bias_silu": EPI_BIAS_SILU,
    "bias_gelu": EPI_BIAS_GELU,
}

_vp, _i, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t

# name -> (restype, argtypes): one row per declaration in include/flyb200.h
SIGNATURES = {
    "flyb200_gemm_a8w8": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _sz, _vp]),
    "flyb200_gemm_a8w8_acc": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _sz, _vp]),
    "flyb200_gemm_a8w8_static_scratch": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "flyb200_static_scratch_bytes": (_sz, []),
    "flyb200_gemm_a8w8_scatter": (
        _i,
        [ctypes.POINTER(_vp), _i, _i, ctypes.c_longlong, ctypes.c_longlong, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp],
    ),
    "flyb200_pertoken_quant": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "flyb200_shuffle_weight": (_i, [_vp, _vp, _i, _i, _i, _i, _vp]),
    "flyb200_unshuffle_weight": (_i, [_vp, _vp, _i, _i, _i, _vp]),
    "flyb200_describe_plan": (_i, [_i, _i, _i, _i, _i, _i, ctypes.POINTER(_i)]),
    "flyb200_layout_kind": (_i, [_i, _i, _i]),
    "flyb200_workspace_bytes": (_sz, [_i, _i, _i, _i, _i]),
    "flyb200_read_status": (_i, [ctypes.POINTER(_i)]),
    "flyb200_selftest_bounded_wait": (_i, [ctypes.c_uint, _vp]),
    "flyb200_moe_gather_rows": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "flyb200_moe_gemm": (_i, [_i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp] + [_i] * 12 + [_vp]),
    "flyb200_moe_reduce": (_i, [_vp, _vp, _i, _i, _i, _i, _vp, _vp, _i, _vp]),
    "flyb200_moe_sorting": (_i, [_vp, _vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "flyb200_gemm_mxfp8": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "flyb200_gemm_mx_mixed": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "flyb200_gemm_mxfp4": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "flyb200_mx_scale_image": (_i, [_vp, _vp, _i, _i, _vp]),
    "flyb200_mx_scale_image_bytes": (_sz, [_i, _i]),
    "flyb200_strerror": (ctypes.c_char_p, [_i]),
    "flyb200_last_cuda_error": (ctypes.c_char_p, []),
    "flyb200_version": (_i, []),
}

_lock = threading.Lock()
_lib = None


class FlyB200Error(RuntimeError):
    def __init__(self, code: int, what: str):
        self.code = code
        super().__init__(what)


def load() -> ctypes.CDLL:
    """Load (building first if the in-tree library is missing or stale)."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            path = _build.build_library()
            lib = ctypes.CDLL(path)
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(lib, name)  # AttributeError if the symbol is not exported
                fn.restype = res
                fn.argtypes = args
            _lib = lib
    return _lib


def check(code: int, what: str = "libflyb200") -> None:
    if code == OK:
        return
    lib = load()
    msg = lib.flyb200_strerror(code).decode()
    if code == E_CUDA:
        msg += ": " + lib.flyb200_last_cuda_error().decode()
    raise FlyB200Error(code, f"{what}: {msg} (code {code})")


PLAN_FIELDS = ("kernel", "bn", "split_k", "kb_per_split", "reduce", "stages", "pdl", "token_blocks")


def describe_plan(m: int, n: int, k: int, in_dtype: str = "fp8", variant_hint: int = 0, sm_count: int = 148) -> dict:
    """The kernel variant the library would pick (no GPU needed)."""
    out = (_i * 8)()
    check(load().flyb200_describe_plan(m, n, k, IN_DTYPES[in_dtype], variant_hint, sm_count, out), "describe_plan")
    return dict(zip(PLAN_FIELDS, list(out)))


_failure_hooks: list = []


def on_failure_status(fn) -> None:
    """Register a callback run whenever :func:`read_status` finds a failure recorded by a kernel."""
    _failure_hooks.append(fn)


def read_status() -> int:
    """Synchronise the current device and return (and clear) its status word.
    A non-zero status means a kernel gave up on a bounded wait; state that such
    a kernel may have left half-updated (split-K arrival counters) is reset."""
    out = _i(0)
    check(load().flyb200_read_status(ctypes.byref(out)), "read_status")
    if out.value != 0:
        for fn in _failure_hooks:
            fn()
    return out.value
