"""Host-side mirror of the reference operator surface and the C ABI's exported
symbols.  No GPU compute here."""

import ctypes
import os
import re

import pytest
import torch

from flydsl_b200 import _lib, compile_preshuffle_gemm, shuffle_weight
from flydsl_b200 import compiler as flyc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "flyb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(flyb200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = declared_functions()
    assert len(names) >= 10
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/flyb200.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert lib.flyb200_version() >= 1


def test_layout_kind_and_strerror():
    lib = _lib.load()
    assert lib.flyb200_layout_kind(4096, 4096, 1) == 1
    assert lib.flyb200_layout_kind(5120, 8320, 1) == 1  # K = 65 * 128
    assert lib.flyb200_layout_kind(1024, 2048, 2) == 1
    assert lib.flyb200_layout_kind(1000, 4096, 1) == 0  # N % 16
    assert lib.flyb200_layout_kind(1024, 96, 1) == 0  # K % 128
    assert lib.flyb200_layout_kind(1024, 96, 2) == 0
    assert lib.flyb200_layout_kind(1024, 64, 2) == 1
    assert lib.flyb200_layout_kind(1024, 1024, 4) == 0
    assert lib.flyb200_strerror(0) == b"ok"
    for code in range(1, 8):
        assert lib.flyb200_strerror(code) not in (b"ok", b"unknown error")
    assert lib.flyb200_strerror(99) == b"unknown error"


def test_argument_checks_need_no_gpu():
    """Bad arguments are rejected before any CUDA call is made."""
    lib = _lib.load()
    buf = (ctypes.c_char * 64)()
    p = ctypes.addressof(buf)
    p16 = (p + 15) & ~15
    assert lib.flyb200_gemm_a8w8(None, p16, p16, p16, p16, None, 1, 16, 128, 0, 0, 0, 0, None, 0, None) == _lib.E_BAD_ARG
    assert lib.flyb200_gemm_a8w8(p16, p16, p16, None, None, None, 1, 16, 128, 0, 0, 0, 0, None, 0, None) == _lib.E_BAD_ARG
    assert lib.flyb200_gemm_a8w8(p16, p16, p16, p16, p16, None, 1, 16, 128, 9, 0, 0, 0, None, 0, None) == _lib.E_BAD_ARG
    assert lib.flyb200_gemm_a8w8(p16, p16, p16, p16, p16, None, 1, 16, 128, 0, 7, 0, 0, None, 0, None) == _lib.E_BAD_ARG
    assert lib.flyb200_gemm_a8w8(p16, p16, p16, p16, p16, None, 1, 16, 128, 0, 0, 2, 0, None, 0, None) == _lib.E_BAD_ARG
    assert lib.flyb200_gemm_a8w8(p16, p16, p16, p16, p16, None, 1, 24, 128, 0, 0, 0, 0, None, 0, None) == _lib.E_UNSUPPORTED
    assert lib.flyb200_gemm_a8w8(p16, p16, p16, p16, p16, None, 1, 16, 100, 0, 0, 0, 0, None, 0, None) == _lib.E_UNSUPPORTED
    assert lib.flyb200_gemm_a8w8(p16 + 4, p16, p16, p16, p16, None, 1, 16, 128, 0, 0, 0, 0, None, 0, None) == _lib.E_BAD_ALIGN
    assert lib.flyb200_shuffle_weight(p16, p16, 16, 128, 1, 0, None) == _lib.E_BAD_ARG  # overlap
    assert lib.flyb200_shuffle_weight(p16, p16 + 4096, 16, 128, 1, 5, None) == _lib.E_BAD_ARG
    assert lib.flyb200_shuffle_weight(p16, p16 + 4096, 20, 128, 1, 0, None) == _lib.E_UNSUPPORTED
    assert lib.flyb200_gemm_a8w8_acc(p16, p16, p16, 1, 16, 128, _lib.DT_BF16, 0, None, 0, None) == _lib.E_UNSUPPORTED
    assert lib.flyb200_workspace_bytes(32, 24, 128, 0, 0) == 0  # unsupported shape: nothing to size
    with pytest.raises(_lib.FlyB200Error, match="16-byte"):
        _lib.check(_lib.E_BAD_ALIGN)


# --- builder validation: the cases the reference pins
#     (tests/kernels/test_preshuffle_gemm.py:983-1039, kernels/gemm/preshuffle_gemm.py:129-136)


@pytest.mark.parametrize("tile_m", [48, 80, 112, 144])
def test_rejects_partial_a_tile(tile_m):
    with pytest.raises(ValueError, match=r"must be a multiple of"):
        compile_preshuffle_gemm(N=1024, K=2048, tile_m=tile_m, tile_n=256, tile_k=64, in_dtype="bf16", out_dtype="bf16")


@pytest.mark.parametrize("tile_m", [64, 96, 128, 160])
def test_accepts_whole_a_tile(tile_m):
    fn = compile_preshuffle_gemm(N=1024, K=2048, tile_m=tile_m, tile_n=256, tile_k=64, in_dtype="bf16", out_dtype="bf16")
    assert callable(fn)


@pytest.mark.parametrize("bad", [(1,), (1, 2, 3), (-1, 0), (0, -1), 4])
def test_preload_validation(bad):
    with pytest.raises((ValueError, TypeError)):
        compile_preshuffle_gemm(
            N=1024, K=2048, tile_m=128, tile_n=256, tile_k=64, in_dtype="bf16", out_dtype="bf16", preload=bad
        )


def test_builder_value_errors():
    ok = dict(N=1024, K=2048, tile_m=128, tile_n=128, tile_k=128)
    compile_preshuffle_gemm(**ok)
    compile_preshuffle_gemm(**ok, in_dtype="int8", preload=(2, 2), waves_per_eu=2, xcd_swizzle=4, use_async_copy=True)
    with pytest.raises(ValueError, match="in_dtype"):
        compile_preshuffle_gemm(**ok, in_dtype="fp4")
    with pytest.raises(ValueError, match="tile_k"):
        compile_preshuffle_gemm(**{**ok, "tile_k": 96})
    with pytest.raises(ValueError, match="tile_k"):
        compile_preshuffle_gemm(**{**ok, "tile_k": 0})
    with pytest.raises(ValueError, match="epilogue"):
        compile_preshuffle_gemm(**ok, epilogue="bias_tanh")
    with pytest.raises(ValueError, match="lds_stage"):
        compile_preshuffle_gemm(**ok, lds_stage=3)
    with pytest.raises(ValueError, match="out_dtype"):
        compile_preshuffle_gemm(**ok, out_dtype="fp32")
    with pytest.raises(ValueError, match="N % 16"):
        compile_preshuffle_gemm(**{**ok, "N": 1000})
    with pytest.raises(ValueError, match="K\\*elem_bytes"):
        compile_preshuffle_gemm(N=1024, K=2080, tile_m=128, tile_n=128, tile_k=32)
    with pytest.raises(TypeError):
        compile_preshuffle_gemm(1024, 2048, 128, 128, 128)  # keyword-only, as in the reference


def test_launcher_rejects_inconsistent_calls_without_touching_the_gpu():
    fn = compile_preshuffle_gemm(N=64, K=256, tile_m=16, tile_n=64, tile_k=256, in_dtype="int8")
    c = torch.empty(16 * 64, dtype=torch.bfloat16)
    a = torch.empty(16 * 256, dtype=torch.int8)
    b = torch.empty(64 * 256, dtype=torch.int8)
    sa, sb = torch.empty(16), torch.empty(64)
    bias = torch.empty(0, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="differs from the N"):
        fn(c, a, b, sa, sb, bias, 16, 128, None)
    with pytest.raises(ValueError, match="CUDA tensor"):
        fn(c, a, b, sa, sb, bias, 16, 64, None)  # CPU tensors: there is no CPU path
    with pytest.raises(ValueError, match="CUDA tensor"):
        flyc.compile(fn, c, a, b, sa, sb, bias, 16, 64, None)


def test_shuffle_weight_argument_errors():
    with pytest.raises(ValueError, match="N % 16"):
        shuffle_weight(torch.zeros(24, 128, dtype=torch.int8))
    with pytest.raises(ValueError, match="N % 16"):
        shuffle_weight(torch.zeros(32, 96, dtype=torch.int8))
    with pytest.raises(ValueError, match="layout"):
        shuffle_weight(torch.zeros(32, 128, dtype=torch.int8), layout=(16, 32))
    with pytest.raises(NotImplementedError):
        shuffle_weight(torch.zeros(32, 128, dtype=torch.int8), use_int4=True)


def test_reference_import_paths():
    from tests.utils import pertoken_quant as pq, shuffle_weight as sw  # noqa: F401
    from flydsl_b200.kernels.gemm.preshuffle_gemm import compile_preshuffle_gemm as cpg  # noqa: F401

    assert callable(flyc.compile)


def test_reference_import_lines_resolve_after_compat_install():
    import flydsl_b200.compat

    names = flydsl_b200.compat.install()
    assert "flydsl.compiler" in names and "kernels.gemm.preshuffle_gemm" in names
    import flydsl.compiler as ref_flyc  # the reference's line (tests/kernels/test_preshuffle_gemm.py:21)
    from kernels.gemm.preshuffle_gemm import compile_preshuffle_gemm as ref_cpg  # (:35)
    from kernels.moe.moe_gemm_2stage import compile_moe_gemm1  # noqa: F401

    assert ref_flyc.compile is flyc.compile and ref_cpg is compile_preshuffle_gemm


def test_variant_selection_is_a_pure_host_function():
    """The M-bucket dispatch (the counterpart of the reference's per-tile tuning
    table) can be inspected without a GPU."""
    d = _lib.describe_plan
    # decode shapes at N = K = 8192 on 148 SMs: 64 channel tiles x split-K 2 as clusters
    p = d(32, 8192, 8192, "int8", variant_hint=1 << 8)
    assert (p["kernel"], p["bn"], p["split_k"], p["reduce"], p["token_blocks"]) == (1, 32, 2, 2, 1)
    assert p["split_k"] * p["kb_per_split"] >= 64
    assert d(32, 8192, 8192, "int8")["kernel"] == 1  # also the automatic choice
    # ... or, on request, 128 tiles of 64 channels with no split at all
    p = d(32, 8192, 8192, "int8", variant_hint=4 << 8)
    assert (p["kernel"], p["bn"], p["split_k"], p["reduce"]) == (4, 32, 1, 0)
    with pytest.raises(_lib.FlyB200Error):
        d(128, 8192, 8192, variant_hint=4 << 8)  # too many tokens for the half-height tiles
    assert d(1, 8192, 8192)["bn"] == 16 and d(17, 8192, 8192)["bn"] == 32 and d(256, 8192, 8192)["bn"] == 256
    # more channel tiles than SMs: no split
    assert d(8, 57344, 8192)["split_k"] == 1 and d(8, 57344, 8192)["reduce"] == 0
    # benchmark config 1: 32 tiles -> split 4
    assert d(128, 4096, 4096)["split_k"] == 4
    # large M: persistent kernel, one CTA per tile unless asked otherwise
    assert d(257, 8192, 8192)["kernel"] == 2 and d(8192, 28672, 8192, variant_hint=3 << 8)["kernel"] == 3
    # explicit requests are honoured or refused, never changed silently
    assert d(32, 8192, 8192, variant_hint=(1 << 8) | (1 << 12) | 16)["reduce"] == 1
    with pytest.raises(_lib.FlyB200Error):
        d(32, 8192, 8192, variant_hint=(1 << 8) | (2 << 12) | 16)  # a cluster cannot hold 16 splits
    assert d(300, 8192, 8192, variant_hint=1 << 8)["token_blocks"] == 2  # beyond 256 tokens: blocks of 256
    # a single k-block cannot be split
    assert d(16, 1024, 128)["split_k"] == 1
    # fewer SMs -> smaller split
    assert d(32, 8192, 8192, sm_count=64, variant_hint=1 << 8)["split_k"] == 1
    # the automatic split keeps the launch within one round of CTAs also where K is long
    p = d(64, 8192, 28672)
    assert (p["kernel"], p["split_k"], p["reduce"]) == (1, 2, 2)
    # wide outputs (more channel tiles than SMs) go to the persistent kernel above 64 tokens, badly
    # filled rounds from 32, very wide ones from 16; narrow ones stay on the small-M kernel
    assert d(64, 28672, 8192)["kernel"] == 1 and d(65, 28672, 8192)["kernel"] == 2 and d(256, 28672, 8192)["kernel"] == 2
    assert d(64, 18944, 4096)["kernel"] == 1 and d(200, 18944, 4096)["kernel"] == 1  # exactly one round of CTAs
    assert d(16, 24576, 8192)["kernel"] == 1 and d(32, 24576, 8192)["kernel"] == 2  # second round 30 % full
    assert d(8, 57344, 8192)["kernel"] == 1 and d(16, 57344, 8192)["kernel"] == 2
    assert d(256, 16384, 8192)["kernel"] == 1
    assert d(128, 28672, 8192, variant_hint=1 << 8)["kernel"] == 1  # a request for the small-M kernel stands
    # 256-row tiles: on request, and by themselves where they cover the output in one nearly full round
    assert d(4096, 8192, 8192, variant_hint=6 << 8)["kernel"] == 6 and d(4096, 8192, 8192)["kernel"] == 2
    p = d(1024, 8192, 8192)
    assert (p["kernel"], p["bn"], p["stages"]) == (6, 256, 3)
    assert d(1024, 4096, 8192)["kernel"] == 2 and d(2048, 8192, 8192)["kernel"] == 2
    assert d(300, 16384, 8192)["kernel"] == 2  # 2 x 64 tiles would fit, but rows 384..511 would be padding
    assert d(128, 37888, 8192)["kernel"] == 2  # wide output routed to the large-M kernel: 128-row tiles
    # 257..1024 tokens on a narrow output with a long K: token blocks of 256 on the small-M kernel
    p = d(512, 2048, 8192)
    assert (p["kernel"], p["bn"], p["token_blocks"], p["split_k"], p["reduce"]) == (1, 256, 2, 4, 2)
    assert d(1024, 2048, 8192)["token_blocks"] == 4 and d(1025, 2048, 8192)["kernel"] == 2
    assert d(512, 8192, 8192)["kernel"] == 2 and d(512, 4096, 2048)["kernel"] == 2  # too many tiles; K too short
    with pytest.raises(_lib.FlyB200Error):
        d(1025, 2048, 8192, variant_hint=1 << 8)  # four token blocks of 256 are the limit
    # small-M kernel as CTA pairs: on request, for token tiles of 64 and more and an even number of channel tiles
    p = d(256, 8192, 8192, variant_hint=5 << 8)
    assert (p["kernel"], p["bn"], p["split_k"], p["reduce"], p["stages"]) == (5, 256, 2, 2, 6)
    assert d(64, 8192, 8192, variant_hint=5 << 8)["stages"] == 8
    for m, n in ((32, 8192), (64, 1040)):  # too few tokens; nine channel tiles
        with pytest.raises(_lib.FlyB200Error):
            d(m, n, 8192, variant_hint=5 << 8)
    with pytest.raises(_lib.FlyB200Error):
        d(64, 8192, 8192, variant_hint=(5 << 8) | (1 << 12) | 2)  # pairs reduce inside their cluster only
