"""Shared pieces of the GPU parity tests."""

import ctypes

import torch

from flydsl_b200 import _lib
from oracle import a8w8_oracle as oracle


def as_i8(t):
    return t.view(torch.int8) if "float8" in str(t.dtype) else t


def quantised_inputs(m, n, k, in_dtype, seed, weight_scale=1.0, rne_int8=False):
    """CPU-generated, seeded quantised operands (so that the oracle and the GPU
    see the same bytes) plus their CUDA copies."""
    a_q, b_q, sa, sb = oracle.make_inputs(m, n, k, in_dtype, seed, weight_scale, rne_int8)
    return a_q, b_q, sa, sb


def gpu_acc(a_q, b_shuf, m, n, k, in_dtype, variant_hint=0, workspace=None):
    """Raw 32-bit accumulators through the C ABI."""
    lib = _lib.load()
    out = torch.empty(m, n, dtype=torch.int32, device=a_q.device)
    ws_ptr, ws_len = (workspace.data_ptr(), workspace.numel()) if workspace is not None else (None, 0)
    rc = lib.flyb200_gemm_a8w8_acc(
        out.data_ptr(), as_i8(a_q).data_ptr(), as_i8(b_shuf).data_ptr(), m, n, k,
        _lib.IN_DTYPES[in_dtype], variant_hint, ws_ptr, ws_len, torch.cuda.current_stream().cuda_stream,
    )  # fmt: skip
    _lib.check(rc, "gemm_a8w8_acc")
    return out


def make_workspace(m, n, k, in_dtype, device, variant_hint=0):
    lib = _lib.load()
    nbytes = int(lib.flyb200_workspace_bytes(m, n, k, _lib.IN_DTYPES[in_dtype], variant_hint))
    return torch.zeros(max(nbytes, 16), dtype=torch.uint8, device=device)


def device_status():
    return _lib.read_status()
