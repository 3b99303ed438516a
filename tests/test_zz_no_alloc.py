"""The allocation-free entry point ``flyb200_gemm_a8w8_static_scratch``.

Some users of this library cannot give it a workspace: their code runs where
device memory can no longer be allocated (a host application owns the whole
pool, or an allocation's device-wide stall is not tolerable at that point).
For them the library carries its own fixed scratch array.  This test calls the
entry point through the C ABI twice in a row, with different problems, and
compares each result with what the regular entry point produces; the second
call also shows that nothing left in the array by the first call leaks into
the result.  The file name makes pytest collect it after every other test.
"""

import pytest
import torch

from flydsl_b200 import _lib, shuffle_weight
from oracle import a8w8_oracle as oracle
from tests.helpers import as_i8, device_status

pytestmark = pytest.mark.gpu
RTOL = ATOL = 1e-2  # the tolerance of the other parity tests


def _regular(lib, c, a, w, sa, sb, m, n, k, dt, stream):
    rc = lib.flyb200_gemm_a8w8(c.data_ptr(), a.data_ptr(), w.data_ptr(), sa.data_ptr(), sb.data_ptr(), None,
                               m, n, k, dt, _lib.OUT_BF16, _lib.EPI_NONE, 0, None, 0, stream)  # fmt: skip
    _lib.check(rc, "gemm_a8w8")


def _no_alloc(lib, c, a, w, sa, sb, m, n, k, dt, split, stream):
    return lib.flyb200_gemm_a8w8_static_scratch(c.data_ptr(), a.data_ptr(), w.data_ptr(), sa.data_ptr(), sb.data_ptr(),
                                                None, m, n, k, dt, _lib.OUT_BF16, _lib.EPI_NONE, split, stream)  # fmt: skip


def test_static_scratch_entry_matches_regular_entry_twice_in_a_row():
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    lib = _lib.load()
    assert lib.flyb200_static_scratch_bytes() == 8 << 20
    stream = torch.cuda.current_stream().cuda_stream
    # two different problems back to back: the second meets the leftovers of the first
    problems = [("fp8", 32, 2048, 4096, 4), ("int8", 7, 1040, 2048, 0), ("fp8", 200, 512, 2048, 2)]
    prepared = []
    for in_dtype, m, n, k, split in problems:
        a_q, b_q, sa, sb = oracle.make_inputs(m, n, k, in_dtype, seed=900 + m)
        prepared.append((in_dtype, m, n, k, split, a_q, b_q, sa, sb,
                         as_i8(a_q.to(dev)), as_i8(shuffle_weight(b_q.to(dev))), sa.to(dev), sb.to(dev)))  # fmt: skip
    torch.cuda.synchronize()
    outs = []
    for in_dtype, m, n, k, split, a_q, b_q, sa, sb, a_d, w_d, sa_d, sb_d in prepared:
        c_new = torch.full((m + 4, n), -8192.0, dtype=torch.bfloat16, device=dev)
        rc = _no_alloc(lib, c_new, a_d, w_d, sa_d, sb_d, m, n, k, _lib.IN_DTYPES[in_dtype], split, stream)
        _lib.check(rc, "gemm_a8w8_static_scratch")
        outs.append(c_new)  # no synchronisation between the calls: they run back to back on one stream
    torch.cuda.synchronize()
    assert device_status() == 0
    for (in_dtype, m, n, k, split, a_q, b_q, sa, sb, a_d, w_d, sa_d, sb_d), c_new in zip(prepared, outs):
        c_ref = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        _regular(lib, c_ref, a_d, w_d, sa_d, sb_d, m, n, k, _lib.IN_DTYPES[in_dtype], stream)
        torch.cuda.synchronize()
        got, want = c_new[:m].float().cpu(), c_ref.float().cpu()
        assert oracle.strict_mismatches(got, want, RTOL, ATOL) == 0
        if in_dtype == "int8":
            assert torch.equal(got, want)  # exact integer sums: identical whatever the split
        assert oracle.strict_mismatches(got, oracle.run_torch(a_q, b_q, sa, sb), RTOL, ATOL) == 0
        assert bool((c_new[m:] == -8192.0).all())  # rows past M untouched
    assert device_status() == 0


def _generic(lib, entry, c, a, w, sa, sb, bias, m, n, k, dt, epi, split, stream):
    sa_p, sb_p = (sa.data_ptr(), sb.data_ptr()) if sa is not None else (None, None)
    bias_p = bias.data_ptr() if bias is not None else None
    if entry == "static":
        return lib.flyb200_gemm_a8w8_static_scratch(c.data_ptr(), a.data_ptr(), w.data_ptr(), sa_p, sb_p, bias_p,
                                                    m, n, k, dt, _lib.OUT_BF16, epi, split, stream)  # fmt: skip
    return lib.flyb200_gemm_a8w8(c.data_ptr(), a.data_ptr(), w.data_ptr(), sa_p, sb_p, bias_p,
                                 m, n, k, dt, _lib.OUT_BF16, epi, 0, None, 0, stream)  # fmt: skip


def test_static_scratch_entry_allocates_nothing_with_bias_and_16_bit_inputs():
    """A fused-bias FP8 problem and a bf16-input problem through the entry point,
    with the device's free memory and torch's own allocation counter read before
    and after: once the kernels' code is resident (first call), further calls
    must leave both unchanged."""
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator().manual_seed(11)
    cases = []
    m, n, k = 48, 1024, 2048
    a_q, b_q, sa, sb = oracle.make_inputs(m, n, k, "fp8", seed=41)
    bias = torch.randn(n, generator=g).to(torch.bfloat16)
    ref = oracle.epilogue(a_q.float() @ b_q.float().T, sa, sb, bias, "bias_relu", out_dtype=torch.float32)
    cases.append((m, n, k, _lib.DT_FP8, _lib.EPI_BIAS_RELU, 3, as_i8(a_q.to(dev)), as_i8(shuffle_weight(b_q.to(dev))),
                  sa.to(dev), sb.to(dev), bias.to(dev), ref))  # fmt: skip
    m, n, k = 100, 512, 1024
    a16 = torch.randn(m, k, generator=g).to(torch.bfloat16)
    b16 = torch.randn(n, k, generator=g).to(torch.bfloat16)
    cases.append((m, n, k, _lib.DT_BF16, _lib.EPI_NONE, 4, a16.to(dev), shuffle_weight(b16.to(dev)), None, None, None,
                  a16.float() @ b16.float().T))  # fmt: skip
    outs = [torch.empty(c[0], c[1], dtype=torch.bfloat16, device=dev) for c in cases]
    refs = [torch.empty(c[0], c[1], dtype=torch.bfloat16, device=dev) for c in cases]

    def run_all(entry, dst):
        for (m, n, k, dt, epi, split, a_d, w_d, sa_d, sb_d, bias_d, _), c in zip(cases, dst):
            _lib.check(_generic(lib, entry, c, a_d, w_d, sa_d, sb_d, bias_d, m, n, k, dt, epi, split, stream), entry)

    run_all("static", outs)  # first use: kernels become resident, the array's address is looked up
    torch.cuda.synchronize()
    free_before, _total = torch.cuda.mem_get_info(dev)
    torch_before = torch.cuda.memory_allocated(dev)
    for _ in range(3):
        run_all("static", outs)
    torch.cuda.synchronize()
    free_after, _total = torch.cuda.mem_get_info(dev)
    assert torch.cuda.memory_allocated(dev) == torch_before
    assert free_after >= free_before, f"device memory shrank by {free_before - free_after} bytes across the calls"
    run_all("regular", refs)
    torch.cuda.synchronize()
    assert device_status() == 0
    for case, c_new, c_ref in zip(cases, outs, refs):
        got = c_new.float().cpu()
        assert oracle.strict_mismatches(got, c_ref.float().cpu(), RTOL, ATOL) == 0
        assert oracle.strict_mismatches(got, case[-1], RTOL, ATOL) == 0


def test_static_scratch_entry_rejects_what_does_not_fit():
    dev = torch.device("cuda:0")
    lib = _lib.load()
    t = torch.zeros(1024, dtype=torch.uint8, device=dev)
    p = t.data_ptr()
    # M = 256, N = 8192, split 8 would need 8 * 64 * 256 * 512 B = 64 MiB of partial sums
    rc = lib.flyb200_gemm_a8w8_static_scratch(p, p, p, p, p, None, 256, 8192, 8192, _lib.DT_FP8, 0, 0, 8, None)
    assert rc == _lib.E_SCRATCH_LIMIT
    assert b"8 MiB" in lib.flyb200_strerror(rc)
    # beyond the small-M kernel, and bad arguments
    assert lib.flyb200_gemm_a8w8_static_scratch(p, p, p, p, p, None, 257, 8192, 8192, _lib.DT_FP8, 0, 0, 2, None) == _lib.E_UNSUPPORTED
    assert lib.flyb200_gemm_a8w8_static_scratch(p, p, p, None, p, None, 16, 1024, 1024, _lib.DT_FP8, 0, 0, 2, None) == _lib.E_BAD_ARG
    assert lib.flyb200_gemm_a8w8_static_scratch(p, p, p, p, p, None, 16, 1024, 1024, _lib.DT_FP8, 0, 0, -1, None) == _lib.E_BAD_ARG
    # a null or misaligned operand, or a bias epilogue without bias, is refused before anything is queued on the stream
    assert lib.flyb200_gemm_a8w8_static_scratch(p, None, p, p, p, None, 16, 1024, 1024, _lib.DT_FP8, 0, 0, 2, None) == _lib.E_BAD_ARG
    assert lib.flyb200_gemm_a8w8_static_scratch(p + 4, p, p, p, p, None, 16, 1024, 1024, _lib.DT_FP8, 0, 0, 2, None) == _lib.E_BAD_ALIGN
    assert lib.flyb200_gemm_a8w8_static_scratch(p, p, p, p, p, None, 16, 1024, 1024, _lib.DT_FP8, 0, _lib.EPI_BIAS, 2, None) == _lib.E_BAD_ARG
    torch.cuda.synchronize()
    assert device_status() == 0
