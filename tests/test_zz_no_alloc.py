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
    torch.cuda.synchronize()
    assert device_status() == 0
