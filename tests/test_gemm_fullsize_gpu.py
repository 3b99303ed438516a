"""Benchmark-sized configurations on the GPU.  The oracle is evaluated on a
sample of rows (all columns), which it finishes in seconds; size-independent
properties cover the rest."""

import pytest
import torch

from flydsl_b200 import compile_preshuffle_gemm, pertoken_quant, shuffle_weight
from oracle import a8w8_oracle as oracle
from tests.helpers import as_i8, device_status

pytestmark = pytest.mark.gpu
RTOL = ATOL = 1e-2


def gpu_inputs(m, n, k, dev, seed, weight_scale=1.0):
    g = torch.Generator(device=dev).manual_seed(seed)
    a = torch.randn(m, k, generator=g, device=dev)
    w = torch.randn(n, k, generator=g, device=dev) * weight_scale
    a_q, sa = pertoken_quant(a, quant_dtype=torch.float8_e4m3fn)
    b_q, sb = pertoken_quant(w, quant_dtype=torch.float8_e4m3fn)
    return a_q, b_q, sa.view(-1), sb.view(-1)


@pytest.mark.parametrize(
    "m,n,k,wscale",
    [
        (8192, 28672, 8192, 0.02),  # benchmark config 3 (prefill, MLP up-projection)
        (5133, 5120, 8320, 1.0),  # the reference's ragged large shape
        (5120, 2048, 8320, 1.0),  # reference large shape, narrow N
        (9728, 8192, 8320, 1.0),  # reference large shape (its int8 benchmark shape, here fp8)
        (16384, 8192, 8192, 1.0),  # top of the M sweep
        (4096, 8192, 8192, 1.0),  # M sweep
        (16384, 57344, 8192, 1.0),  # benchmark config 5 on one GPU (the multi-GPU workload, unsplit)
    ],
)
def test_large_fp8_sampled_rows_and_properties(m, n, k, wscale):
    dev = torch.device("cuda:0")
    a_q, b_q, sa, sb = gpu_inputs(m, n, k, dev, seed=1003, weight_scale=wscale)
    fn = compile_preshuffle_gemm(N=n, K=k, tile_m=128, tile_n=256, tile_k=128, in_dtype="fp8")
    b_shuf = shuffle_weight(b_q)
    rows = ((m + 127) // 128) * 128
    c = torch.full((rows, n), -8192.0, dtype=torch.bfloat16, device=dev)
    bias = torch.empty(0, dtype=torch.bfloat16, device=dev)
    fn(c.view(-1), as_i8(a_q).view(-1), as_i8(b_shuf).view(-1), sa, sb, bias, m, n, torch.cuda.current_stream())
    torch.cuda.synchronize()
    assert device_status() == 0
    assert int((c[m:] != -8192.0).sum().item()) == 0
    # oracle on sampled rows: first/last rows of tiles, the ragged edge, random rows
    gen = torch.Generator().manual_seed(0)
    pick = torch.cat([torch.tensor([0, 1, 127, 128, m - 129, m - 2, m - 1]), torch.randint(0, m, (57,), generator=gen)])
    pick = pick.clamp_(0, m - 1).unique()
    ref = oracle.run_torch(a_q[pick.to(dev)].cpu(), b_q.cpu(), sa[pick.to(dev)].cpu(), sb.cpu())
    got = c[pick.to(dev)].float().cpu()
    bad = oracle.strict_mismatches(got, ref, RTOL, ATOL)
    assert bad == 0, f"{bad} mismatches; max abs diff {(got - ref).abs().max()}"
    # property: every output row depends only on its own token -> recomputing a
    # slice of tokens alone (through the small-M kernel) gives the same values
    # up to accumulation order
    sl = slice(256, 256 + 64)
    c2 = torch.empty(64, n, dtype=torch.bfloat16, device=dev)
    fn(c2.view(-1), as_i8(a_q[sl]).contiguous().view(-1), as_i8(b_shuf).view(-1), sa[sl].contiguous(), sb, bias, 64, n, None)
    torch.cuda.synchronize()
    assert oracle.strict_mismatches(c2.float().cpu(), c[sl].float().cpu(), RTOL, ATOL) == 0
    # property: a second launch is bitwise identical
    c3 = torch.empty(rows, n, dtype=torch.bfloat16, device=dev)
    fn(c3.view(-1), as_i8(a_q).view(-1), as_i8(b_shuf).view(-1), sa, sb, bias, m, n, torch.cuda.current_stream())
    torch.cuda.synchronize()
    assert torch.equal(c3[:m], c[:m])


@pytest.mark.parametrize("m", [1, 16, 64, 256, 1024])
def test_m_sweep_fp8_every_row_against_the_oracle(m):
    """Benchmark config 4 (N = K = 8192) below the sampled sizes: every output element
    against the fp32 dequantise-and-matmul reference, inputs quantised per token /
    per channel from seeded N(0,1) as the configuration states."""
    dev = torch.device("cuda:0")
    n = k = 8192
    a_q, b_q, sa, sb = gpu_inputs(m, n, k, dev, seed=1040 + m)
    fn = compile_preshuffle_gemm(N=n, K=k, tile_m=128, tile_n=256, tile_k=128, in_dtype="fp8")
    rows = ((m + 127) // 128) * 128
    c = torch.full((rows, n), -8192.0, dtype=torch.bfloat16, device=dev)
    bias = torch.empty(0, dtype=torch.bfloat16, device=dev)
    fn(c.view(-1), as_i8(a_q).view(-1), as_i8(shuffle_weight(b_q)).view(-1), sa, sb, bias, m, n, torch.cuda.current_stream())
    torch.cuda.synchronize()
    assert device_status() == 0
    assert int((c[m:] != -8192.0).sum().item()) == 0
    ref = oracle.run_torch(a_q.cpu(), b_q.cpu(), sa.cpu(), sb.cpu())
    got = c[:m].float().cpu()
    bad = oracle.strict_mismatches(got, ref, RTOL, ATOL)
    assert bad == 0, f"M={m}: {bad} mismatches; max abs diff {(got - ref).abs().max()}"


def test_int8_decode_config_scaled_bf16_output():
    """Benchmark config 2 (INT8 32 x 8192 x 8192, round-to-nearest quantisation) through the
    scaled bf16 path, next to the accumulator check of the parity file."""
    dev = torch.device("cuda:0")
    m, n, k = 32, 8192, 8192
    a_q, b_q, sa, sb = oracle.make_inputs(m, n, k, "int8", seed=1002, rne_int8=True)
    fn = compile_preshuffle_gemm(N=n, K=k, tile_m=32, tile_n=128, tile_k=128, in_dtype="int8")
    c = torch.full((m + 8, n), -8192.0, dtype=torch.bfloat16, device=dev)
    bias = torch.empty(0, dtype=torch.bfloat16, device=dev)
    fn(c.view(-1), a_q.to(dev).view(-1), shuffle_weight(b_q.to(dev)).view(-1), sa.to(dev).view(-1), sb.to(dev).view(-1), bias, m, n,
       torch.cuda.current_stream())
    torch.cuda.synchronize()
    assert device_status() == 0
    assert int((c[m:] != -8192.0).sum().item()) == 0
    # exact int32 sums scaled in fp32 and rounded once: the kernel's arithmetic, so the bf16 results are equal
    want = oracle.epilogue(oracle.int32_acc(a_q, b_q), sa, sb, None, "none", out_dtype=torch.bfloat16)
    assert torch.equal(c[:m].cpu(), want)
    assert oracle.strict_mismatches(c[:m].float().cpu(), oracle.run_torch(a_q, b_q, sa, sb), RTOL, ATOL) == 0


def test_int8_large_accumulators_exact_on_sample():
    dev = torch.device("cuda:0")
    from flydsl_b200 import _lib
    from tests.helpers import gpu_acc

    m, n, k = 9728, 8192, 8320  # the reference's int8 benchmark shape
    g = torch.Generator(device=dev).manual_seed(7)
    a_q = torch.randint(-127, 128, (m, k), generator=g, device=dev, dtype=torch.int8)
    b_q = torch.randint(-127, 128, (n, k), generator=g, device=dev, dtype=torch.int8)
    acc = gpu_acc(a_q, shuffle_weight(b_q), m, n, k, "int8")
    torch.cuda.synchronize()
    assert device_status() == 0
    pick = torch.tensor([0, 127, 128, 4095, 9727, 5000, 6001, 7002])
    want = oracle.int32_acc(a_q[pick.to(dev)].cpu(), b_q.cpu())
    assert torch.equal(acc[pick.to(dev)].cpu(), want)
    # checksum of checksums: column sums of the exact product equal (sum of A rows) . B^T
    col_sum = acc.to(torch.int64).sum(dim=0).cpu()
    want_sum = (a_q.to(torch.float64).sum(dim=0, keepdim=True).cpu() @ b_q.to(torch.float64).cpu().T).to(torch.int64).view(-1)
    assert torch.equal(col_sum, want_sum)


def test_cta_pair_kernel_matches_single_cta_kernel_at_full_size():
    """Both large-M kernels accumulate each output in the same k order, so their bf16 outputs are bitwise equal."""
    dev = torch.device("cuda:0")
    m, n, k = 4096, 8192, 8192
    a_q, b_q, sa, sb = gpu_inputs(m, n, k, dev, seed=77)
    b_shuf = shuffle_weight(b_q)
    bias = torch.empty(0, dtype=torch.bfloat16, device=dev)
    outs = []
    for hint in (2 << 8, 3 << 8):
        fn = compile_preshuffle_gemm(N=n, K=k, tile_m=128, tile_n=256, tile_k=128, in_dtype="fp8", variant_hint=hint)
        c = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        fn(c.view(-1), as_i8(a_q).view(-1), as_i8(b_shuf).view(-1), sa, sb, bias, m, n, torch.cuda.current_stream())
        outs.append(c)
    torch.cuda.synchronize()
    assert device_status() == 0
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize(
    "m,n,k",
    [
        (65536, 1024, 1024),  # the largest M the reference's launcher can address (its views use M_max = 65536)
        (40, 16, 128),  # the smallest weight image: 16 channels, one k-block
        (300, 16, 128),  # the same through the large-M kernel
        (7, 256, 65536),  # a very long K: 512 k-blocks per channel tile
        (1000, 57344, 256),  # many channel tiles, short K (int32 tile counters, ragged last row tile)
    ],
)
@pytest.mark.parametrize("in_dtype", ["fp8", "int8"])
def test_extreme_shapes(m, n, k, in_dtype):
    dev = torch.device("cuda:0")
    a_q, b_q, sa, sb = oracle.make_inputs(m, n, k, in_dtype, seed=m + n + k)
    fn = compile_preshuffle_gemm(N=n, K=k, tile_m=128, tile_n=256, tile_k=128, in_dtype=in_dtype)
    c = torch.full((m + 8, n), -8192.0, dtype=torch.bfloat16, device=dev)
    bias = torch.empty(0, dtype=torch.bfloat16, device=dev)
    fn(c.view(-1), as_i8(a_q.to(dev)).view(-1), as_i8(shuffle_weight(b_q.to(dev))).view(-1), sa.to(dev).view(-1),
       sb.to(dev).view(-1), bias, m, n, torch.cuda.current_stream())
    torch.cuda.synchronize()
    assert device_status() == 0
    assert int((c[m:] != -8192.0).sum().item()) == 0
    gen = torch.Generator().manual_seed(1)
    pick = torch.cat([torch.tensor([0, m // 2, m - 1]), torch.randint(0, m, (61,), generator=gen)]).unique() if m > 64 else torch.arange(m)
    ref = oracle.run_torch(a_q[pick], b_q, sa[pick], sb)
    got = c[pick.to(dev)].float().cpu()
    # a K of 65536 sums 64 times more terms than the benchmark shapes: the absolute floor scales with the result's size
    atol = max(ATOL, 1e-2 * float(ref.abs().max()) / 16) if k > 8192 else ATOL
    bad = oracle.strict_mismatches(got, ref, RTOL, atol)
    assert bad == 0, f"{bad} mismatches; max abs diff {(got - ref).abs().max()}"
