"""The fused per-token quantiser kernel against the torch statement of the
reference helper (tests/utils.py:29-73) on the same GPU tensor (bit-exact) and
against the CPU oracle."""

import pytest
import torch

from flydsl_b200 import pertoken_quant
from flydsl_b200.utils import pertoken_quant_kernel
from oracle import a8w8_oracle as oracle

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn


def special_input(rows, k, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, k, generator=g) * 3.0
    if rows > 9:
        x[3] = 0.0
        x[5, 7] = float("nan")
        x[6, 9] = float("inf")
        x[7, 11] = float("-inf")
        x[8] = x[8].abs()
        x[9] = -x[9].abs()
    return x.to(dtype)


@pytest.mark.parametrize("qd", [FP8, torch.int8], ids=["fp8", "int8"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,k", [(1, 8192), (37, 256), (33, 2056), (4096, 8192)])
def test_kernel_is_bit_identical_to_torch_on_gpu(qd, dtype, rows, k):
    dev = torch.device("cuda:0")
    x = special_input(rows, k, dtype, seed=rows + k).to(dev)
    y_k, s_k = pertoken_quant_kernel(x, qd)
    y_t, s_t = pertoken_quant(x, quant_dtype=qd, use_kernel=False)
    torch.cuda.synchronize()
    assert s_k.shape == s_t.shape == (rows, 1) and s_k.dtype == torch.float32
    assert torch.equal(s_k, s_t)
    assert torch.equal(y_k.view(torch.uint8), y_t.view(torch.uint8))
    # default dispatch takes the kernel
    y_d, s_d = pertoken_quant(x, quant_dtype=qd)
    assert torch.equal(y_d.view(torch.uint8), y_k.view(torch.uint8)) and torch.equal(s_d, s_k)


@pytest.mark.parametrize("qd,qmax", [(FP8, 448.0), (torch.int8, 127.0)], ids=["fp8", "int8"])
def test_kernel_against_cpu_oracle(qd, qmax):
    """The CPU evaluates amax / qmax as a true division, the GPU multiplies by
    the fp32 reciprocal: scales may differ in the last bit, values then by at
    most one quantisation step on a handful of elements."""
    dev = torch.device("cuda:0")
    x = special_input(64, 4096, torch.float32, seed=5)
    y_k, s_k = pertoken_quant_kernel(x.to(dev), qd)
    y_o, s_o = oracle.pertoken_quant(x, quant_dtype=qd)
    s_k, y_k = s_k.cpu(), y_k.cpu()
    assert torch.allclose(s_k, s_o, rtol=2.0**-22, atol=0)
    same = s_k.view(-1) == s_o.view(-1)
    assert torch.equal(y_k[same].view(torch.uint8), y_o[same].view(torch.uint8))  # identical scale -> identical bytes
    deq_k, deq_o = y_k.float() * s_k, y_o.float() * s_o
    step = s_o * (32.0 if qd == FP8 else 1.0)  # one e4m3 step at the top binade / one int8 step
    assert bool(((deq_k - deq_o).abs() <= step * 1.001).all())


def test_quantised_activations_feed_the_gemm():
    """End to end: fused quantiser -> GEMM, against the CPU oracle on the same fp32 inputs."""
    from flydsl_b200 import compile_preshuffle_gemm, shuffle_weight

    dev = torch.device("cuda:0")
    m, n, k = 48, 1024, 2048
    g = torch.Generator().manual_seed(1)
    a, w = torch.randn(m, k, generator=g), torch.randn(n, k, generator=g)
    a_q, sa = pertoken_quant(a.to(dev), quant_dtype=FP8)
    b_q, sb = pertoken_quant(w.to(dev), quant_dtype=FP8)
    c = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    fn = compile_preshuffle_gemm(N=n, K=k, tile_m=16, tile_n=64, tile_k=256, in_dtype="fp8")
    fn(c.view(-1), a_q.view(torch.int8).view(-1), shuffle_weight(b_q).view(torch.int8).view(-1), sa.view(-1), sb.view(-1),
       torch.empty(0, dtype=torch.bfloat16, device=dev), m, n, torch.cuda.current_stream())
    torch.cuda.synchronize()
    ref = oracle.run_torch(a_q.cpu(), b_q.cpu(), sa.cpu(), sb.cpu())
    assert oracle.strict_mismatches(c.float().cpu(), ref, 1e-2, 1e-2) == 0
    exact = a @ w.T  # unquantised product: only the fp8 quantisation error separates the two
    rel = ((c.float().cpu() - exact).norm() / exact.norm()).item()
    assert rel < 0.05, rel


@pytest.mark.parametrize("qd", [FP8, torch.int8], ids=["fp8", "int8"])
def test_kernel_bit_identical_on_adversarial_values(qd):
    """Rows built to sit on the rounding boundaries of the target type (exact
    ties, values one fp32 ulp either side of them, e4m3 subnormals, integers
    and near-integers): the kernel's shortcut around the IEEE division must not
    change a single byte."""
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(99)
    k = 4096
    qmax = 448.0 if qd == FP8 else 127.0
    rows = []
    for scale in (1.0, 0.37, 3.0e-3, 17.25, 1.0 / 3.0):
        if qd == FP8:
            mant = torch.arange(16, 32, dtype=torch.float32)  # neighbouring e4m3 mantissas x2: every second value is a tie
            exps = 2.0 ** torch.arange(-10, 9, dtype=torch.float32)
            base = (mant[None, :] * exps[:, None] / 16.0).reshape(-1)
        else:
            base = torch.arange(0, 128, dtype=torch.float32)
        base = base[base <= qmax]
        cand = torch.cat([base, torch.nextafter(base, torch.tensor(1e9)), torch.nextafter(base, torch.tensor(-1e9)), -base])
        cand = cand[torch.randint(0, cand.numel(), (k - 1,), generator=g)] * scale
        row = torch.cat([torch.tensor([qmax * scale]), cand])  # first element pins amax so that the scale is `scale`-like
        rows.append(row)
    x = torch.stack(rows).to(dev)
    y_k, s_k = pertoken_quant_kernel(x, qd)
    y_t, s_t = pertoken_quant(x, quant_dtype=qd, use_kernel=False)
    torch.cuda.synchronize()
    assert torch.equal(s_k, s_t)
    assert torch.equal(y_k.view(torch.uint8), y_t.view(torch.uint8))
