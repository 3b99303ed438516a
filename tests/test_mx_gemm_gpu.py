"""GPU parity of the MXFP8 x MXFP8 GEMM (tcgen05 block-scaled MMA) against the CPU oracle.

Tolerance: the reference accepts rtol = atol = 0.1 (tests/kernels/test_preshuffle_gemm.py:692);
here every element must be within rtol 1e-2 / atol 1e-2 * max|ref| of the fp32 oracle (the
products are exact, only the fp32 summation order and the 16-bit output rounding differ)."""

import numpy as np
import os
import pytest
import torch

from flydsl_b200 import _lib, shuffle_weight
from flydsl_b200.kernels.gemm.mxfp8_preshuffle import compile_mxfp8_preshuffle_gemm, per_1x32_f8_quant, shuffle_scale
from oracle import mx_oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda:0")


def run(dev, a_q, sa, b_q, sb, out_dtype="bf16", guard=8):
    m, k = a_q.shape
    n = b_q.shape[0]
    c = torch.full((m + guard, n), 7.0, dtype=torch.bfloat16 if out_dtype == "bf16" else torch.float16, device=dev)
    fn = compile_mxfp8_preshuffle_gemm(N=n, K=k, out_dtype=out_dtype)
    fn(c.view(-1), a_q.to(dev).view(torch.uint8).view(-1), shuffle_weight(b_q.to(dev)).view(torch.uint8).view(-1),
       shuffle_scale(sa.to(dev)), shuffle_scale(sb.to(dev)), torch.empty(0, dtype=torch.bfloat16, device=dev), m, n,
       torch.cuda.current_stream())
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    assert torch.all(c[m:] == 7.0), "guard rows were written"
    return c[:m]


def check(c, ref):
    got = c.float().cpu()
    tol = 1e-2 * float(ref.abs().max())
    bad = ((got - ref).abs() > tol + 1e-2 * ref.abs()).sum().item()
    assert bad == 0, f"{bad} elements outside tolerance; max abs err {float((got - ref).abs().max()):.4g}"


def test_scale_image_kernel_matches_layout_statement(dev):
    for rows, k in ((40, 256), (128, 128), (300, 1024), (1, 128)):
        s = torch.randint(0, 255, (rows, k // 32), dtype=torch.uint8)
        assert torch.equal(shuffle_scale(s.to(dev)).cpu(), mx_oracle.scale_image(s))


def test_golden_fixture(dev):
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "mx_fp8.npz"))
    a_q = torch.from_numpy(z["a_q"]).view(torch.float8_e4m3fn)
    b_q = torch.from_numpy(z["b_q"]).view(torch.float8_e4m3fn)
    sa, sb = torch.from_numpy(z["sa"]), torch.from_numpy(z["sb"])
    n_pad = 128  # the fixture has 48 channels: pad the weights to one 128-channel tile with zero codes
    b_pad = torch.zeros(n_pad, b_q.shape[1], dtype=torch.uint8)
    b_pad[: b_q.shape[0]] = b_q.view(torch.uint8)
    sb_pad = torch.full((n_pad, sb.shape[1]), 127, dtype=torch.uint8)
    sb_pad[: sb.shape[0]] = sb
    c = run(dev, a_q, sa, b_pad.view(torch.float8_e4m3fn), sb_pad)
    check(c[:, : b_q.shape[0]], torch.from_numpy(z["c"]))
    assert torch.all(c[:, b_q.shape[0]:] == 0)


@pytest.mark.parametrize("m,n,k", [(128, 128, 128), (16, 256, 512), (300, 384, 1024), (1, 128, 256), (1000, 1024, 2048),
                                   (128, 8192, 8192), (64, 8192, 8192), (32, 8192, 8192), (1024, 8192, 8192),  # the reference's shapes
                                   (17, 1024, 4096), (100, 512, 8192), (129, 256, 1024)])
@pytest.mark.parametrize("out_dtype", ["bf16", "fp16"])
def test_mxfp8_gemm(dev, m, n, k, out_dtype):
    a_q, sa, b_q, sb = mx_oracle.make_inputs(m, n, k, seed=m + n)
    c = run(dev, a_q, sa, b_q, sb, out_dtype)
    check(c, mx_oracle.mx_gemm(a_q, sa, b_q, sb))


def test_scales_matter_per_block(dev):
    """Different scales in every 32-element block and row: a kernel that mixed up rows, blocks or
    the scale-factor ids cannot pass."""
    m, n, k = 128, 128, 512
    g = torch.Generator().manual_seed(5)
    a_q = (torch.randn(m, k, generator=g) * 16).to(torch.float8_e4m3fn)
    b_q = (torch.randn(n, k, generator=g) * 16).to(torch.float8_e4m3fn)
    sa = torch.randint(120, 134, (m, k // 32), generator=g, dtype=torch.uint8)
    sb = torch.randint(120, 134, (n, k // 32), generator=g, dtype=torch.uint8)
    c = run(dev, a_q, sa, b_q, sb)
    check(c, mx_oracle.mx_gemm(a_q, sa, b_q, sb))


def test_device_quantiser_matches_oracle(dev):
    x = torch.randn(64, 512)
    x[3] = 0
    q, s = per_1x32_f8_quant(x.to(dev))
    q0, s0 = mx_oracle.per_1x32_f8_quant(x)
    assert torch.equal(q.cpu().view(torch.uint8), q0.view(torch.uint8)) and torch.equal(s.cpu(), s0)


@pytest.mark.parametrize("shape", ["1", "2"], ids=["tiles128x128", "tiles128x256"])
@pytest.mark.parametrize("m,n,k", [(300, 512, 1024), (130, 256, 256), (2048, 2048, 4096)])
def test_both_tile_shapes(dev, monkeypatch, shape, m, n, k):
    """FLYB200_MX_BN forces the 128-channel (two accumulators) or the 256-channel (one accumulator) kernel."""
    monkeypatch.setenv("FLYB200_MX_BN", shape)
    a_q, sa, b_q, sb = mx_oracle.make_inputs(m, n, k, seed=m + k)
    c = run(dev, a_q, sa, b_q, sb)
    check(c, mx_oracle.mx_gemm(a_q, sa, b_q, sb))


@pytest.mark.parametrize("m,n,k", [(32, 1024, 2048), (128, 512, 1024), (5, 256, 256), (24, 19200, 256)])
def test_small_m_kernel_and_large_m_kernel_agree(dev, monkeypatch, m, n, k):
    """Up to 128 tokens run the weight-streaming kernel where its CTAs fit one round (the last shape, 150
    channel tiles, goes to the large-M kernel by itself); FLYB200_MX_SMALL=1 / 0 forces one or the other."""
    a_q, sa, b_q, sb = mx_oracle.make_inputs(m, n, k, seed=3 * m + k)
    check(run(dev, a_q, sa, b_q, sb), mx_oracle.mx_gemm(a_q, sa, b_q, sb))  # the automatic choice
    monkeypatch.setenv("FLYB200_MX_SMALL", "1")
    small = run(dev, a_q, sa, b_q, sb)
    monkeypatch.setenv("FLYB200_MX_SMALL", "0")
    large = run(dev, a_q, sa, b_q, sb)
    ref = mx_oracle.mx_gemm(a_q, sa, b_q, sb)
    check(small, ref)
    check(large, ref)
