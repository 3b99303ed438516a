"""GPU parity of the MXFP4 x MXFP4 GEMM (tcgen05 kind::mxf4 block-scaled MMA) against the CPU oracle.

Tolerance: the reference accepts rtol = atol = 0.1 (tests/kernels/test_preshuffle_gemm.py:453);
here every element must be within rtol 1e-2 / atol 1e-2 * max|ref| of the fp32 oracle (the
products are exact, only the fp32 summation order and the 16-bit output rounding differ)."""

import os

import numpy as np
import pytest
import torch

from flydsl_b200 import _lib
from flydsl_b200.kernels.gemm.mxfp4_preshuffle import (compile_mxfp4_preshuffle_gemm, per_1x32_f4_quant, shuffle_scale_w4,
                                                       shuffle_weight_w4)
from oracle import mx_oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda:0")


def run(dev, a_q, sa, b_q, sb, out_dtype="bf16", guard=8):
    m, n, k = a_q.shape[0], b_q.shape[0], a_q.shape[1] * 2
    c = torch.full((m + guard, n), 7.0, dtype=torch.bfloat16 if out_dtype == "bf16" else torch.float16, device=dev)
    fn = compile_mxfp4_preshuffle_gemm(N=n, K=k, out_dtype=out_dtype)
    fn(c.view(-1), a_q.to(dev).view(-1), shuffle_weight_w4(b_q.to(dev), 16, False, False).view(-1),
       shuffle_scale_w4(sa.to(dev), 1, False), shuffle_scale_w4(sb.to(dev), 1, False),
       torch.empty(0, dtype=torch.bfloat16, device=dev), m, n, torch.cuda.current_stream())
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    assert torch.all(c[m:] == 7.0), "guard rows were written"
    return c[:m]


def check(c, ref):
    got = c.float().cpu()
    tol = 1e-2 * float(ref.abs().max())
    bad = ((got - ref).abs() > tol + 1e-2 * ref.abs()).sum().item()
    assert bad == 0, f"{bad} elements outside tolerance; max abs err {float((got - ref).abs().max()):.4g}"


def test_which_scale_meets_which_block(dev):
    """All codes 1.0; the weights' scales are all 2^0 and the activations' scale of (row m, block j)
    is 2^j in ONE block and 2^-20 elsewhere, so every output says which block's scale the tensor core
    applied where; then the same with the roles of the operands swapped."""
    m, n, k = 128, 128, 512
    ones = torch.full((m, k // 2), 0x22, dtype=torch.uint8)  # E2M1 code 2 = 1.0 in both nibbles
    blocks = k // 32
    for probe_side in ("a", "w"):
        s_probe = torch.full((m, blocks), 127 - 20, dtype=torch.uint8)
        hot = torch.arange(m) % blocks
        s_probe[torch.arange(m), hot] = (127 + hot % 8).to(torch.uint8)
        s_flat = torch.full((m, blocks), 127, dtype=torch.uint8)
        sa, sb = (s_probe, s_flat) if probe_side == "a" else (s_flat, s_probe)
        c = run(dev, ones, sa, ones, sb)
        check(c, mx_oracle.mx4_gemm(ones, sa, ones, sb))


def test_golden_fixture(dev):
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "mx_fp4.npz"))
    a_q, b_q = torch.from_numpy(z["a_q"]), torch.from_numpy(z["b_q"])
    sa, sb = torch.from_numpy(z["sa"]), torch.from_numpy(z["sb"])
    n_pad = 128  # the fixture has 48 channels: pad the weights to one 128-channel tile with zero codes
    b_pad = torch.zeros(n_pad, b_q.shape[1], dtype=torch.uint8)
    b_pad[: b_q.shape[0]] = b_q
    sb_pad = torch.full((n_pad, sb.shape[1]), 127, dtype=torch.uint8)
    sb_pad[: sb.shape[0]] = sb
    c = run(dev, a_q, sa, b_pad, sb_pad)
    check(c[:, : b_q.shape[0]], torch.from_numpy(z["c"]))
    assert torch.all(c[:, b_q.shape[0]:] == 0)


@pytest.mark.parametrize("m,n,k", [(128, 128, 256), (16, 256, 512), (300, 384, 1024), (1, 128, 256), (1000, 1024, 4096),
                                   (64, 8192, 8192), (32, 8192, 8192), (128, 8192, 8192), (1024, 8192, 8192),  # the reference's shapes
                                   (17, 1024, 4096), (129, 256, 1024)])
@pytest.mark.parametrize("out_dtype", ["bf16", "fp16"])
def test_mxfp4_gemm(dev, m, n, k, out_dtype):
    a_q, sa, b_q, sb = mx_oracle.make_inputs_fp4(m, n, k, seed=m + n)
    c = run(dev, a_q, sa, b_q, sb, out_dtype)
    check(c, mx_oracle.mx4_gemm(a_q, sa, b_q, sb))


def test_ragged_large_m(dev):
    m, n, k = 5133, 1024, 2048  # the reference's ragged M
    a_q, sa, b_q, sb = mx_oracle.make_inputs_fp4(m, n, k, seed=9)
    check(run(dev, a_q, sa, b_q, sb), mx_oracle.mx4_gemm(a_q, sa, b_q, sb))


def test_scales_matter_per_block(dev):
    """Random codes with a different random scale in every 32-element block and row."""
    m, n, k = 128, 256, 1024
    g = torch.Generator().manual_seed(5)
    a_q = torch.randint(0, 256, (m, k // 2), generator=g, dtype=torch.uint8)
    b_q = torch.randint(0, 256, (n, k // 2), generator=g, dtype=torch.uint8)
    sa = torch.randint(120, 134, (m, k // 32), generator=g, dtype=torch.uint8)
    sb = torch.randint(120, 134, (n, k // 32), generator=g, dtype=torch.uint8)
    c = run(dev, a_q, sa, b_q, sb)
    check(c, mx_oracle.mx4_gemm(a_q, sa, b_q, sb))


def test_device_quantiser_matches_oracle(dev):
    g = torch.Generator().manual_seed(2)
    x = torch.randn(64, 512, generator=g) * torch.exp2(torch.randint(-6, 7, (64, 512 // 32), generator=g).float()).repeat_interleave(32, dim=1)
    x[3] = 0
    q, s = per_1x32_f4_quant(x.to(dev))
    q0, s0 = mx_oracle.per_1x32_f4_quant(x)
    assert torch.equal(q.cpu(), q0) and torch.equal(s.cpu(), s0)


@pytest.mark.parametrize("shape", ["1", "2"], ids=["tiles128x128", "tiles128x256"])
@pytest.mark.parametrize("m,n,k", [(300, 512, 1024), (130, 256, 256), (2048, 2048, 8192)])
def test_both_tile_shapes(dev, monkeypatch, shape, m, n, k):
    monkeypatch.setenv("FLYB200_MX_BN", shape)
    a_q, sa, b_q, sb = mx_oracle.make_inputs_fp4(m, n, k, seed=m + k)
    check(run(dev, a_q, sa, b_q, sb), mx_oracle.mx4_gemm(a_q, sa, b_q, sb))


@pytest.mark.parametrize("m,n,k", [(32, 1024, 2048), (128, 512, 1024), (5, 256, 256), (64, 8192, 8192), (100, 384, 4096), (24, 19200, 256)])
def test_small_m_kernel_and_large_m_kernel_agree(dev, monkeypatch, m, n, k):
    """Up to 128 tokens run the weight-streaming kernel where its CTAs fit one round (the last shape, 150
    channel tiles, goes to the large-M kernel by itself); FLYB200_MX_SMALL=1 / 0 forces one or the other."""
    a_q, sa, b_q, sb = mx_oracle.make_inputs_fp4(m, n, k, seed=3 * m + k)
    check(run(dev, a_q, sa, b_q, sb), mx_oracle.mx4_gemm(a_q, sa, b_q, sb))  # the automatic choice
    monkeypatch.setenv("FLYB200_MX_SMALL", "1")
    small = run(dev, a_q, sa, b_q, sb)
    monkeypatch.setenv("FLYB200_MX_SMALL", "0")
    large = run(dev, a_q, sa, b_q, sb)
    ref = mx_oracle.mx4_gemm(a_q, sa, b_q, sb)
    check(small, ref)
    check(large, ref)


def test_small_m_kernel_scale_probe(dev):
    """The which-scale-meets-which-block probe on the weight-streaming kernel (16 tokens)."""
    m, n, k = 16, 256, 1024
    blocks = k // 32
    ones_a = torch.full((m, k // 2), 0x22, dtype=torch.uint8)
    ones_w = torch.full((n, k // 2), 0x22, dtype=torch.uint8)
    sa = torch.full((m, blocks), 127 - 20, dtype=torch.uint8)
    sa[torch.arange(m), (torch.arange(m) * 5) % blocks] = (127 + torch.arange(m) % 8).to(torch.uint8)
    sw = torch.full((n, blocks), 127 - 20, dtype=torch.uint8)
    sw[torch.arange(n), (torch.arange(n) * 3) % blocks] = (127 + torch.arange(n) % 6).to(torch.uint8)
    flat_a = torch.full((m, blocks), 127, dtype=torch.uint8)
    flat_w = torch.full((n, blocks), 127, dtype=torch.uint8)
    check(run(dev, ones_a, sa, ones_w, flat_w), mx_oracle.mx4_gemm(ones_a, sa, ones_w, flat_w))
    check(run(dev, ones_a, flat_a, ones_w, sw), mx_oracle.mx4_gemm(ones_a, flat_a, ones_w, sw))
