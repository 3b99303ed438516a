"""GPU parity of the mixed block-scaled kinds (MXFP6 or MXFP8 activations x MXFP4 weights,
tcgen05 kind::mxf8f6f4 on byte containers) against the CPU oracle.  Tolerance as for the other
block-scaled GEMMs: rtol 1e-2 / atol 1e-2 * max|ref| (the reference accepts 0.1,
tests/kernels/test_preshuffle_gemm.py:580)."""

import os

import numpy as np
import pytest
import torch

from flydsl_b200 import _lib
from flydsl_b200.kernels.gemm.mxfp4_preshuffle import (compile_mxfp4_preshuffle_gemm, per_1x32_f4_quant, per_1x32_f6_quant,
                                                       shuffle_scale_w4, shuffle_weight_w4)
from oracle import mx_oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda:0")


def run(dev, a_dtype, a_bytes, sa, b_packed, sb, out_dtype="bf16", packed_weights=False, guard=8):
    m, k = a_bytes.shape
    n = b_packed.shape[0]
    c = torch.full((m + guard, n), 7.0, dtype=torch.bfloat16 if out_dtype == "bf16" else torch.float16, device=dev)
    fn = compile_mxfp4_preshuffle_gemm(N=n, K=k, out_dtype=out_dtype, a_dtype=a_dtype, b_dtype="fp4")
    if packed_weights:  # what the reference's test passes: the image of the packed codes
        w = shuffle_weight_w4(b_packed.to(dev), 16, False, False)
    else:
        w = shuffle_weight_w4(b_packed.to(dev), 16, False, False, for_a_dtype=a_dtype)
    fn(c.view(-1), a_bytes.to(dev).view(torch.uint8).view(-1), w.view(-1), shuffle_scale_w4(sa.to(dev), 1, False),
       shuffle_scale_w4(sb.to(dev), 1, False), torch.empty(0, dtype=torch.bfloat16, device=dev), m, n, torch.cuda.current_stream())
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    assert torch.all(c[m:] == 7.0), "guard rows were written"
    return c[:m]


def check(c, ref):
    got = c.float().cpu()
    tol = 1e-2 * float(ref.abs().max())
    bad = ((got - ref).abs() > tol + 1e-2 * ref.abs()).sum().item()
    assert bad == 0, f"{bad} elements outside tolerance; max abs err {float((got - ref).abs().max()):.4g}"


def fp6_inputs(m, n, k, seed):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(m, k, generator=g)
    b = torch.randn(n, k, generator=g)
    a_pad, sa, a_codes = mx_oracle.per_1x32_f6_quant(a)
    b_q, sb = mx_oracle.per_1x32_f4_quant(b)
    return a_pad, sa, a_codes, b_q, sb


def test_which_element_meets_which(dev):
    """Weights one-hot per channel (a single code 1.0 at element n * 7 % K), activations a different
    value at every position: every output names the activation element the tensor core paired with
    that weight element, so a wrong nibble order, bit offset or padding position cannot pass."""
    m, n, k = 128, 128, 256
    hot = (torch.arange(n) * 7) % k
    w_codes = torch.zeros(n, k, dtype=torch.uint8)
    w_codes[torch.arange(n), hot] = 2  # E2M1 code 2 = 1.0
    b_packed = mx_oracle.pack_fp4(w_codes)
    flat_a = torch.full((m, k // 32), 127, dtype=torch.uint8)
    flat_w = torch.full((n, k // 32), 127, dtype=torch.uint8)
    # fp6 activations: codes cycle through all 64 values with a row-dependent offset
    a_codes = ((torch.arange(k).view(1, k) * 5 + torch.arange(m).view(m, 1) * 3) % 64).to(torch.uint8)
    a_pad = torch.zeros(m, k // 32, 32, dtype=torch.uint8)
    a_pad[:, :, :24] = mx_oracle.pack_fp6(a_codes).view(m, k // 32, 24)
    c = run(dev, "fp6", a_pad.view(m, k), flat_a, b_packed, flat_w)
    check(c, mx_oracle.a6w4_gemm(a_codes, flat_a, b_packed, flat_w))
    # fp8 activations: every E4M3 code that is a finite number
    a8 = ((torch.arange(k).view(1, k) * 3 + torch.arange(m).view(m, 1)) % 120).to(torch.uint8).view(torch.float8_e4m3fn)
    c = run(dev, "fp8", a8.view(torch.uint8), flat_a, b_packed, flat_w)
    check(c, mx_oracle.a8w4_gemm(a8, flat_a, b_packed, flat_w))


def test_golden_fixture_a6w4(dev):
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "mx_fp6.npz"))
    a_pad, sa, b_q, sb = (torch.from_numpy(z[n]) for n in ("a_pad", "sa", "b_q", "sb"))
    n_pad = 128
    b_pad = torch.zeros(n_pad, b_q.shape[1], dtype=torch.uint8)
    b_pad[: b_q.shape[0]] = b_q
    sb_pad = torch.full((n_pad, sb.shape[1]), 127, dtype=torch.uint8)
    sb_pad[: sb.shape[0]] = sb
    c = run(dev, "fp6", a_pad, sa, b_pad, sb_pad)
    check(c[:, : b_q.shape[0]], torch.from_numpy(z["c"]))
    assert torch.all(c[:, b_q.shape[0]:] == 0)


@pytest.mark.parametrize("m,n,k", [(64, 8192, 8192), (32, 8192, 8192), (128, 8192, 8192), (1024, 8192, 8192), (256, 4096, 14336),  # the reference's shapes
                                   (1, 128, 256), (300, 384, 1024), (5133, 512, 2048)])
@pytest.mark.parametrize("out_dtype", ["bf16", "fp16"])
def test_a6w4_gemm(dev, m, n, k, out_dtype):
    a_pad, sa, a_codes, b_q, sb = fp6_inputs(m, n, k, seed=m + n)
    c = run(dev, "fp6", a_pad, sa, b_q, sb, out_dtype)
    check(c, mx_oracle.a6w4_gemm(a_codes, sa, b_q, sb))


@pytest.mark.parametrize("m,n,k", [(64, 8192, 8192), (300, 384, 1024), (1000, 1024, 4096)])
def test_a8w4_gemm(dev, m, n, k):
    g = torch.Generator().manual_seed(m)
    a_q, sa = mx_oracle.per_1x32_f8_quant(torch.randn(m, k, generator=g))
    b_q, sb = mx_oracle.per_1x32_f4_quant(torch.randn(n, k, generator=g))
    c = run(dev, "fp8", a_q.view(torch.uint8), sa, b_q, sb)
    check(c, mx_oracle.a8w4_gemm(a_q, sa, b_q, sb))


def test_packed_weight_image_is_expanded_once(dev):
    """The reference's test passes shuffle_weight_w4(b_q) without saying which activation type
    follows: the launcher expands that packed image to containers on first sight."""
    m, n, k = 40, 256, 512
    a_pad, sa, a_codes, b_q, sb = fp6_inputs(m, n, k, seed=4)
    c = run(dev, "fp6", a_pad, sa, b_q, sb, packed_weights=True)
    check(c, mx_oracle.a6w4_gemm(a_codes, sa, b_q, sb))


def test_device_quantiser_matches_oracle(dev):
    g = torch.Generator().manual_seed(3)
    x = torch.randn(64, 512, generator=g) * torch.exp2(torch.randint(-6, 7, (64, 16), generator=g).float()).repeat_interleave(32, dim=1)
    x[3] = 0
    a_pad, s, codes = per_1x32_f6_quant(x.to(dev))
    a_pad0, s0, codes0 = mx_oracle.per_1x32_f6_quant(x)
    assert torch.equal(a_pad.cpu(), a_pad0) and torch.equal(s.cpu(), s0) and torch.equal(codes.cpu(), codes0)
