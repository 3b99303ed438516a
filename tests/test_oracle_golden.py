"""The oracle and the shipped host helpers against fixtures generated from the
reference's own helper module (tests/golden/make_golden.py).  CPU only."""

import os

import numpy as np
import pytest
import torch

from flydsl_b200 import utils as host
from oracle import a8w8_oracle as oracle

GOLD = os.path.join(os.path.dirname(__file__), "golden")
FP8 = torch.float8_e4m3fn


def load(name):
    return np.load(os.path.join(GOLD, name))


def as_dtype(u8, dtype):
    return torch.from_numpy(np.ascontiguousarray(u8)).view(dtype)


@pytest.mark.parametrize("impl", [oracle.pertoken_quant, host.pertoken_quant], ids=["oracle", "host"])
@pytest.mark.parametrize("name,qd", [("fp8", FP8), ("int8", torch.int8)])
def test_pertoken_quant_matches_reference(impl, name, qd):
    g = load(f"quant_{name}.npz")
    y, s = impl(torch.from_numpy(g["x"]), quant_dtype=qd)
    assert torch.equal(y.view(torch.uint8), torch.from_numpy(g["y"]))  # bit-exact bytes
    assert torch.equal(s, torch.from_numpy(g["scale"]))  # bit-exact fp32 scales
    assert s.shape == (g["x"].shape[0], 1) and s.dtype == torch.float32


def test_pertoken_quant_conventions():
    """int8 cast truncates toward zero; zero rows get scale 1; e4m3fn rounds to
    nearest even and the row maximum maps to +-448."""
    x = torch.tensor([[1.6, -1.6, 127.0, 126.7], [0.0, 0.0, 0.0, 0.0]])
    y, s = oracle.pertoken_quant(x, quant_dtype=torch.int8)
    assert y[0].tolist() == [1, -1, 127, 126] and s[1].item() == 1.0
    x = torch.tensor([[448.0, -3.3, 0.07, 224.0]])
    y, s = oracle.pertoken_quant(x, quant_dtype=FP8)
    assert s.item() == 1.0 and y.float()[0, 0].item() == 448.0
    y2, s2 = host.pertoken_quant(x, quant_dtype=FP8)
    assert torch.equal(y.view(torch.uint8), y2.view(torch.uint8))


@pytest.mark.parametrize("name,dtype", [("i8", torch.int8), ("f16", torch.float16)])
def test_reference_layout_restatement(name, dtype):
    g = load(f"shuffle_ref_{name}.npz")
    x = torch.from_numpy(g["x"]) if name == "i8" else as_dtype(g["x"], dtype)
    want = torch.from_numpy(g["y"]) if name == "i8" else as_dtype(g["y"], dtype)
    got = oracle.shuffle_weight_mfma(x)
    assert torch.equal(got.view(torch.uint8), want.view(torch.uint8))
    assert torch.equal(oracle.mfma_to_rowmajor(got), x)
    # converter path: reference-shuffled weights -> B200 image == direct image
    direct = oracle.shuffle_weight_b200(x)
    via = host.shuffle_weight(want, src_layout="mfma")
    assert torch.equal(via.view(torch.uint8), direct.view(torch.uint8))


def test_reference_layout_index_formula():
    """8-bit closed form of the reference layout: byte (n, k) sits at
    ((n/16)*(K/16) + k/16)*256 + (n%16)*16 + k%16."""
    n, k = 48, 128
    x = torch.arange(n * k, dtype=torch.int32).remainder(251).to(torch.int8).view(n, k)
    y = oracle.shuffle_weight_mfma(x).reshape(-1)
    nn, kk = torch.meshgrid(torch.arange(n), torch.arange(k), indexing="ij")
    off = ((nn // 16) * (k // 16) + kk // 16) * 256 + (nn % 16) * 16 + kk % 16
    assert torch.equal(y[off.reshape(-1)].view(n, k), x)


@pytest.mark.parametrize("dtype", [torch.int8, torch.float16, FP8])
@pytest.mark.parametrize("shape", [(16, 128), (48, 384), (3, 32, 256)])
def test_b200_layout_roundtrip_and_host_agreement(dtype, shape):
    if dtype == torch.float16 and shape[-1] * 2 % 128:
        pytest.skip("K*2 not a multiple of 128")
    g = torch.Generator().manual_seed(1)
    x = torch.randint(-100, 100, shape, generator=g).to(torch.float32).to(dtype)
    img = oracle.shuffle_weight_b200(x)
    assert img.shape == x.shape and img.dtype == x.dtype
    assert torch.equal(oracle.unshuffle_weight_b200(img).view(torch.uint8), x.view(torch.uint8))
    himg = host.shuffle_weight(x)
    assert getattr(himg, "is_shuffled", False)
    assert torch.equal(himg.view(torch.uint8), img.view(torch.uint8))
    assert torch.equal(host.unshuffle_weight(himg).view(torch.uint8), x.view(torch.uint8))


def test_b200_layout_is_the_swizzled_smem_image():
    """Row r of k-block b occupies bytes [(b*N + r)*128, +128) and its 16-byte
    chunk c is stored at chunk position c ^ (r % 8)."""
    n, kb = 32, 256
    x = torch.arange(n * kb, dtype=torch.int32).remainder(253).to(torch.uint8).view(n, kb)
    img = oracle.shuffle_weight_b200(x).reshape(kb // 128, n, 8, 16)
    for b in range(kb // 128):
        for r in (0, 1, 7, 8, 13, 31):
            for c in range(8):
                assert torch.equal(img[b, r, c ^ (r % 8)], x[r, b * 128 + c * 16 : b * 128 + c * 16 + 16])


@pytest.mark.parametrize("name", ["fp8", "int8"])
def test_dequant_matmul_check_matches_reference(name):
    g = load(f"gemm_{name}.npz")
    qd = FP8 if name == "fp8" else torch.int8
    a_q, sa = oracle.pertoken_quant(torch.from_numpy(g["a"]), quant_dtype=qd)
    b_q, sb = oracle.pertoken_quant(torch.from_numpy(g["w"]), quant_dtype=qd)
    assert torch.equal(a_q.view(torch.uint8), torch.from_numpy(g["a_q"]))
    assert torch.equal(b_q.view(torch.uint8), torch.from_numpy(g["b_q"]))
    c = oracle.run_torch(a_q, b_q, sa, sb)
    assert torch.allclose(c, torch.from_numpy(g["c"]), rtol=1e-6, atol=1e-5)
    assert torch.equal(oracle.shuffle_weight_mfma(b_q).view(torch.uint8), torch.from_numpy(g["b_shuf_ref"]))
    if name == "int8":
        assert torch.equal(oracle.int32_acc(a_q, b_q), torch.from_numpy(g["acc"]))
        # the scaled epilogue applied to exact accumulators agrees with the fp32 check
        out = oracle.epilogue(oracle.int32_acc(a_q, b_q), sa, sb).float()
        assert oracle.strict_mismatches(out, c) == 0


def test_epilogue_formulas():
    g = torch.Generator().manual_seed(3)
    acc = torch.randn(8, 32, generator=g) * 4
    sa, sb = torch.rand(8, generator=g) + 0.5, torch.rand(32, generator=g) + 0.5
    bias = torch.randn(32, generator=g).to(torch.bfloat16)
    base = (acc * sa[:, None]) * sb[None, :] + bias.float()
    F = torch.nn.functional
    for kind, want in (
        ("bias", base),
        ("bias_relu", F.relu(base)),
        ("bias_silu", F.silu(base)),
        ("bias_gelu", F.gelu(base, approximate="tanh")),
    ):
        got = oracle.epilogue(acc, sa, sb, bias, kind, out_dtype=torch.float32)
        assert torch.allclose(got, want, rtol=1e-5, atol=1e-5), kind


def test_verify_output_rule():
    ref = torch.linspace(-4, 4, 1000)
    assert oracle.verify_output(ref.clone(), ref)
    few = ref.clone()
    few[:40] += 1.0  # 4 % off: still passes the reference's 5 % rule
    assert oracle.verify_output(few, ref)
    assert oracle.strict_mismatches(few, ref) == 40
    many = ref + 1.0
    assert not oracle.verify_output(many, ref)


def test_work_model():
    assert oracle.gemm_flops(128, 4096, 4096) == 2 * 128 * 4096 * 4096
    assert oracle.gemm_bytes(128, 4096, 4096) == 18366976
    assert oracle.gemm_bytes(32, 8192, 8192) == 67928192
