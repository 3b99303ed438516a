"""The MXFP8 oracle against the fixture produced by the reference's own utilities. CPU only."""

import os

import numpy as np
import torch

from oracle import mx_oracle

Z = np.load(os.path.join(os.path.dirname(__file__), "golden", "mx_fp8.npz"))


def t(name):
    return torch.from_numpy(Z[name])


def test_e8m0_table():
    got = mx_oracle.e8m0_to_f32(torch.arange(256, dtype=torch.uint8)).view(torch.int32)
    assert torch.equal(got, t("e8m0_table"))


def test_quantiser_matches_reference():
    for x, q, s in (("a", "a_q", "sa"), ("b", "b_q", "sb")):
        codes, scale = mx_oracle.per_1x32_f8_quant(t(x))
        assert torch.equal(codes.view(torch.uint8), t(q))
        assert torch.equal(scale, t(s))


def test_gemm_reference_matches():
    c = mx_oracle.mx_gemm(t("a_q").view(torch.float8_e4m3fn), t("sa"), t("b_q").view(torch.float8_e4m3fn), t("sb"))
    assert torch.equal(c, t("c"))


def test_scale_image_layout():
    rows, kb32 = 130, 8  # two row tiles (the second mostly padding), two 128-element k-blocks
    s = torch.arange(rows * kb32, dtype=torch.int32).remainder(251).to(torch.uint8).view(rows, kb32)
    img = mx_oracle.scale_image(s)
    assert img.numel() == 2 * 2 * 512
    for r, kb in ((0, 0), (31, 3), (32, 4), (77, 5), (129, 7), (128, 0)):
        tile, rr = divmod(r, 128)
        k_block, j = divmod(kb, 4)
        off = (k_block * 2 + tile) * 512 + (rr % 32) * 16 + (rr // 32) * 4 + j
        assert int(img[off]) == int(s[r, kb])
    assert int(img[(0 * 2 + 1) * 512 + (5 % 32) * 16 + 0 + 0]) == 0  # padding row 128 + 5


# --- MXFP4 (E2M1 codes, two per byte): fixture from the reference's per_1x32_f4_quant / mxfp4_to_f32

Z4 = np.load(os.path.join(os.path.dirname(__file__), "golden", "mx_fp4.npz"))


def t4(name):
    return torch.from_numpy(Z4[name])


def test_fp4_rounding_at_every_boundary():
    got = mx_oracle.f32_to_fp4_codes(t4("probe"))
    assert torch.equal(got, t4("probe_codes"))


def test_fp4_decode_table():
    all_bytes = torch.arange(256, dtype=torch.uint8).view(1, 256)
    assert torch.equal(mx_oracle.mxfp4_to_f32(all_bytes), t4("table"))


def test_fp4_quantiser_matches_reference():
    for x, q, s in (("a", "a_q", "sa"), ("b", "b_q", "sb")):
        codes, scale = mx_oracle.per_1x32_f4_quant(t4(x))
        assert torch.equal(codes, t4(q))
        assert torch.equal(scale, t4(s))


def test_fp4_gemm_reference_matches():
    c = mx_oracle.mx4_gemm(t4("a_q"), t4("sa"), t4("b_q"), t4("sb"))
    assert torch.equal(c, t4("c"))


def test_shipped_fp4_quantiser_matches_reference_fixture():
    from flydsl_b200.kernels.gemm.mxfp4_preshuffle import mxfp4_to_f32, per_1x32_f4_quant

    for x, q, s in (("a", "a_q", "sa"), ("b", "b_q", "sb")):
        codes, scale = per_1x32_f4_quant(t4(x))
        assert torch.equal(codes, t4(q)) and torch.equal(scale, t4(s))
    assert torch.equal(mxfp4_to_f32(torch.arange(256, dtype=torch.uint8).view(1, 256)), t4("table"))


# --- MXFP6 activations (E2M3): fixture from the reference's per_1x32_f6_quant / fp6_e2m3_to_f32

Z6 = np.load(os.path.join(os.path.dirname(__file__), "golden", "mx_fp6.npz"))


def t6(name):
    return torch.from_numpy(Z6[name])


def test_fp6_rounding_table_quantiser_and_gemm_match_reference():
    assert torch.equal(mx_oracle.f32_to_fp6_codes(t6("probe")), t6("probe_codes"))
    assert torch.equal(mx_oracle.fp6_to_f32(torch.arange(64, dtype=torch.uint8)), t6("table"))
    a_pad, sa, codes = mx_oracle.per_1x32_f6_quant(t6("a"))
    assert torch.equal(a_pad, t6("a_pad")) and torch.equal(sa, t6("sa")) and torch.equal(codes, t6("a_codes"))
    assert torch.equal(mx_oracle.a6w4_gemm(t6("a_codes"), t6("sa"), t6("b_q"), t6("sb")), t6("c"))


def test_shipped_fp6_helpers_match_reference_fixture():
    from flydsl_b200.kernels.gemm import mxfp4_preshuffle as mp

    a_pad, sa, codes = mp.per_1x32_f6_quant(t6("a"))
    assert torch.equal(a_pad, t6("a_pad")) and torch.equal(sa, t6("sa")) and torch.equal(codes, t6("a_codes"))
    assert torch.equal(mp.fp6_e2m3_to_f32(torch.arange(64, dtype=torch.uint8)), t6("table"))
    # container forms: what the kernel reads
    assert torch.equal(mp.fp6_containers_from_padded(t6("a_pad")), mx_oracle.fp6_containers(t6("a_codes")))
    assert torch.equal(mp.fp4_containers(t6("b_q")), mx_oracle.fp4_containers(t6("b_q")))
    row = mx_oracle.fp6_containers(t6("a_codes"))[0]
    assert int(row[12:16].sum()) == 0 and row.numel() == t6("a_codes").shape[1]  # 12 data bytes + 4 padding per 16 codes
