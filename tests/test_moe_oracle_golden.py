"""The mixture-of-experts oracle against the fixtures produced by the reference's
own torch functions (tests/golden/make_golden_moe.py), and the host-side routing
helper against both.  CPU only."""

import os

import numpy as np
import pytest
import torch

from oracle import moe_oracle
from flydsl_b200.kernels.moe.moe_gemm_2stage import (
    compile_moe_gemm1,
    compile_moe_gemm2,
    compile_moe_reduction,
    moe_sorting,
)

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
QD = {"fp8": torch.float8_e4m3fn, "int8": torch.int8}


def load(name):
    z = np.load(os.path.join(GOLDEN, f"moe_{name}.npz"))
    d = {k: torch.from_numpy(z[k]) for k in z.files}
    for k in ("x_q", "w1_q", "w2_q", "a2_q"):
        d[k] = d[k].view(QD[name])
    d["dims"] = [int(v) for v in z["dims"]]
    return d


@pytest.mark.parametrize("name", ["fp8", "int8"])
def test_sorting_matches_reference(name):
    d = load(name)
    tokens, _, _, experts, topk, block = d["dims"]
    for fn in (moe_oracle.moe_sorting, lambda i, w, e, b: moe_sorting(i, w, num_experts=e, block_size=b)):
        ids, w, e_ids, post = fn(d["topk_ids"], d["topk_weights"], experts, block)
        assert torch.equal(ids, d["sorted_ids"])
        assert torch.equal(e_ids, d["sorted_expert_ids"])
        assert torch.equal(post, d["post_pad"])
        n = int(post[0])
        valid = (ids[:n] & 0xFFFFFF) < tokens
        assert torch.equal(w[:n] * valid, d["sorted_weights_valid"])


@pytest.mark.parametrize("name", ["fp8", "int8"])
def test_stage1_matches_reference(name):
    d = load(name)
    _, model_dim, inter_dim, experts, _, _ = d["dims"]
    for doweight, key in ((False, "out1"), (True, "out1_weighted")):
        got = moe_oracle.moe_gemm1(
            d["x_q"], d["w1_q"].view(experts * 2 * inter_dim, model_dim), d["scale_x"], d["scale_w1"].view(-1, 1),
            d["topk_ids"].long(), d["topk_weights"], inter_dim, doweight,
        )
        assert torch.equal(got, d[key])


@pytest.mark.parametrize("name", ["fp8", "int8"])
def test_stage2_matches_reference(name):
    d = load(name)
    _, model_dim, _, _, topk, _ = d["dims"]
    for doweight, key in ((True, "out2"), (False, "out2_unweighted")):
        got = moe_oracle.moe_gemm2(
            d["a2_q"], d["w2_q"], d["scale_a2"], d["scale_w2"], d["topk_ids"].long(), d["topk_weights"], model_dim, doweight
        )
        torch.testing.assert_close(got, d[key], rtol=0, atol=0)
        per_slot = moe_oracle.moe_gemm2_per_slot(
            d["a2_q"], d["w2_q"], d["scale_a2"], d["scale_w2"], d["topk_ids"].long(), d["topk_weights"], model_dim, doweight
        )
        torch.testing.assert_close(per_slot.sum(dim=1), d[key], rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("name", ["fp8", "int8"])
def test_stage2_input_is_quantised_stage1_output(name):
    d = load(name)
    a2_q, scale_a2 = moe_oracle.pertoken_quant(d["out1"], QD[name])
    assert torch.equal(a2_q.view(torch.uint8), d["a2_q"].view(torch.uint8))
    assert torch.equal(scale_a2, d["scale_a2"])


def test_stage1_per_route_activations_match_reference():
    """The reference's torch definition with one activation row per (token, slot): the int8smooth case."""
    d = load("int8")
    _, model_dim, inter_dim, experts, _, _ = d["dims"]
    got = moe_oracle.moe_gemm1(
        d["x_route_q"].view(torch.int8), d["w1_q"].view(experts * 2 * inter_dim, model_dim), d["scale_x_route"],
        d["scale_w1"].view(-1, 1), d["topk_ids"].long(), d["topk_weights"], inter_dim, False,
    )
    assert torch.equal(got, d["out1_route"])


def test_make_inputs_is_seeded_and_consistent():
    a = moe_oracle.make_inputs(8, 128, 64, 4, 2, "fp8", seed=5)
    b = moe_oracle.make_inputs(8, 128, 64, 4, 2, "fp8", seed=5)
    assert torch.equal(a["x_q"].view(torch.uint8), b["x_q"].view(torch.uint8))
    assert a["a2_q"].shape == (8, 2, 64) and a["scale_a2"].shape == (8, 2, 1)


def test_sorting_edge_cases():
    # an expert nobody chose, a block size larger than the token count, topk = 1
    ids = torch.tensor([[2], [2], [0]], dtype=torch.int32)
    w = torch.ones(3, 1)
    for fn in (moe_oracle.moe_sorting, lambda i, ww, e, b: moe_sorting(i, ww, num_experts=e, block_size=b)):
        s, _, e, post = fn(ids, w, 4, 32)
        assert post.tolist() == [64, 3]
        assert e.tolist()[:2] == [0, 2] and all(v == -1 for v in e.tolist()[2:])
        assert s[0].item() == 2 and s[32].item() == 0 and s[33].item() == 1
        assert s[1].item() == (1 << 24) | 3  # padding: slot = topk, token = tokens


def test_builders_validate_like_the_reference():
    kw = dict(model_dim=256, inter_dim=128, experts=4, topk=2, tile_m=64, tile_n=64, tile_k=128)
    compile_moe_gemm1(**kw, doweight_stage1=False, out_dtype="bf16", in_dtype="fp8")
    compile_moe_gemm2(**kw, doweight_stage2=True, out_dtype="f32", accumulate=True, in_dtype="int8")
    compile_moe_gemm1(**kw, doweight_stage1=False, out_dtype="f16", in_dtype="int8smooth")
    with pytest.raises(ValueError, match="out_dtype"):
        compile_moe_gemm1(**kw, doweight_stage1=False, out_dtype="f32")
    with pytest.raises(ValueError, match="in_dtype"):
        compile_moe_gemm1(**kw, doweight_stage1=False, in_dtype="fp4")
    compile_moe_gemm1(**kw, doweight_stage1=False, in_dtype="int4")  # W4A8: packed weights, expanded to the int8 image once
    with pytest.raises(ValueError, match="accumulate=False"):
        compile_moe_gemm2(**kw, doweight_stage2=True, out_dtype="f32", accumulate=False)
    with pytest.raises(ValueError, match="tile_m"):
        compile_moe_gemm1(**{**kw, "tile_m": 24}, doweight_stage1=False)
    with pytest.raises(ValueError, match="tile_k"):
        compile_moe_gemm2(**{**kw, "tile_k": 64}, doweight_stage2=True)
    with pytest.raises(ValueError, match="num_experts"):
        compile_moe_reduction(topk=2, model_dim=256, use_mask=True)
    compile_moe_reduction(topk=2, model_dim=256, use_mask=True, num_experts=8)


def test_int4_pack_helper_round_trip():
    from flydsl_b200.kernels.moe.moe_gemm_2stage import pack_shuffled_int8_to_packed_int4, unpack_packed_int4_to_shuffled_int8

    x = torch.arange(-8, 8, dtype=torch.int8).repeat(64)
    packed = pack_shuffled_int8_to_packed_int4(x)
    assert packed.numel() == x.numel() // 2
    # byte j of every 4-byte group holds v_j in the low and v_{j+4} in the high nibble
    assert int(packed.view(torch.uint8)[0]) == ((-8 & 15) | ((-4 & 15) << 4))
    assert torch.equal(unpack_packed_int4_to_shuffled_int8(packed), x)
