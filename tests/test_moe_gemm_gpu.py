"""GPU parity of the two-stage mixture-of-experts GEMM against the CPU oracle,
through the reference's operator surface (compile_moe_gemm1 / compile_moe_gemm2 /
compile_moe_reduction).  The cases follow tests/kernels/test_moe_gemm_2stage.py
of the reference: numeric checks for both stages (atomic and per-slot output),
the output canary, padded-row sentinels and the num_valid_ids guard.

Tolerances: the reference accepts cosine similarity > 0.99.  Here, in addition,
every element must be within 2e-2 of the fp32 oracle relative to the largest
reference magnitude (the outputs are 16-bit; atomic accumulation in 16 bits
rounds once per added slot)."""

import pytest
import torch

from flydsl_b200 import _lib, compiler as flyc, shuffle_weight
from flydsl_b200.kernels.moe.moe_gemm_2stage import (
    compile_moe_gemm1,
    compile_moe_gemm2,
    compile_moe_reduction,
    moe_sorting,
)
from oracle import moe_oracle

pytestmark = pytest.mark.gpu

OUT_T = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}
SHAPE = dict(model_dim=256, inter_dim=128, experts=4, topk=2)  # the reference's small tile-valid shape


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda:0")


def close_enough(got, ref, what, rel=2e-2):
    got = got.float().cpu()
    cos = moe_oracle.cosine_sim(got, ref)
    assert cos > 0.99, f"{what}: cosine {cos:.5f}"
    bound = rel * float(ref.abs().max())
    err = float((got - ref).abs().max())
    assert err <= bound, f"{what}: max abs error {err:.4g} > {bound:.4g}"


def routing_on(dev, d, experts, tile_m):
    ids, w, e_ids, post = moe_sorting(d["topk_ids"].to(dev), d["topk_weights"].to(dev), num_experts=experts, block_size=tile_m)
    return ids, w, e_ids, post[:1].contiguous(), int(e_ids.numel())


def run_stage1(dev, d, *, model_dim, inter_dim, experts, topk, tile_m, in_dtype, out_dtype, doweight=False, tile_n=64,
               extra_rows=0, routing=None, use_compile=False):
    tokens = d["x_q"].shape[0]
    ids, w, e_ids, n_valid, blocks = routing or routing_on(dev, d, experts, tile_m)
    x = d["x_q"].to(dev)
    w1 = shuffle_weight(d["w1_q"].to(dev)).view(experts * 2 * inter_dim, model_dim).contiguous()
    out = torch.full((tokens * topk + extra_rows, inter_dim), 7.0, dtype=OUT_T[out_dtype], device=dev)
    exe = compile_moe_gemm1(model_dim=model_dim, inter_dim=inter_dim, experts=experts, topk=topk, tile_m=tile_m,
                            tile_n=tile_n, tile_k=128, doweight_stage1=doweight, out_dtype=out_dtype, in_dtype=in_dtype)
    args = (out, x.view(-1), w1.view(-1), d["scale_x"].to(dev).view(-1), d["scale_w1"].to(dev).view(-1), ids, e_ids,
            w.view(-1), n_valid, tokens, inter_dim, model_dim, blocks, torch.cuda.current_stream())
    fn = flyc.compile(exe, *args) if use_compile else exe
    fn(*args)
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    return out


def run_stage2(dev, d, *, model_dim, inter_dim, experts, topk, tile_m, in_dtype, out_dtype, accumulate, doweight=True,
               tile_n=64, extra_rows=0, routing=None):
    tokens = d["x_q"].shape[0]
    ids, w, e_ids, n_valid, blocks = routing or routing_on(dev, d, experts, tile_m)
    a2 = d["a2_q"].to(dev)
    w2 = shuffle_weight(d["w2_q"].to(dev)).view(experts * model_dim, inter_dim).contiguous()
    rows = tokens if accumulate else tokens * topk
    out = torch.zeros((rows + extra_rows, model_dim), dtype=OUT_T[out_dtype], device=dev)
    if extra_rows:
        out[rows:] = 7.0
    exe = compile_moe_gemm2(model_dim=model_dim, inter_dim=inter_dim, experts=experts, topk=topk, tile_m=tile_m,
                            tile_n=tile_n, tile_k=128, doweight_stage2=doweight, out_dtype=out_dtype,
                            accumulate=accumulate, in_dtype=in_dtype)
    exe(out, a2.view(-1), w2.view(-1), d["scale_a2"].to(dev).view(-1), d["scale_w2"].to(dev).view(-1), ids, e_ids,
        w.view(-1), n_valid, tokens, model_dim, inter_dim, blocks, torch.cuda.current_stream())
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    return out


def ref_stage1(d, inter_dim, doweight=False):
    experts = d["w1_q"].shape[0]
    return moe_oracle.moe_gemm1(d["x_q"], d["w1_q"].view(experts * 2 * inter_dim, -1), d["scale_x"],
                                d["scale_w1"].view(-1, 1), d["topk_ids"].long(), d["topk_weights"], inter_dim, doweight)


def ref_stage2(d, model_dim, doweight=True):
    return moe_oracle.moe_gemm2(d["a2_q"], d["w2_q"], d["scale_a2"], d["scale_w2"], d["topk_ids"].long(),
                                d["topk_weights"], model_dim, doweight)


# --- the reference's numeric tests --------------------------------------------------------


@pytest.mark.parametrize("in_dtype", ["fp8", "int8"])
@pytest.mark.parametrize("out_dtype", ["f16", "bf16"])
@pytest.mark.parametrize("tile_m,tokens", [(64, 128), (16, 8)])
def test_moe_gemm1_numeric(dev, in_dtype, out_dtype, tile_m, tokens):
    d = moe_oracle.make_inputs(tokens, SHAPE["model_dim"], SHAPE["inter_dim"], SHAPE["experts"], SHAPE["topk"], in_dtype, seed=tokens)
    out = run_stage1(dev, d, **SHAPE, tile_m=tile_m, in_dtype=in_dtype, out_dtype=out_dtype, use_compile=True)
    close_enough(out.view(tokens, SHAPE["topk"], -1), ref_stage1(d, SHAPE["inter_dim"]), "stage 1")


@pytest.mark.parametrize("in_dtype", ["fp8", "int8"])
@pytest.mark.parametrize("accumulate,out_dtype", [(True, "f16"), (True, "bf16"), (True, "f32"), (False, "f16"), (False, "bf16")])
@pytest.mark.parametrize("tile_m,tokens", [(16, 8), (64, 128)])
def test_moe_gemm2_numeric(dev, accumulate, out_dtype, tile_m, tokens, in_dtype):
    d = moe_oracle.make_inputs(tokens, SHAPE["model_dim"], SHAPE["inter_dim"], SHAPE["experts"], SHAPE["topk"], in_dtype, seed=100 + tokens)
    out = run_stage2(dev, d, **SHAPE, tile_m=tile_m, in_dtype=in_dtype, out_dtype=out_dtype, accumulate=accumulate)
    got = out if accumulate else out.view(tokens, SHAPE["topk"], -1).float().sum(dim=1)
    close_enough(got, ref_stage2(d, SHAPE["model_dim"]), "stage 2")


# --- wider shapes: several blocks per expert, partial channel tiles, odd routing block sizes ---


@pytest.mark.parametrize(
    "tokens,model_dim,inter_dim,experts,topk,tile_m",
    [
        (300, 1024, 512, 8, 2, 32),    # many blocks per expert
        (300, 512, 256, 8, 4, 128),
        (1000, 512, 256, 4, 2, 256),   # widest routing block
        (40, 384, 256, 4, 2, 48),      # tile_m not a power of two; odd number of 128-channel tiles in stage 2
        (5, 256, 128, 16, 4, 16),      # more experts than routed rows: most experts have no block
        (1, 128, 128, 2, 1, 16),       # one token, topk 1
    ],
)
@pytest.mark.parametrize("in_dtype", ["fp8", "int8"])
def test_both_stages_wider_shapes(dev, in_dtype, tokens, model_dim, inter_dim, experts, topk, tile_m):
    d = moe_oracle.make_inputs(tokens, model_dim, inter_dim, experts, topk, in_dtype, seed=tokens + experts)
    kw = dict(model_dim=model_dim, inter_dim=inter_dim, experts=experts, topk=topk, tile_m=tile_m, in_dtype=in_dtype)
    out1 = run_stage1(dev, d, **kw, out_dtype="bf16")
    close_enough(out1.view(tokens, topk, -1), ref_stage1(d, inter_dim), "stage 1")
    out2 = run_stage2(dev, d, **kw, out_dtype="bf16", accumulate=False)
    per_slot = moe_oracle.moe_gemm2_per_slot(d["a2_q"], d["w2_q"], d["scale_a2"], d["scale_w2"], d["topk_ids"].long(),
                                             d["topk_weights"], model_dim, True)
    close_enough(out2.view(tokens, topk, -1), per_slot, "stage 2 per slot")
    out2a = run_stage2(dev, d, **kw, out_dtype="f32", accumulate=True)
    close_enough(out2a, ref_stage2(d, model_dim), "stage 2 accumulated", rel=2e-3)


def test_stage1_partial_channel_tile(dev):
    """inter_dim = 192: the second channel tile of stage 1 has 64 of its 128 channels."""
    tokens, model_dim, inter_dim, experts, topk = 50, 256, 192, 4, 2
    g = torch.Generator().manual_seed(12)
    ids, wts = moe_oracle.make_routing(tokens, experts, topk, g)
    x_q, sx = moe_oracle.pertoken_quant(torch.randn(tokens, model_dim, generator=g), torch.float8_e4m3fn)
    w1_q, sw1 = moe_oracle.pertoken_quant(torch.randn(experts, 2 * inter_dim, model_dim, generator=g) / 16, torch.float8_e4m3fn)
    d = dict(topk_ids=ids, topk_weights=wts, x_q=x_q, scale_x=sx, w1_q=w1_q, scale_w1=sw1)
    out = run_stage1(dev, d, model_dim=model_dim, inter_dim=inter_dim, experts=experts, topk=topk, tile_m=32,
                     in_dtype="fp8", out_dtype="bf16", extra_rows=8)
    close_enough(out[: tokens * topk].view(tokens, topk, -1), ref_stage1(d, inter_dim), "stage 1, inter_dim 192")
    assert torch.all(out[tokens * topk:] == 7.0)


@pytest.mark.parametrize("in_dtype", ["fp8", "int8"])
@pytest.mark.parametrize("out_dtype", ["f16", "bf16"])
def test_large_routing_blocks_all_outputs(dev, in_dtype, out_dtype):
    """tile_m = 128 runs the persistent form (tokens on the UMMA M side): every output mode,
    a last channel tile of 64 channels in stage 1 and an odd number of tiles in stage 2."""
    tokens, model_dim, inter_dim, experts, topk, tile_m = 333, 384, 256, 4, 2, 128
    d = moe_oracle.make_inputs(tokens, model_dim, inter_dim, experts, topk, in_dtype, seed=33)
    kw = dict(model_dim=model_dim, inter_dim=inter_dim, experts=experts, topk=topk, tile_m=tile_m, in_dtype=in_dtype)
    out1 = run_stage1(dev, d, **kw, out_dtype=out_dtype, extra_rows=16)
    close_enough(out1[: tokens * topk].view(tokens, topk, -1), ref_stage1(d, inter_dim), "stage 1")
    assert torch.all(out1[tokens * topk:] == 7.0)
    for accumulate in (True, False):
        out2 = run_stage2(dev, d, **kw, out_dtype=out_dtype, accumulate=accumulate, extra_rows=16)
        rows = tokens if accumulate else tokens * topk
        got = out2[:rows] if accumulate else out2[:rows].view(tokens, topk, -1).float().sum(dim=1)
        close_enough(got, ref_stage2(d, model_dim), f"stage 2 accumulate={accumulate}")
        assert torch.all(out2[rows:] == 7.0)


@pytest.mark.parametrize("tile_m,experts,tokens", [(128, 4, 500), (64, 4, 500), (64, 16, 90), (64, 3, 33)])
def test_both_kernel_forms_agree(dev, monkeypatch, tile_m, experts, tokens):
    """The persistent form and the two-tiles-per-CTA form do the same arithmetic per output element.
    With 64-row routing blocks the persistent form works a 128-row block twice where the expert
    changes inside it (many experts with few rows: nearly every block)."""
    model_dim, inter_dim, topk = 512, 384, 2
    d = moe_oracle.make_inputs(tokens, model_dim, inter_dim, experts, topk, "fp8", seed=34)
    kw = dict(model_dim=model_dim, inter_dim=inter_dim, experts=experts, topk=topk, tile_m=tile_m, in_dtype="fp8")
    a1 = run_stage1(dev, d, **kw, out_dtype="bf16")
    a2 = run_stage2(dev, d, **kw, out_dtype="bf16", accumulate=False)
    monkeypatch.setenv("FLYB200_MOE_KERNEL", "1")
    b1 = run_stage1(dev, d, **kw, out_dtype="bf16")
    b2 = run_stage2(dev, d, **kw, out_dtype="bf16", accumulate=False)
    assert torch.equal(a1, b1) and torch.equal(a2, b2)


def test_stage1_partial_tile_large_block(dev):
    tokens, model_dim, inter_dim, experts, topk = 150, 256, 192, 2, 2
    g = torch.Generator().manual_seed(13)
    ids, wts = moe_oracle.make_routing(tokens, experts, topk, g)
    x_q, sx = moe_oracle.pertoken_quant(torch.randn(tokens, model_dim, generator=g), torch.int8)
    w1_q, sw1 = moe_oracle.pertoken_quant(torch.randn(experts, 2 * inter_dim, model_dim, generator=g) / 16, torch.int8)
    d = dict(topk_ids=ids, topk_weights=wts, x_q=x_q, scale_x=sx, w1_q=w1_q, scale_w1=sw1)
    out = run_stage1(dev, d, model_dim=model_dim, inter_dim=inter_dim, experts=experts, topk=topk, tile_m=256,
                     in_dtype="int8", out_dtype="bf16", extra_rows=8)
    close_enough(out[: tokens * topk].view(tokens, topk, -1), ref_stage1(d, inter_dim), "stage 1, inter_dim 192, tile_m 256")
    assert torch.all(out[tokens * topk:] == 7.0)


def test_stage1_routed_weight(dev):
    d = moe_oracle.make_inputs(64, 256, 128, 4, 2, "fp8", seed=9)
    out = run_stage1(dev, d, **SHAPE, tile_m=32, in_dtype="fp8", out_dtype="bf16", doweight=True)
    close_enough(out.view(64, 2, -1), ref_stage1(d, 128, doweight=True), "stage 1 with routed weight")


def test_stage2_without_routed_weight(dev):
    d = moe_oracle.make_inputs(64, 256, 128, 4, 2, "int8", seed=10)
    out = run_stage2(dev, d, **SHAPE, tile_m=32, in_dtype="int8", out_dtype="f32", accumulate=True, doweight=False)
    close_enough(out, ref_stage2(d, 256, doweight=False), "stage 2 without routed weight", rel=2e-3)


# --- guards: rows that are not routed stay untouched -----------------------------------------


@pytest.mark.parametrize("in_dtype", ["fp8", "int8"])
@pytest.mark.parametrize("tile_m,tokens", [(16, 8), (64, 100)])
def test_output_canary(dev, in_dtype, tile_m, tokens):
    d = moe_oracle.make_inputs(tokens, SHAPE["model_dim"], SHAPE["inter_dim"], SHAPE["experts"], SHAPE["topk"], in_dtype, seed=3)
    out1 = run_stage1(dev, d, **SHAPE, tile_m=tile_m, in_dtype=in_dtype, out_dtype="bf16", extra_rows=64)
    assert torch.all(out1[tokens * SHAPE["topk"]:] == 7.0)
    for accumulate in (True, False):
        out2 = run_stage2(dev, d, **SHAPE, tile_m=tile_m, in_dtype=in_dtype, out_dtype="bf16", accumulate=accumulate, extra_rows=64)
        rows = tokens if accumulate else tokens * SHAPE["topk"]
        assert torch.all(out2[rows:] == 7.0)


def test_num_valid_ids_guard(dev):
    """Blocks at or past num_valid_ids[0] do no work (tests/kernels/test_moe_gemm_2stage.py:1810-1866)."""
    tokens, tile_m = 64, 16
    d = moe_oracle.make_inputs(tokens, SHAPE["model_dim"], SHAPE["inter_dim"], SHAPE["experts"], SHAPE["topk"], "fp8", seed=4)
    ids, w, e_ids, n_valid, blocks = routing_on(dev, d, SHAPE["experts"], tile_m)
    cut = (int(n_valid[0]) // tile_m // 2) * tile_m  # only the first half of the blocks is in use
    n_cut = torch.tensor([cut], dtype=torch.int32, device=dev)
    out1 = run_stage1(dev, d, **SHAPE, tile_m=tile_m, in_dtype="fp8", out_dtype="bf16", routing=(ids, w, e_ids, n_cut, blocks))
    ref = ref_stage1(d, SHAPE["inter_dim"]).view(tokens * SHAPE["topk"], -1)
    keep = torch.zeros(tokens * SHAPE["topk"], dtype=torch.bool)
    srt = ids.cpu()[:cut]
    tok, slot = srt & 0xFFFFFF, srt >> 24
    ok = tok < tokens
    keep[(tok[ok] * SHAPE["topk"] + slot[ok]).long()] = True
    got = out1.float().cpu()
    assert torch.all(got[~keep] == 7.0)
    close_enough(got[keep], ref[keep], "rows of the blocks in use")


def test_expert_id_minus_one_blocks_are_skipped(dev):
    tokens, tile_m = 32, 16
    d = moe_oracle.make_inputs(tokens, SHAPE["model_dim"], SHAPE["inter_dim"], SHAPE["experts"], SHAPE["topk"], "int8", seed=6)
    ids, w, e_ids, n_valid, blocks = routing_on(dev, d, SHAPE["experts"], tile_m)
    e_ids = e_ids.clone()
    e_ids[0] = -1  # the first block loses its expert
    out = run_stage2(dev, d, **SHAPE, tile_m=tile_m, in_dtype="int8", out_dtype="bf16", accumulate=False,
                     routing=(ids, w, e_ids, n_valid, blocks))
    srt = ids.cpu()[:tile_m]
    tok, slot = srt & 0xFFFFFF, srt >> 24
    ok = tok < tokens
    rows = (tok[ok] * SHAPE["topk"] + slot[ok]).long()
    assert torch.all(out.cpu()[rows] == 0)


# --- the pieces around the GEMM ---------------------------------------------------------------


def test_gather_rows_bit_exact(dev):
    lib = _lib.load()
    tokens, topk, experts, tile_m, k = 37, 2, 4, 16, 256
    g = torch.Generator().manual_seed(1)
    ids_t, w_t = moe_oracle.make_routing(tokens, experts, topk, g)
    ids, _, e_ids, post = moe_sorting(ids_t.to(dev), w_t.to(dev), num_experts=experts, block_size=tile_m)
    rows = int(e_ids.numel()) * tile_m
    for by_slot in (0, 1):
        n_src = tokens * (topk if by_slot else 1)
        src = torch.randint(0, 256, (n_src, k), dtype=torch.uint8, generator=g).to(dev)
        ssc = torch.rand(n_src, generator=g).to(dev)
        dst = torch.full((rows, k), 0xAB, dtype=torch.uint8, device=dev)
        dsc = torch.full((rows,), -1.0, device=dev)
        _lib.check(lib.flyb200_moe_gather_rows(dst.data_ptr(), dsc.data_ptr(), src.data_ptr(), ssc.data_ptr(), ids.data_ptr(),
                                               post.data_ptr(), tokens, topk, by_slot, k, rows, None), "gather")
        torch.cuda.synchronize()
        srt = torch.full((rows,), (topk << 24) | tokens, dtype=torch.int64)  # the id list may end inside the last block
        srt[: min(rows, ids.numel())] = ids.cpu()[:rows].long()
        tok, slot = srt & 0xFFFFFF, srt >> 24
        valid = (tok < tokens) & (torch.arange(rows) < int(post[0]))
        want = torch.zeros((rows, k), dtype=torch.uint8)
        want_s = torch.zeros(rows)
        r = (tok * topk + slot) if by_slot else tok
        want[valid] = src.cpu()[r[valid]]
        want_s[valid] = ssc.cpu()[r[valid]]
        assert torch.equal(dst.cpu(), want) and torch.equal(dsc.cpu(), want_s)


@pytest.mark.parametrize("dtype_str", ["f16", "bf16"])
def test_topk_reduction(dev, dtype_str):
    tokens, topk, dim = 77, 4, 384
    x = torch.randn(tokens, topk, dim, device=dev).to(OUT_T[dtype_str])
    y = torch.full((tokens + 3, dim), 7.0, dtype=OUT_T[dtype_str], device=dev)
    compile_moe_reduction(topk=topk, model_dim=dim, dtype_str=dtype_str)(x, y, None, None, tokens, torch.cuda.current_stream())
    torch.cuda.synchronize()
    assert torch.equal(y[:tokens], x.float().sum(dim=1).to(OUT_T[dtype_str]))
    assert torch.all(y[tokens:] == 7.0)


def test_two_stage_pipeline_end_to_end(dev):
    """x -> stage 1 -> per-token quantisation on the GPU -> stage 2 (per slot) -> top-k reduction."""
    from flydsl_b200 import pertoken_quant

    tokens, model_dim, inter_dim, experts, topk, tile_m = 200, 512, 256, 8, 2, 64
    d = moe_oracle.make_inputs(tokens, model_dim, inter_dim, experts, topk, "fp8", seed=21)
    kw = dict(model_dim=model_dim, inter_dim=inter_dim, experts=experts, topk=topk, tile_m=tile_m, in_dtype="fp8")
    out1 = run_stage1(dev, d, **kw, out_dtype="bf16")
    a2_q, a2_s = pertoken_quant(out1.view(tokens, topk, inter_dim), quant_dtype=torch.float8_e4m3fn)
    d2 = dict(d, a2_q=a2_q.cpu(), scale_a2=a2_s.cpu())
    out2 = run_stage2(dev, d2, **kw, out_dtype="bf16", accumulate=False)
    y = torch.empty(tokens, model_dim, dtype=torch.bfloat16, device=dev)
    compile_moe_reduction(topk=topk, model_dim=model_dim, dtype_str="bf16")(out2, y, None, None, tokens, None)
    torch.cuda.synchronize()
    # oracle on the same chain, with its own (fp32) stage-1 output quantised
    close_enough(y, ref_stage2(d, model_dim), "two-stage pipeline", rel=5e-2)


@pytest.mark.parametrize("tile_m", [16, 128])
def test_graph_replay_equals_eager(dev, tile_m):
    """Both stages capture into a CUDA graph (no allocation or synchronisation on the launch path
    once the gather scratch exists) and the replay reproduces the eager result bit for bit."""
    tokens, model_dim, inter_dim, experts, topk = 96, 256, 128, 4, 2
    d = moe_oracle.make_inputs(tokens, model_dim, inter_dim, experts, topk, "fp8", seed=40 + tile_m)
    ids, w, e_ids, n_valid, blocks = routing_on(dev, d, experts, tile_m)
    kw = dict(model_dim=model_dim, inter_dim=inter_dim, experts=experts, topk=topk, tile_m=tile_m, tile_n=64, tile_k=128,
              out_dtype="bf16", in_dtype="fp8")
    g1 = compile_moe_gemm1(**kw, doweight_stage1=False)
    g2 = compile_moe_gemm2(**kw, doweight_stage2=True, accumulate=False)
    x, a2 = d["x_q"].to(dev), d["a2_q"].to(dev)
    w1 = shuffle_weight(d["w1_q"].to(dev))
    w2 = shuffle_weight(d["w2_q"].to(dev))
    sx, sa2 = d["scale_x"].to(dev).view(-1), d["scale_a2"].to(dev).view(-1)
    sw1, sw2 = d["scale_w1"].to(dev).view(-1), d["scale_w2"].to(dev).view(-1)
    out1 = torch.zeros(tokens * topk, inter_dim, dtype=torch.bfloat16, device=dev)
    out2 = torch.zeros(tokens * topk, model_dim, dtype=torch.bfloat16, device=dev)
    st = torch.cuda.Stream()

    def both():
        g1(out1, x.view(-1), w1.view(-1), sx, sw1, ids, e_ids, w, n_valid, tokens, inter_dim, model_dim, blocks, st)
        g2(out2, a2.view(-1), w2.view(-1), sa2, sw2, ids, e_ids, w, n_valid, tokens, model_dim, inter_dim, blocks, st.cuda_stream)

    with torch.cuda.stream(st):
        both()  # eager: also creates the gather scratch
        st.synchronize()
        eager1, eager2 = out1.clone(), out2.clone()
        out1.zero_()
        out2.zero_()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=st):
            both()
        out1.zero_()
        out2.zero_()
        graph.replay()
        st.synchronize()
    assert torch.equal(out1, eager1) and torch.equal(out2, eager2)
    assert _lib.read_status() == 0
    close_enough(out1.view(tokens, topk, -1), ref_stage1(d, inter_dim), "stage 1 from the graph")


def test_launch_argument_checks(dev):
    d = moe_oracle.make_inputs(8, 256, 128, 4, 2, "fp8", seed=2)
    ids, w, e_ids, n_valid, blocks = routing_on(dev, d, 4, 16)
    exe = compile_moe_gemm1(**SHAPE, tile_m=16, tile_n=64, tile_k=128, doweight_stage1=False, out_dtype="bf16", in_dtype="fp8")
    x = d["x_q"].to(dev)
    w1 = shuffle_weight(d["w1_q"].to(dev))
    sx, sw1 = d["scale_x"].to(dev).view(-1), d["scale_w1"].to(dev).view(-1)
    out = torch.zeros(16, 128, dtype=torch.bfloat16, device=dev)
    good = (out, x.view(-1), w1.view(-1), sx, sw1, ids, e_ids, w, n_valid, 8, 128, 256, blocks, None)
    exe(*good)
    with pytest.raises(ValueError, match="dims"):
        exe(*good[:10], 256, 128, blocks, None)
    with pytest.raises(ValueError, match="out must be"):
        exe(out.half(), *good[1:])
    with pytest.raises(ValueError, match="holds"):
        exe(out[:4], *good[1:])
    with pytest.raises(ValueError, match="int32"):
        exe(*good[:5], ids.long(), *good[6:])
    with pytest.raises(TypeError):
        exe(*good[:13], "stream")
    torch.cuda.synchronize()


@pytest.mark.parametrize(
    "tokens,experts,topk,block",
    [(8, 4, 2, 16), (128, 4, 2, 64), (1000, 8, 2, 128), (5, 16, 4, 16), (1, 2, 1, 16), (4096, 64, 8, 32), (300, 256, 6, 16)],
)
def test_device_sorting_matches_oracle(dev, tokens, experts, topk, block):
    g = torch.Generator().manual_seed(tokens + experts)
    ids, wts = moe_oracle.make_routing(tokens, experts, topk, g)
    want = moe_oracle.moe_sorting(ids, wts, experts, block)
    got = moe_sorting(ids.to(dev), wts.to(dev), num_experts=experts, block_size=block)
    torch.cuda.synchronize()
    for name, a, b in zip(("sorted_ids", "sorted_weights", "sorted_expert_ids", "post_pad"), got, want):
        assert torch.equal(a.cpu(), b), name


def test_device_sorting_skewed_routing(dev):
    """Everything routed to one expert; an expert id outside the range is ignored."""
    ids = torch.full((70, 2), 3, dtype=torch.int32)
    ids[:, 1] = 0
    wts = torch.rand(70, 2)
    want = moe_oracle.moe_sorting(ids, wts, 5, 32)
    got = moe_sorting(ids.to(dev), wts.to(dev), num_experts=5, block_size=32)
    for a, b in zip(got, want):
        assert torch.equal(a.cpu(), b)
    ids[0, 0] = 9
    got = moe_sorting(ids.to(dev), wts.to(dev), num_experts=5, block_size=32)
    assert int(got[3][0]) == 96 + 96  # 69 -> 96 rows for expert 3, 70 -> 96 for expert 0


def test_whole_layer_in_one_graph(dev):
    """Routing table, both stages, the quantiser in between and the top-k reduction captured into
    ONE CUDA graph: nothing on the path synchronises with the host."""
    from flydsl_b200 import pertoken_quant

    tokens, model_dim, inter_dim, experts, topk, tile_m = 64, 256, 128, 4, 2, 32
    d = moe_oracle.make_inputs(tokens, model_dim, inter_dim, experts, topk, "fp8", seed=50)
    kw = dict(model_dim=model_dim, inter_dim=inter_dim, experts=experts, topk=topk, tile_m=tile_m, tile_n=64, tile_k=128,
              out_dtype="bf16", in_dtype="fp8")
    g1 = compile_moe_gemm1(**kw, doweight_stage1=False)
    g2 = compile_moe_gemm2(**kw, doweight_stage2=True, accumulate=False)
    red = compile_moe_reduction(topk=topk, model_dim=model_dim, dtype_str="bf16")
    x = d["x_q"].to(dev)
    w1, w2 = shuffle_weight(d["w1_q"].to(dev)), shuffle_weight(d["w2_q"].to(dev))
    sx, sw1, sw2 = d["scale_x"].to(dev).view(-1), d["scale_w1"].to(dev).view(-1), d["scale_w2"].to(dev).view(-1)
    t_ids, t_w = d["topk_ids"].to(dev), d["topk_weights"].to(dev)
    y = torch.zeros(tokens, model_dim, dtype=torch.bfloat16, device=dev)
    st = torch.cuda.Stream()

    def layer():
        ids, w, e_ids, post = moe_sorting(t_ids, t_w, num_experts=experts, block_size=tile_m)
        blocks = int(e_ids.numel())
        out1 = torch.empty(tokens * topk, inter_dim, dtype=torch.bfloat16, device=dev)
        g1(out1, x.view(-1), w1.view(-1), sx, sw1, ids, e_ids, w, post, tokens, inter_dim, model_dim, blocks, st)
        a2, sa2 = pertoken_quant(out1, quant_dtype=torch.float8_e4m3fn)
        out2 = torch.empty(tokens * topk, model_dim, dtype=torch.bfloat16, device=dev)
        g2(out2, a2.view(-1), w2.view(-1), sa2.view(-1), sw2, ids, e_ids, w, post, tokens, model_dim, inter_dim, blocks, st)
        red(out2, y, None, None, tokens, st)

    with torch.cuda.stream(st):
        layer()
        st.synchronize()
        eager = y.clone()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=st):
            layer()
        y.zero_()
        graph.replay()
        st.synchronize()
    assert torch.equal(y, eager)
    close_enough(y, ref_stage2(d, model_dim), "whole layer", rel=5e-2)
    assert _lib.read_status() == 0


@pytest.mark.parametrize("tile_m,tokens", [(16, 8), (64, 128), (128, 300)])
def test_int8smooth_stage1(dev, tile_m, tokens):
    """in_dtype="int8smooth": x and scale_x are slot-major [topk * tokens, ...] with one quantised row
    per route (tests/kernels/test_moe_gemm_2stage.py:487-583 of the reference)."""
    g = torch.Generator().manual_seed(60 + tokens)
    ids, wts = moe_oracle.make_routing(tokens, SHAPE["experts"], SHAPE["topk"], g)
    x = torch.randn(tokens, SHAPE["model_dim"], generator=g)
    w1 = torch.randn(SHAPE["experts"], 2 * SHAPE["inter_dim"], SHAPE["model_dim"], generator=g) / 16
    w1_q, sw1 = moe_oracle.pertoken_quant(w1, torch.int8)
    sm = moe_oracle.smooth_stage1_inputs(x, w1, ids, g)
    ref = moe_oracle.moe_gemm1(sm["x_ref"], w1_q.view(-1, SHAPE["model_dim"]), sm["sx_ref"], sw1.view(-1, 1), ids.long(), wts,
                               SHAPE["inter_dim"], False)
    d = dict(topk_ids=ids, topk_weights=wts, x_q=sm["x_slot_major"], scale_x=sm["sx_slot_major"], w1_q=w1_q, scale_w1=sw1)
    tokens_topk = tokens * SHAPE["topk"]
    srt, w, e_ids, post = moe_sorting(ids.to(dev), wts.to(dev), num_experts=SHAPE["experts"], block_size=tile_m)
    out = torch.full((tokens_topk + 8, SHAPE["inter_dim"]), 7.0, dtype=torch.bfloat16, device=dev)
    exe = compile_moe_gemm1(**SHAPE, tile_m=tile_m, tile_n=64, tile_k=128, doweight_stage1=False, out_dtype="bf16",
                            in_dtype="int8smooth")
    exe(out, d["x_q"].to(dev).view(-1), shuffle_weight(w1_q.to(dev)).view(-1), d["scale_x"].to(dev), sw1.to(dev).view(-1),
        srt, e_ids, w, post[:1].contiguous(), tokens, SHAPE["inter_dim"], SHAPE["model_dim"], int(e_ids.numel()), None)
    torch.cuda.synchronize()
    close_enough(out[:tokens_topk].view(tokens, SHAPE["topk"], -1), ref, "int8smooth stage 1")
    assert torch.all(out[tokens_topk:] == 7.0)


def test_int8smooth_stage2_is_the_int8_path(dev):
    d = moe_oracle.make_inputs(64, 256, 128, 4, 2, "int8", seed=61)
    a = run_stage2(dev, d, **SHAPE, tile_m=32, in_dtype="int8", out_dtype="bf16", accumulate=False)
    b = run_stage2(dev, d, **SHAPE, tile_m=32, in_dtype="int8smooth", out_dtype="bf16", accumulate=False)
    assert torch.equal(a, b)


@pytest.mark.parametrize("dtype_str", ["f16", "bf16"])
def test_topk_reduction_with_expert_mask(dev, dtype_str):
    """Slot k of token t counts only if expert_mask[topk_ids[t, k]] != 0; masked rows may hold anything (NaN here)."""
    tokens, topk, dim, experts = 50, 3, 256, 6
    g = torch.Generator().manual_seed(8)
    ids, _ = moe_oracle.make_routing(tokens, experts, topk, g)
    mask = torch.tensor([1, 0, 1, 1, 0, 0], dtype=torch.int32)
    x = torch.randn(tokens, topk, dim, generator=g).to(OUT_T[dtype_str])
    keep = mask[ids.long()].bool()
    x_dev = x.clone()
    x_dev[~keep] = float("nan")
    y = torch.full((tokens, dim), 7.0, dtype=OUT_T[dtype_str], device=dev)
    fn = compile_moe_reduction(topk=topk, model_dim=dim, dtype_str=dtype_str, use_mask=True, num_experts=experts)
    fn(x_dev.to(dev), y, mask.to(dev), ids.to(dev), tokens, None)
    torch.cuda.synchronize()
    want = (x.float() * keep.unsqueeze(-1)).sum(dim=1).to(OUT_T[dtype_str])
    assert torch.equal(y.cpu(), want)


# --- W4A8: int8 activations, weights in [-8, 7] passed packed two per byte (in_dtype="int4")


@pytest.mark.parametrize("tile_m,tokens", [(16, 5), (32, 64), (64, 300), (128, 600)])
def test_int4_weights_both_stages(dev, tile_m, tokens):
    """The reference's W4A8 flow (tests/kernels/test_moe_gemm_2stage.py:212-220, 302-325): quantise the
    weights to [-8, 7], preshuffle the int8 values, pack two per byte, launch with in_dtype="int4"."""
    from flydsl_b200.kernels.moe.moe_gemm_2stage import pack_shuffled_int8_to_packed_int4

    d = moe_oracle.make_inputs(tokens, seed=31 + tokens, in_dtype="int4", **SHAPE)
    assert int(d["w1_q"].min()) >= -8 and int(d["w1_q"].max()) <= 7
    experts, topk, model_dim, inter_dim = SHAPE["experts"], SHAPE["topk"], SHAPE["model_dim"], SHAPE["inter_dim"]
    ids, w, e_ids, n_valid, blocks = routing_on(dev, d, experts, tile_m)
    st = torch.cuda.current_stream()
    # stage 1
    w1_packed = pack_shuffled_int8_to_packed_int4(shuffle_weight(d["w1_q"].to(dev)))
    assert w1_packed.numel() == experts * 2 * inter_dim * model_dim // 2
    out1 = torch.full((tokens * topk, inter_dim), 7.0, dtype=torch.bfloat16, device=dev)
    exe1 = compile_moe_gemm1(model_dim=model_dim, inter_dim=inter_dim, experts=experts, topk=topk, tile_m=tile_m, tile_n=64,
                             tile_k=128, doweight_stage1=False, out_dtype="bf16", in_dtype="int4")
    for _ in range(2):  # the second call takes the cached expansion
        exe1(out1, d["x_q"].to(dev).view(-1), w1_packed, d["scale_x"].to(dev).view(-1), d["scale_w1"].to(dev).view(-1), ids, e_ids,
             w.view(-1), n_valid, tokens, inter_dim, model_dim, blocks, st)
    torch.cuda.synchronize()
    close_enough(out1.view(tokens, topk, -1), ref_stage1(d, inter_dim), "int4 stage 1")
    # the packed form and the plain int8 image give bit-identical results
    plain = run_stage1(dev, d, **SHAPE, tile_m=tile_m, in_dtype="int8", out_dtype="bf16")
    assert torch.equal(plain, out1)
    # stage 2
    w2_packed = pack_shuffled_int8_to_packed_int4(shuffle_weight(d["w2_q"].to(dev)))
    out2 = torch.zeros((tokens * topk, model_dim), dtype=torch.bfloat16, device=dev)
    exe2 = compile_moe_gemm2(model_dim=model_dim, inter_dim=inter_dim, experts=experts, topk=topk, tile_m=tile_m, tile_n=64,
                             tile_k=128, doweight_stage2=True, out_dtype="bf16", accumulate=False, in_dtype="int4")
    exe2(out2, d["a2_q"].to(dev).view(-1), w2_packed, d["scale_a2"].to(dev).view(-1), d["scale_w2"].to(dev).view(-1), ids, e_ids,
         w.view(-1), n_valid, tokens, model_dim, inter_dim, blocks, st)
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    close_enough(out2.view(tokens, topk, -1).float().sum(dim=1), ref_stage2(d, model_dim), "int4 stage 2")


def test_int4_nibble_order_matters(dev):
    """Swapping the nibble halves of the packed weights must change the result (the reference guards the
    same property, tests/kernels/test_moe_gemm_2stage.py:411-460): the unpacking order is really used."""
    from flydsl_b200.kernels.moe.moe_gemm_2stage import pack_shuffled_int8_to_packed_int4

    tokens, tile_m = 64, 32
    d = moe_oracle.make_inputs(tokens, seed=5, in_dtype="int4", **SHAPE)
    experts, topk, model_dim, inter_dim = SHAPE["experts"], SHAPE["topk"], SHAPE["model_dim"], SHAPE["inter_dim"]
    ids, w, e_ids, n_valid, blocks = routing_on(dev, d, experts, tile_m)
    good = pack_shuffled_int8_to_packed_int4(shuffle_weight(d["w1_q"].to(dev)))
    u = good.view(torch.uint8)
    swapped = ((u << 4) | (u >> 4)).view(torch.int8).contiguous()
    outs = []
    for packed in (good, swapped):
        out = torch.zeros((tokens * topk, inter_dim), dtype=torch.bfloat16, device=dev)
        exe = compile_moe_gemm1(model_dim=model_dim, inter_dim=inter_dim, experts=experts, topk=topk, tile_m=tile_m, tile_n=64,
                                tile_k=128, doweight_stage1=False, out_dtype="bf16", in_dtype="int4")
        exe(out, d["x_q"].to(dev).view(-1), packed, d["scale_x"].to(dev).view(-1), d["scale_w1"].to(dev).view(-1), ids, e_ids,
            w.view(-1), n_valid, tokens, inter_dim, model_dim, blocks, torch.cuda.current_stream())
        torch.cuda.synchronize()
        outs.append(out.float().cpu())
    ref = ref_stage1(d, inter_dim)
    assert moe_oracle.cosine_sim(outs[0].view(tokens, topk, -1), ref) > 0.99
    assert moe_oracle.cosine_sim(outs[1].view(tokens, topk, -1), ref) < 0.9
