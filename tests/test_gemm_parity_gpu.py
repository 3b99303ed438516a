"""GPU parity: the CUDA path (through the C ABI) against the CPU oracle.

Bars: INT8 int32 accumulators bit-exact; FP8/INT8 bf16 outputs with every
element within rtol 1e-2 / atol 1e-2 of the fp32 dequantise-and-matmul
reference; guard rows past M untouched; CUDA-graph replay == eager.
Shapes follow the reference's test matrix
(tests/kernels/test_preshuffle_gemm.py:119-126,779-883) and the benchmark
configurations.
"""

import os

import pytest
import torch

from flydsl_b200 import _lib, compile_preshuffle_gemm, shuffle_weight, unshuffle_weight
from flydsl_b200 import compiler as flyc
from oracle import a8w8_oracle as oracle
from tests.helpers import as_i8, device_status, gpu_acc, make_workspace

pytestmark = pytest.mark.gpu

RTOL = ATOL = 1e-2  # stated tolerance for fp8 / scaled outputs against the fp32 reference
SENTINEL = -8192.0
DEC, ROWS, ROWS2, W64 = 1 << 8, 2 << 8, 3 << 8, 4 << 8  # variant_hint: kernel field (small-M, large-M, large-M as CTA pairs, small-M with 64-channel tiles)
PAIR = 5 << 8  # variant_hint: kernel field, small-M kernel as CTA pairs
TALL = 6 << 8  # variant_hint: kernel field, large-M kernel with 256-row tiles
WS, CL = 1 << 12, 2 << 12  # variant_hint: split-K reduction through a global workspace / a cluster
PDL = 1 << 28  # variant_hint: programmatic dependent launch
TOK1, TOK2, TOK4 = 1 << 30, 2 << 30, (3 << 30) - (1 << 32)  # variant_hint: token blocks (as signed 32-bit)


def STAGES(n):
    return n << 24


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda:0")


def run_gemm(dev, a_q, b_q, sa, sb, m, n, k, in_dtype, hint=0, tile=(128, 128, 128), use_compile=True):
    fn = compile_preshuffle_gemm(
        N=n, K=k, tile_m=tile[0], tile_n=tile[1], tile_k=tile[2], in_dtype=in_dtype, variant_hint=hint
    )
    rows = ((m + 127) // 128) * 128 + 8
    c_alloc = torch.full((rows, n), SENTINEL, dtype=torch.bfloat16, device=dev)
    b_shuf = shuffle_weight(b_q.to(dev), layout=(16, 16))
    args = (
        c_alloc.view(-1),
        as_i8(a_q.to(dev)).contiguous().view(-1),
        as_i8(b_shuf).contiguous().view(-1),
        sa.to(dev).contiguous().view(-1),
        sb.to(dev).contiguous().view(-1),
        torch.empty(0, dtype=torch.bfloat16, device=dev),
        m,
        n,
        torch.cuda.current_stream(),
    )
    f = flyc.compile(fn, *args) if use_compile else fn
    assert f(*args) is None
    torch.cuda.synchronize()
    assert device_status() == 0
    return c_alloc


def check_scaled(c_alloc, a_q, b_q, sa, sb, m):
    ref = oracle.run_torch(a_q, b_q, sa, sb)
    got = c_alloc[:m].float().cpu()
    bad = oracle.strict_mismatches(got, ref, RTOL, ATOL)
    assert bad == 0, f"{bad} of {got.numel()} elements outside rtol/atol {RTOL}; max abs diff {(got - ref).abs().max()}"
    assert oracle.verify_output(got, ref, rtol=0.1, atol=0.1)  # the reference's own (looser) rule
    n_guard = int((c_alloc[m:] != SENTINEL).sum().item())
    assert n_guard == 0, f"{n_guard} element(s) written past row M={m}"


# --- the reference's small shapes + ragged M, both 8-bit dtypes, both kernels


@pytest.mark.parametrize("in_dtype", ["fp8", "int8"])
@pytest.mark.parametrize(
    "m,n,k,tile",
    [
        (16, 5120, 8192, (16, 64, 512)),
        (33, 1024, 2048, (32, 64, 512)),
        (1, 8192, 8192, (16, 64, 256)),
        (128, 4096, 4096, (128, 128, 128)),  # benchmark config 1
        (257, 1024, 1152, (128, 128, 128)),  # just past the small-M kernel; K = 9 * 128
        (513, 2064, 2048, (64, 256, 128)),  # N not a multiple of the tile
    ],
)
def test_scaled_output_matches_reference_check(dev, in_dtype, m, n, k, tile):
    a_q, b_q, sa, sb = oracle.make_inputs(m, n, k, in_dtype, seed=1000 + m)
    c = run_gemm(dev, a_q, b_q, sa, sb, m, n, k, in_dtype, tile=tile)
    check_scaled(c, a_q, b_q, sa, sb, m)


@pytest.mark.parametrize(
    "hint",
    [DEC | 1, DEC | CL | 2, DEC | CL | 5, DEC | CL | 8, DEC | WS | 3, DEC | WS | 16, DEC | 2 | STAGES(3), DEC | 2 | PDL,
     DEC | 2 | (2 << 28), W64, W64 | STAGES(3), DEC | TOK1 | 2, DEC | TOK2, DEC | TOK4, DEC | TOK2 | CL | 2, DEC | TOK4 | WS | 3, ROWS, ROWS2, TALL],
    ids=["nosplit", "cluster2", "cluster5", "cluster8", "ws3", "ws16", "stages3", "pdl", "nopdl", "w64", "w64_stages3", "tok1", "tok2", "tok4",
         "tok2_cluster2", "tok4_ws3", "rows", "rows2", "tall"],
)
@pytest.mark.parametrize("m", [1, 16, 17, 64, 100, 256])
def test_every_kernel_variant_small_m(dev, hint, m):
    if (hint & 0xF00) == W64 and m > 64:
        pytest.skip("64-channel tiles are built for up to 64 tokens")
    n, k = 1040, 2048
    a_q, b_q, sa, sb = oracle.make_inputs(m, n, k, "fp8", seed=77 + m)
    c = run_gemm(dev, a_q, b_q, sa, sb, m, n, k, "fp8", hint=hint)
    check_scaled(c, a_q, b_q, sa, sb, m)


@pytest.mark.parametrize(
    "hint",
    [PAIR | 1, PAIR | CL | 2, PAIR | CL | 3, PAIR | CL | 4, PAIR | 2 | STAGES(4), PAIR | 2 | PDL, PAIR | 2 | (2 << 28),
     PAIR | TOK2, PAIR | TOK4 | CL | 2, PAIR],
    ids=["nosplit", "cluster2", "cluster3", "cluster4", "stages4", "pdl", "nopdl", "tok2", "tok4_cluster2", "auto_split"],
)
@pytest.mark.parametrize("m", [33, 64, 100, 128, 129, 200, 256])
def test_small_m_kernel_as_cta_pairs(dev, hint, m):
    """Two CTAs on neighbouring channel tiles share the token tile (half each); N = 1936 gives 16
    channel tiles, the last one 16 channels wide."""
    n, k = 1936, 2048
    blocks = {1: 1, 2: 2, 3: 4}.get((hint >> 30) & 3, 1)
    if -(-m // blocks) <= 32:
        pytest.skip("pairs are built for token tiles of 64 and more")
    a_q, b_q, sa, sb = oracle.make_inputs(m, n, k, "fp8", seed=99 + m)
    fn = compile_preshuffle_gemm(N=n, K=k, tile_m=128, tile_n=128, tile_k=128, in_dtype="fp8", variant_hint=hint)
    assert fn.plan(m)["kernel"] == 5
    c = run_gemm(dev, a_q, b_q, sa, sb, m, n, k, "fp8", hint=hint)
    check_scaled(c, a_q, b_q, sa, sb, m)


@pytest.mark.parametrize("in_dtype", ["fp8", "int8"])
@pytest.mark.parametrize("m,n,k", [(257, 1024, 1152), (513, 2064, 2048), (2048, 4096, 4096)])
def test_cta_pair_kernel_scaled_output(dev, in_dtype, m, n, k):
    a_q, b_q, sa, sb = oracle.make_inputs(m, n, k, in_dtype, seed=31 + m)
    c = run_gemm(dev, a_q, b_q, sa, sb, m, n, k, in_dtype, hint=ROWS2)
    check_scaled(c, a_q, b_q, sa, sb, m)


@pytest.mark.parametrize("in_dtype", ["fp8", "int8", "bf16"])
@pytest.mark.parametrize("m,n,k", [(300, 2048, 4096), (512, 1024, 8192), (1024, 2048, 4096), (777, 1040, 4096)])
def test_narrow_output_mid_m_runs_on_the_small_m_kernel(dev, in_dtype, m, n, k):
    """257..1024 tokens, few channel tiles, long K: token blocks of 256 on the small-M kernel (automatic)."""
    fn = compile_preshuffle_gemm(N=n, K=k, tile_m=128, tile_n=128, tile_k=128, in_dtype=in_dtype)
    assert fn.plan(m)["kernel"] in (1, 5) and fn.plan(m)["token_blocks"] == -(-m // 256)  # 5: pairs, if the environment asks
    if in_dtype == "bf16":
        g = torch.Generator().manual_seed(m)
        a = (torch.randn(m, k, generator=g) * 0.5).to(torch.bfloat16)
        b = (torch.randn(n, k, generator=g) * 0.5).to(torch.bfloat16)
        got = run_gemm_generic(dev, a, b, None, None, None, m, n, k, in_dtype)
        assert oracle.strict_mismatches(got, oracle.run_torch(a, b, None, None), RTOL, ATOL) == 0
        return
    a_q, b_q, sa, sb = oracle.make_inputs(m, n, k, in_dtype, seed=41 + m)
    c = run_gemm(dev, a_q, b_q, sa, sb, m, n, k, in_dtype)
    check_scaled(c, a_q, b_q, sa, sb, m)


@pytest.mark.parametrize("in_dtype", ["fp8", "int8"])
@pytest.mark.parametrize("m,n,k", [(257, 1024, 1152), (513, 2064, 2048), (2048, 4096, 4096), (130, 528, 256)])
def test_tall_tile_kernel_scaled_output(dev, in_dtype, m, n, k):
    """256-row tiles: two accumulators per CTA share every weight block."""
    a_q, b_q, sa, sb = oracle.make_inputs(m, n, k, in_dtype, seed=37 + m)
    fn = compile_preshuffle_gemm(N=n, K=k, tile_m=128, tile_n=128, tile_k=128, in_dtype=in_dtype, variant_hint=TALL)
    assert fn.plan(m)["kernel"] == 6
    c = run_gemm(dev, a_q, b_q, sa, sb, m, n, k, in_dtype, hint=TALL)
    check_scaled(c, a_q, b_q, sa, sb, m)


def test_first_captured_call_allocates_nothing_when_compiled(dev):
    """A launcher asked to reduce its K splits through a global workspace.  flyc.compile allocates
    that workspace for the stream it is given, so the launcher's very first call may be a captured
    one; without compile a first call inside a capture is refused with a clear message instead of
    allocating behind the capture."""
    m, n, k = 16, 1024, 8192
    a_q, b_q, sa, sb = oracle.make_inputs(m, n, k, "fp8", seed=77)
    s = torch.cuda.Stream()
    hint = DEC | WS | 16
    fn = compile_preshuffle_gemm(N=n, K=k, tile_m=16, tile_n=64, tile_k=256, in_dtype="fp8", variant_hint=hint)
    assert fn.plan(m)["reduce"] == 1 and fn.workspace_bytes(dev) > 16384  # the workspace path
    c = torch.zeros(m, n, dtype=torch.bfloat16, device=dev)
    args = (c.view(-1), as_i8(a_q.to(dev)).view(-1), as_i8(shuffle_weight(b_q.to(dev))).view(-1), sa.to(dev), sb.to(dev),
            torch.empty(0, dtype=torch.bfloat16, device=dev), m, n, s)
    torch.cuda.synchronize()
    # (1) not compiled, first call under capture: refused
    g0 = torch.cuda.CUDAGraph()
    with pytest.raises(RuntimeError, match="before capturing"):
        with torch.cuda.graph(g0, stream=s):
            fn(*args)
    torch.cuda.synchronize()
    # (2) compiled on the capture stream: the first call is the captured one and allocates nothing
    fn2 = compile_preshuffle_gemm(N=n, K=k, tile_m=16, tile_n=64, tile_k=256, in_dtype="fp8", variant_hint=hint)
    cf = flyc.compile(fn2, *args)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated(dev)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        cf(*args)
    assert torch.cuda.memory_allocated(dev) == before
    c.zero_()
    g.replay()
    torch.cuda.synchronize()
    assert device_status() == 0
    ref = oracle.run_torch(a_q, b_q, sa, sb)
    assert oracle.strict_mismatches(c.float().cpu(), ref, RTOL, ATOL) == 0


# --- INT8: accumulators bit-exact before scaling


@pytest.mark.parametrize(
    "m,n,k,hint",
    [
        (32, 8192, 8192, 0),  # benchmark config 2, automatic variant
        (32, 8192, 8192, DEC | 1),
        (32, 8192, 8192, W64),
        (7, 144, 1024, W64),
        (16, 256, 128, DEC | 1),  # a single k-block: only one of the two MMA issuers has work
        (16, 256, 384, DEC | 1),  # three k-blocks: uneven share between the issuers
        (16, 256, 384, DEC | CL | 3),  # one k-block per split
        (40, 272, 640, W64),
        (64, 1040, 2048, W64),
        (32, 8192, 8192, DEC | CL | 4),
        (32, 8192, 8192, DEC | WS | 4),
        (7, 144, 1024, DEC | WS | 3),
        (7, 144, 1024, DEC | CL | 3),
        (200, 512, 1024, DEC | CL | 2),
        (200, 512, 1024, DEC | WS | 2),
        (200, 512, 1024, DEC | TOK4 | WS | 2),
        (33, 1040, 1024, DEC | TOK2 | CL | 4),
        (64, 256, 128, PAIR | 1),  # CTA pairs, a single k-block
        (64, 256, 384, PAIR | CL | 3),  # one k-block per split
        (130, 1936, 640, PAIR | CL | 4),
        (200, 512, 1024, PAIR | CL | 2),
        (256, 2048, 4096, PAIR),
        (512, 1024, 2048, DEC),  # more than 256 tokens: token blocks of 256 (grid.z), K split over a cluster
        (700, 2048, 1024, DEC | CL | 2),  # three token blocks, the last one part empty
        (1000, 512, 4096, DEC),
        (300, 2048, 4096, 0),  # the automatic choice for a narrow output: small-M kernel, two token blocks
        (8, 57344, 256, 0),  # very wide: more channel tiles than SMs
        (300, 784, 1024, ROWS),
        (1024, 2048, 8320, ROWS),  # K = 65 * 128 as in the reference's large shapes
        (300, 784, 1024, ROWS2),
        (100, 272, 256, ROWS2),
        (1024, 2048, 8320, ROWS2),
        (300, 784, 1024, TALL),
        (100, 272, 256, TALL),
        (1024, 2048, 8320, TALL),
        (700, 1040, 640, TALL | 5),  # 160-channel tiles: a 32-column tail in every tile
        (2049, 512, 384, TALL | (3 << 16)),  # nine row tiles in groups of three
    ],
)
def test_int8_accumulators_bit_exact(dev, m, n, k, hint):
    a_q, b_q, _, _ = oracle.make_inputs(m, n, k, "int8", seed=5 + m + n, rne_int8=True)
    ws = make_workspace(m, n, k, "int8", dev, variant_hint=hint)
    acc = gpu_acc(a_q.to(dev), shuffle_weight(b_q.to(dev)), m, n, k, "int8", variant_hint=hint, workspace=ws)
    torch.cuda.synchronize()
    assert device_status() == 0
    want = oracle.int32_acc(a_q, b_q)
    assert torch.equal(acc.cpu(), want)
    if ws.numel() > 16384:
        assert int(ws[:16384].any().item()) == 0, "split-K tickets must be left at zero"


def test_int8_extreme_values_exact(dev):
    """All-(-128) x all-(-128) and mixed signs: the largest accumulators int32 can be asked to hold here."""
    m, n, k = 16, 256, 8192
    a = torch.full((m, k), -128, dtype=torch.int8)
    b = torch.full((n, k), -128, dtype=torch.int8)
    b[1::2] = 127
    acc = gpu_acc(a.to(dev), shuffle_weight(b.to(dev)), m, n, k, "int8", variant_hint=DEC | 1)
    assert torch.equal(acc.cpu(), oracle.int32_acc(a, b))


def test_fp8_accumulators_close_to_fp32(dev):
    m, n, k = 64, 512, 8192
    a_q, b_q, _, _ = oracle.make_inputs(m, n, k, "fp8", seed=9)
    acc = gpu_acc(a_q.to(dev), shuffle_weight(b_q.to(dev)), m, n, k, "fp8").view(torch.float32).cpu()
    ref = a_q.float() @ b_q.float().T
    assert torch.allclose(acc, ref, rtol=1e-4, atol=ref.abs().max().item() * 1e-6)


# --- weight preshuffle on the GPU against its CPU statement


@pytest.mark.parametrize("dtype", [torch.int8, torch.float8_e4m3fn, torch.bfloat16])
@pytest.mark.parametrize("shape", [(16, 128), (1024, 2048), (2, 48, 384), (5120, 8320)])
def test_shuffle_weight_kernel(dev, dtype, shape):
    g = torch.Generator().manual_seed(11)
    x = torch.randint(-120, 120, shape, generator=g).to(torch.float32).to(dtype)
    img = shuffle_weight(x.to(dev))
    assert getattr(img, "is_shuffled", False) and img.shape == x.shape and img.dtype == x.dtype
    want = oracle.shuffle_weight_b200(x)
    assert torch.equal(img.cpu().view(torch.uint8), want.view(torch.uint8))
    assert torch.equal(unshuffle_weight(img).cpu().view(torch.uint8), x.view(torch.uint8))
    from_ref = shuffle_weight(oracle.shuffle_weight_mfma(x).to(dev), src_layout="mfma")
    assert torch.equal(from_ref.cpu().view(torch.uint8), want.view(torch.uint8))


# --- call conventions


def test_cudagraph_capture_and_stream_forms(dev):
    """Launch on the current stream is captured; replay == eager
    (tests/kernels/test_preshuffle_gemm.py:779-883).  Also raw-int and None streams."""
    m, n, k = 1, 8192, 8192
    a_q, b_q, sa, sb = oracle.make_inputs(m, n, k, "fp8", seed=42)
    fn = compile_preshuffle_gemm(N=n, K=k, tile_m=16, tile_n=64, tile_k=256, in_dtype="fp8")
    a, b = as_i8(a_q.to(dev)).view(-1), as_i8(shuffle_weight(b_q.to(dev))).view(-1)
    sa_d, sb_d = sa.to(dev), sb.to(dev)
    bias = torch.empty(0, dtype=torch.bfloat16, device=dev)
    c = torch.zeros(m, n, dtype=torch.bfloat16, device=dev)

    def call(stream):
        fn(c.view(-1), a, b, sa_d, sb_d, bias, m, n, stream)

    call(torch.cuda.current_stream())
    torch.cuda.synchronize()
    ref = c.clone()
    assert ref.abs().max().item() > 0
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        call(torch.cuda.current_stream())  # warm-up on the capture stream
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    c.zero_()
    with torch.cuda.graph(g, stream=s):
        call(torch.cuda.current_stream())
    torch.cuda.synchronize()
    c.zero_()
    g.replay()
    torch.cuda.synchronize()
    assert c.abs().max().item() > 0, "graph replay produced zeros: the launch was not captured"
    assert torch.allclose(ref, c, atol=1e-2)
    assert torch.equal(ref, c)  # deterministic reduction order: bitwise equal
    for stream in (None, 0, torch.cuda.current_stream().cuda_stream):
        c.zero_()
        call(stream)
        torch.cuda.synchronize()
        assert torch.equal(ref, c)
    assert device_status() == 0


def test_results_are_deterministic_and_row_independent(dev):
    """Size-independent properties at a benchmark-sized decode shape: repeated
    launches are bitwise equal, permuting tokens permutes output rows bitwise,
    doubling a token scale doubles its row exactly."""
    m, n, k = 32, 8192, 8192
    a_q, b_q, sa, sb = oracle.make_inputs(m, n, k, "fp8", seed=4)
    c1 = run_gemm(dev, a_q, b_q, sa, sb, m, n, k, "fp8")[:m].clone()
    c2 = run_gemm(dev, a_q, b_q, sa, sb, m, n, k, "fp8")[:m]
    assert torch.equal(c1, c2)
    perm = torch.randperm(m, generator=torch.Generator().manual_seed(0))
    cp = run_gemm(dev, a_q[perm], b_q, sa[perm], sb, m, n, k, "fp8")[:m]
    assert torch.equal(cp, c1[perm.to(dev)])
    cd = run_gemm(dev, a_q, b_q, sa * 2, sb, m, n, k, "fp8")[:m]
    assert torch.equal(cd.float(), c1.float() * 2)


def test_m_zero_and_tensor_checks(dev):
    fn = compile_preshuffle_gemm(N=64, K=256, tile_m=16, tile_n=64, tile_k=256, in_dtype="int8")
    c = torch.full((16, 64), SENTINEL, dtype=torch.bfloat16, device=dev)
    a = torch.zeros(16 * 256, dtype=torch.int8, device=dev)
    b = torch.zeros(64 * 256, dtype=torch.int8, device=dev)
    sa, sb = torch.ones(16, device=dev), torch.ones(64, device=dev)
    bias = torch.empty(0, dtype=torch.bfloat16, device=dev)
    assert fn(c.view(-1), a, b, sa, sb, bias, 0, 64, None) is None  # M = 0: nothing to do
    torch.cuda.synchronize()
    assert bool((c == SENTINEL).all())
    with pytest.raises(ValueError, match="buffer sizes"):
        fn(c.view(-1), a[:100], b, sa, sb, bias, 16, 64, None)
    with pytest.raises(ValueError, match="scale"):
        fn(c.view(-1), a, b, sa[:4], sb, bias, 16, 64, None)
    with pytest.raises(ValueError, match="c must be"):
        fn(c.float().view(-1), a, b, sa, sb, bias, 16, 64, None)
    fn(c.view(-1), a, b, torch.nn.Parameter(sa, requires_grad=False), sb, bias, 16, 64, None)  # Parameter accepted
    torch.cuda.synchronize()
    assert bool((c == 0).all())


# --- fp16 / bf16 inputs (no scales) and the fused bias / activation epilogues
#     (tests/kernels/test_preshuffle_gemm.py:116 dtype list, :889-980 epilogue test)

TORCH_DT = {"fp16": torch.float16, "bf16": torch.bfloat16}


def run_gemm_generic(dev, a, b, sa, sb, bias, m, n, k, in_dtype, out_dtype="bf16", epilogue="none", hint=0):
    fn = compile_preshuffle_gemm(
        N=n, K=k, tile_m=16, tile_n=64, tile_k=256, in_dtype=in_dtype, out_dtype=out_dtype, epilogue=epilogue,
        variant_hint=hint,
    )  # fmt: skip
    odt = TORCH_DT[out_dtype]
    c_alloc = torch.full((m + 8, n), SENTINEL, dtype=odt, device=dev)
    empty_f32 = torch.empty(0, dtype=torch.float32, device=dev)
    args = (
        c_alloc.view(-1),
        as_i8(a.to(dev)).contiguous().view(-1),
        as_i8(shuffle_weight(b.to(dev))).contiguous().view(-1),
        sa.to(dev) if sa is not None else empty_f32,
        sb.to(dev) if sb is not None else empty_f32,
        bias.to(dev) if bias is not None else torch.empty(0, dtype=odt, device=dev),
        m,
        n,
        torch.cuda.current_stream(),
    )
    flyc.compile(fn, *args)(*args)
    torch.cuda.synchronize()
    assert device_status() == 0
    assert int((c_alloc[m:] != SENTINEL).sum().item()) == 0
    return c_alloc[:m].float().cpu()


@pytest.mark.parametrize("in_dtype", ["fp16", "bf16"])
@pytest.mark.parametrize("m,n,k,hint", [(16, 5120, 8192, 0), (33, 1024, 2048, 0), (513, 1024, 2048, 0), (513, 1024, 2048, ROWS2), (513, 1024, 2048, TALL), (200, 528, 1280, DEC | WS | 3),
                                        (200, 512, 1280, PAIR | CL | 2), (72, 1024, 2048, PAIR)])
def test_half_precision_inputs(dev, in_dtype, m, n, k, hint):
    g = torch.Generator().manual_seed(m + n)
    a = torch.randn(m, k, generator=g).to(TORCH_DT[in_dtype])
    b = torch.randn(n, k, generator=g).to(TORCH_DT[in_dtype])
    got = run_gemm_generic(dev, a, b, None, None, None, m, n, k, in_dtype, hint=hint)
    ref = oracle.run_torch(a, b, None, None)
    assert oracle.strict_mismatches(got, ref, RTOL, ATOL) == 0


@pytest.mark.parametrize("epilogue", ["bias", "bias_relu", "bias_silu", "bias_gelu"])
@pytest.mark.parametrize("in_dtype,m", [("bf16", 16), ("fp8", 16), ("fp8", 300), ("int8", 40), ("bf16", 136), ("fp8", 250)])
def test_fused_epilogues(dev, epilogue, in_dtype, m):
    n, k = 5120, 2048
    g = torch.Generator().manual_seed(7)
    bias = torch.randn(n, generator=g).to(torch.bfloat16)
    if in_dtype == "bf16":
        a = torch.randn(m, k, generator=g).to(torch.bfloat16)
        b = torch.randn(n, k, generator=g).to(torch.bfloat16)
        sa = sb = None
        acc = a.float() @ b.float().T
    else:
        a, b, sa, sb = oracle.make_inputs(m, n, k, in_dtype, seed=70 + m)
        acc = a.float() @ b.float().T
    got = run_gemm_generic(dev, a, b, sa, sb, bias, m, n, k, in_dtype, epilogue=epilogue)
    ref = oracle.epilogue(acc, sa, sb, bias, epilogue, out_dtype=torch.float32)
    assert not torch.isnan(got).any() and not torch.isinf(got).any()
    assert oracle.strict_mismatches(got, ref, RTOL, ATOL) == 0
    # the reference's own looser bar (tests/kernels/test_preshuffle_gemm.py:967-973)
    assert torch.allclose(got, ref.to(torch.bfloat16).float(), atol=2.0, rtol=0.05)


@pytest.mark.parametrize("in_dtype,m", [("fp8", 24), ("int8", 400), ("fp16", 24)])
def test_fp16_output(dev, in_dtype, m):
    n, k = 1024, 1024
    if in_dtype == "fp16":
        g = torch.Generator().manual_seed(3)
        a = (torch.randn(m, k, generator=g) * 0.25).to(torch.float16)
        b = (torch.randn(n, k, generator=g) * 0.25).to(torch.float16)
        sa = sb = None
    else:
        a, b, sa, sb = oracle.make_inputs(m, n, k, in_dtype, seed=m)
    got = run_gemm_generic(dev, a, b, sa, sb, None, m, n, k, in_dtype, out_dtype="fp16")
    ref = oracle.run_torch(a, b, sa, sb)
    assert oracle.strict_mismatches(got, ref, RTOL, ATOL) == 0


# --- large-M kernel: every tile width (the split field of the hint, in units of 32 channels)


@pytest.mark.parametrize("width", [1, 2, 3, 4, 5, 6, 7, 8])
@pytest.mark.parametrize("m,n,k", [(300, 1040, 2048), (129, 2064, 1152)])
def test_large_m_kernel_every_tile_width(dev, width, m, n, k):
    """128 x (32 * width) tiles: N is no multiple of any width, so the last tile of every row is
    clipped, and widths that are not a multiple of 64 end in the 32-column tail of the epilogue."""
    a_q, b_q, sa, sb = oracle.make_inputs(m, n, k, "fp8", seed=500 + width + m)
    c = run_gemm(dev, a_q, b_q, sa, sb, m, n, k, "fp8", hint=ROWS | width)
    check_scaled(c, a_q, b_q, sa, sb, m)
    a_i, b_i, _, _ = oracle.make_inputs(m, n, k, "int8", seed=600 + width, rne_int8=True)
    acc = gpu_acc(a_i.to(dev), shuffle_weight(b_i.to(dev)), m, n, k, "int8", variant_hint=ROWS | width)
    torch.cuda.synchronize()
    assert device_status() == 0
    assert torch.equal(acc.cpu(), oracle.int32_acc(a_i, b_i))


@pytest.mark.parametrize("width", [3, 7, TALL | 3, TALL | 8])
@pytest.mark.parametrize("in_dtype", ["fp8", "bf16"])
def test_large_m_kernel_tile_tail_with_fused_epilogue(dev, width, in_dtype):
    m, n, k = 200, 1040, 1024
    g = torch.Generator().manual_seed(width)
    bias = torch.randn(n, generator=g).to(torch.bfloat16)
    if in_dtype == "bf16":
        a = torch.randn(m, k, generator=g).to(torch.bfloat16)
        b = torch.randn(n, k, generator=g).to(torch.bfloat16)
        sa = sb = None
    else:
        a, b, sa, sb = oracle.make_inputs(m, n, k, in_dtype, seed=width)
    got = run_gemm_generic(dev, a, b, sa, sb, bias, m, n, k, in_dtype, epilogue="bias_silu",
                           hint=width if width > 8 else ROWS | width)  # a bare width: the one-CTA 128-row form
    ref = oracle.epilogue(a.float() @ b.float().T, sa, sb, bias, "bias_silu", out_dtype=torch.float32)
    assert oracle.strict_mismatches(got, ref, RTOL, ATOL) == 0


def test_automatic_tile_width_fills_whole_rounds():
    """The planner picks the width whose tiles cover the 148 SMs in full rounds: 2048 x 8192 gives
    16 x 37 = 592 tiles of 224 channels (four rounds) instead of 512 tiles of 256 (3.46 rounds); and
    where 256-row tiles cover the output in one nearly full round (1024 x 8192: 128 tiles) it takes those."""
    if os.environ.get("FLYB200_ROWS_TALL") == "1" or os.environ.get("FLYB200_ROWS_2SM") == "1":
        pytest.skip("the environment overrides the automatic choice")
    plan = _lib.describe_plan(2048, 8192, 8192, "fp8", 0, 148)
    assert plan["kernel"] == 2 and plan["bn"] == 224
    plan = _lib.describe_plan(1024, 8192, 8192, "fp8", 2 << 8, 148)  # the 128-row form on request
    assert plan["kernel"] == 2 and plan["bn"] == 224
    plan = _lib.describe_plan(1024, 8192, 8192, "fp8", 0, 148)
    assert plan["kernel"] == 6 and plan["bn"] == 256
    assert _lib.describe_plan(16384, 57344, 8192, "fp8", 0, 148)["bn"] == 256


def test_reference_example_fp16_4096_cubed():
    """The reference's own example (examples/04-preshuffle_gemm.py): fp16 4096^3 with its tolerance."""
    from flydsl_b200.examples.preshuffle_gemm import run

    ok, violation, _ = run(4096, 4096, 4096)
    assert ok, f"max violation of 1e-3 + 1e-3*|expected|: {violation}"
    assert device_status() == 0


# --- failure path: a bounded device-side wait that cannot succeed


def test_bounded_wait_expires_and_reports(dev):
    """A wait on a barrier that nothing completes gives up after its limit, the
    kernel returns normally with FLYB200_E_TIMEOUT in the status word, and the
    device keeps working (no trap, no hang)."""
    import time

    lib = _lib.load()
    assert device_status() == 0
    t0 = time.perf_counter()
    _lib.check(lib.flyb200_selftest_bounded_wait(20000, torch.cuda.current_stream().cuda_stream), "selftest")  # 20 ms
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    assert 0.015 < elapsed < 2.0, elapsed
    assert device_status() == _lib.E_TIMEOUT
    assert device_status() == 0  # reading clears the word
    assert lib.flyb200_selftest_bounded_wait(0, None) == _lib.E_BAD_ARG
    assert lib.flyb200_selftest_bounded_wait(10**6, None) == _lib.E_BAD_ARG
    # the context is still good: a GEMM right after gives exact results
    a_q, b_q, _, _ = oracle.make_inputs(16, 256, 512, "int8", seed=1)
    acc = gpu_acc(a_q.to(dev), shuffle_weight(b_q.to(dev)), 16, 256, 512, "int8")
    assert torch.equal(acc.cpu(), oracle.int32_acc(a_q, b_q))
    assert device_status() == 0


@pytest.mark.parametrize("in_dtype", ["bf16", "int8"])
def test_cudagraph_capture_other_dtypes(dev, in_dtype):
    """Graph capture for the 16-bit path (the reference captures bf16 and fp8) and for INT8."""
    m, n, k = 1, 8192, 8192
    g = torch.Generator().manual_seed(5)
    if in_dtype == "bf16":
        a = torch.randn(m, k, generator=g).to(torch.bfloat16).to(dev)
        b = shuffle_weight(torch.randn(n, k, generator=g).to(torch.bfloat16).to(dev))
        sa = sb = torch.empty(0, dtype=torch.float32, device=dev)
    else:
        a_q, b_q, sa, sb = oracle.make_inputs(m, n, k, "int8", seed=6)
        a, b, sa, sb = a_q.to(dev), shuffle_weight(b_q.to(dev)), sa.to(dev), sb.to(dev)
    fn = compile_preshuffle_gemm(N=n, K=k, tile_m=16, tile_n=64, tile_k=256, in_dtype=in_dtype)
    bias = torch.empty(0, dtype=torch.bfloat16, device=dev)
    c = torch.zeros(m, n, dtype=torch.bfloat16, device=dev)
    args = lambda: (c.view(-1), a.view(-1), b.view(-1), sa, sb, bias, m, n, torch.cuda.current_stream())  # noqa: E731
    cf = flyc.compile(fn, *args())
    cf(*args())
    torch.cuda.synchronize()
    ref = c.clone()
    assert ref.abs().max().item() > 0
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        cf(*args())
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=s):
        cf(*args())
        cf(*args())  # back to back inside one graph: the dependent-launch edge is captured too
    c.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(ref, c)
    assert device_status() == 0
