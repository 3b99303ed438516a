"""The reference's example ``examples/04-preshuffle_gemm.py`` on B200.

    python -m flydsl_b200.examples.preshuffle_gemm [--m 4096 --n 4096 --k 4096]

There the example writes an fp16 GEMM with preshuffled weights in the DSL
(C[M, N] = A[M, K] . B[N, K]^T, M = N = K = 4096, fp16 in and out, fp32
accumulation) and checks it against ``A @ B.T`` with the tolerance
``1e-3 + 1e-3 * |expected|`` (examples/04-preshuffle_gemm.py:187-205).  Here the
same problem, inputs, preshuffle call and check run through the prebuilt
operator: ``shuffle_weight(B, layout=(16, 16))`` produces the B200 weight image
and ``compile_preshuffle_gemm(..., in_dtype="fp16", out_dtype="fp16")`` the
launcher (tcgen05 ``kind::f16``, no scales).
"""

from __future__ import annotations

import argparse

import torch

from flydsl_b200 import compile_preshuffle_gemm, shuffle_weight
from flydsl_b200 import compiler as flyc


def run(m: int = 4096, n: int = 4096, k: int = 4096, seed: int = 0, device: str = "cuda:0"):
    """Returns (is_correct, max_violation, microseconds per launch)."""
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed)
    a = torch.randn(m, k, dtype=torch.float16, device=dev, generator=g)
    b = torch.randn(n, k, dtype=torch.float16, device=dev, generator=g)
    c = torch.zeros(m, n, dtype=torch.float16, device=dev)
    preshuffle_b = shuffle_weight(b, layout=(16, 16))
    launch = compile_preshuffle_gemm(N=n, K=k, tile_m=128, tile_n=128, tile_k=64, in_dtype="fp16", out_dtype="fp16")
    empty = torch.empty(0, dtype=torch.float32, device=dev)  # no scales for 16-bit inputs
    bias = torch.empty(0, dtype=torch.float16, device=dev)
    stream = torch.cuda.current_stream(dev)
    args = (c.view(-1), a.view(-1), preshuffle_b.view(-1), empty, empty, bias, m, n, stream)
    fn = flyc.compile(launch, *args)
    fn(*args)
    torch.cuda.synchronize(dev)
    expected = a.float() @ b.float().T  # fp32 product (the reference's example lets torch multiply in fp16)
    actual = c.to(torch.float32)
    tol = 1e-3 + 1e-3 * expected.abs()
    max_violation = ((actual - expected).abs() - tol).max().item()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(10):
        fn(*args)
    e1.record(stream)
    torch.cuda.synchronize(dev)
    return max_violation <= 0, max_violation, e0.elapsed_time(e1) * 100.0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    a = ap.parse_args()
    ok, violation, us = run(a.m, a.n, a.k)
    print("Result correct:", ok)
    if not ok:
        print("Max violation:", violation)
    print(f"{us:.1f} us per launch, {2.0 * a.m * a.n * a.k / us / 1e6:.0f} TFLOP/s")


if __name__ == "__main__":
    main()
