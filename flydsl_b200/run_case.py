"""Run one GEMM configuration a few times and print its device time.

    python -m flydsl_b200.run_case --m 32 --n 8192 --k 8192 --dtype int8 [--iters 5] [--hint 0]

A small, self-contained driver for profilers (one kernel per iteration, random
operands generated on the GPU, no host reference).
"""

from __future__ import annotations

import argparse
import json

import torch

from . import _lib, compile_preshuffle_gemm, shuffle_weight


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, required=True)
    ap.add_argument("--n", type=int, required=True)
    ap.add_argument("--k", type=int, required=True)
    ap.add_argument("--dtype", default="fp8", choices=["fp8", "int8"])
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--hint", type=lambda s: int(s, 0), default=0)
    ap.add_argument("--op", default="gemm", choices=["gemm", "quant", "shuffle"],
                    help="gemm (default), quant: per-token quantiser on [m, k] bf16, shuffle: weight preshuffle of [n, k]")
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    if a.op != "gemm":
        from .utils import pertoken_quant_kernel

        if a.op == "quant":
            x = torch.randn(a.m, a.k, device=dev, dtype=torch.bfloat16)
            qd = torch.float8_e4m3fn if a.dtype == "fp8" else torch.int8
            fn, byts = (lambda: pertoken_quant_kernel(x, qd)), a.m * a.k * 3 + a.m * 4
        else:
            w8 = torch.randint(-127, 128, (a.n, a.k), device=dev, dtype=torch.int8)
            fn, byts = (lambda: shuffle_weight(w8)), 2 * a.n * a.k
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / a.iters
        print(json.dumps({"op": a.op, "M": a.m, "N": a.n, "K": a.k, "us": round(us, 2), "gbs": round(byts / us / 1e3, 1)}))
        return
    if a.dtype == "fp8":
        x = (torch.randn(a.m, a.k, device=dev) * 64).clamp_(-448, 448).to(torch.float8_e4m3fn).view(torch.int8)
        w = (torch.randn(a.n, a.k, device=dev) * 64).clamp_(-448, 448).to(torch.float8_e4m3fn)
    else:
        x = torch.randint(-127, 128, (a.m, a.k), device=dev, dtype=torch.int8)
        w = torch.randint(-127, 128, (a.n, a.k), device=dev, dtype=torch.int8)
    w = shuffle_weight(w).view(torch.int8)
    sa = torch.rand(a.m, device=dev) + 0.5
    sb = torch.rand(a.n, device=dev) + 0.5
    c = torch.empty(a.m, a.n, dtype=torch.bfloat16, device=dev)
    bias = torch.empty(0, dtype=torch.bfloat16, device=dev)
    fn = compile_preshuffle_gemm(N=a.n, K=a.k, tile_m=128, tile_n=256, tile_k=128, in_dtype=a.dtype, variant_hint=a.hint)
    st = torch.cuda.current_stream()
    fn(c.view(-1), x.view(-1), w.view(-1), sa, sb, bias, a.m, a.n, st)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.iters):
        fn(c.view(-1), x.view(-1), w.view(-1), sa, sb, bias, a.m, a.n, st)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / a.iters
    flops = 2.0 * a.m * a.n * a.k
    byts = a.m * a.k + a.n * a.k + 2 * a.m * a.n + 4 * (a.m + a.n)
    print(json.dumps({"M": a.m, "N": a.n, "K": a.k, "dtype": a.dtype, "us": round(us, 2),
                      "tflops": round(flops / us / 1e6, 1), "gbs": round(byts / us / 1e3, 1),
                      "status": _lib.read_status()}))


if __name__ == "__main__":
    main()
