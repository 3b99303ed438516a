"""Run one GEMM configuration a few times and print its device time.

    python bench_case.py --m 32 --n 8192 --k 8192 --dtype int8 [--iters 5] [--hint 0]
    python bench_case.py --op moe1 --m 4096 --n 2048 --k 4096 --experts 8 --topk 2 --tile-m 128

A small, self-contained driver for profilers (one kernel per iteration, random
operands generated on the GPU, no host reference).
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from flydsl_b200 import _lib, compile_preshuffle_gemm, shuffle_weight  # noqa: E402


def run_moe(a, dev):
    from flydsl_b200.kernels.moe.moe_gemm_2stage import compile_moe_gemm1, compile_moe_gemm2, moe_sorting

    tokens, inter, model, e, topk = a.m, a.n, a.k, a.experts, a.topk
    qd = torch.float8_e4m3fn if a.dtype == "fp8" else torch.int8

    def q8(*shape):
        if a.dtype == "fp8":
            return (torch.randn(*shape, device=dev) * 64).clamp_(-448, 448).to(qd)
        return torch.randint(-127, 128, shape, device=dev, dtype=torch.int8)

    vals, ids = torch.topk(torch.rand(tokens, e, device=dev), k=topk, dim=1)
    srt, wts, e_ids, post = moe_sorting(ids.to(torch.int32), torch.softmax(vals, dim=1), num_experts=e, block_size=a.tile_m)
    kw = dict(model_dim=model, inter_dim=inter, experts=e, topk=topk, tile_m=a.tile_m, tile_n=128, tile_k=128,
              out_dtype="bf16", in_dtype=a.dtype)
    if a.op == "moe1":
        fn = compile_moe_gemm1(**kw, doweight_stage1=False)
        x, w = q8(tokens, model), shuffle_weight(q8(e, 2 * inter, model))
        sx, sw = torch.rand(tokens, device=dev) + 0.5, torch.rand(e * 2 * inter, device=dev) * 1e-3
        out = torch.empty(tokens * topk, inter, dtype=torch.bfloat16, device=dev)
        dims, flops = (inter, model), 2.0 * tokens * topk * 2 * inter * model
        byts = tokens * topk * model + e * 2 * inter * model + tokens * topk * inter * 2
    else:
        fn = compile_moe_gemm2(**kw, doweight_stage2=True, accumulate=False)
        x, w = q8(tokens * topk, inter), shuffle_weight(q8(e, model, inter))
        sx, sw = torch.rand(tokens * topk, device=dev) + 0.5, torch.rand(e * model, device=dev) * 1e-3
        out = torch.empty(tokens * topk, model, dtype=torch.bfloat16, device=dev)
        dims, flops = (model, inter), 2.0 * tokens * topk * model * inter
        byts = tokens * topk * inter + e * model * inter + tokens * topk * model * 2
    st = torch.cuda.current_stream()
    args = (out, x.view(-1), w.view(-1), sx, sw, srt, e_ids, wts, post[:1].contiguous(), tokens, *dims, int(e_ids.numel()), st)
    fn(*args)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.iters):
        fn(*args)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / a.iters
    print(json.dumps({"op": a.op, "tokens": tokens, "inter_dim": inter, "model_dim": model, "experts": e, "topk": topk,
                      "tile_m": a.tile_m, "dtype": a.dtype, "us": round(us, 2), "tflops": round(flops / us / 1e6, 1),
                      "gbs": round(byts / us / 1e3, 1), "status": _lib.read_status()}))


def run_mx(a, dev):
    from flydsl_b200.kernels.gemm.mxfp4_preshuffle import compile_mxfp4_preshuffle_gemm
    from flydsl_b200.kernels.gemm.mxfp8_preshuffle import compile_mxfp8_preshuffle_gemm, shuffle_scale

    m, n, k = a.m, a.n, a.k
    fp4 = a.op == "mx4"
    if fp4:  # random E2M1 pairs, two codes per byte
        x = torch.randint(0, 256, (m, k // 2), dtype=torch.uint8, device=dev)
        w = shuffle_weight(torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=dev))
    else:
        x = (torch.randn(m, k, device=dev) * 64).clamp_(-448, 448).to(torch.float8_e4m3fn)
        w = shuffle_weight((torch.randn(n, k, device=dev) * 64).clamp_(-448, 448).to(torch.float8_e4m3fn))
    sa = shuffle_scale(torch.randint(120, 130, (m, k // 32), dtype=torch.uint8, device=dev))
    sw = shuffle_scale(torch.randint(120, 130, (n, k // 32), dtype=torch.uint8, device=dev))
    c = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    fn = compile_mxfp4_preshuffle_gemm(N=n, K=k) if fp4 else compile_mxfp8_preshuffle_gemm(N=n, K=k)
    args = (c.view(-1), x.view(torch.uint8).view(-1), w.view(torch.uint8).view(-1), sa, sw, None, m, n, torch.cuda.current_stream())
    fn(*args)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.iters):
        fn(*args)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / a.iters
    byts = (m + n) * (k // 2 if fp4 else k) + 2 * m * n + (m + n) * (k // 32)
    print(json.dumps({"op": a.op, "M": m, "N": n, "K": k, "us": round(us, 2), "tflops": round(2.0 * m * n * k / us / 1e6, 1),
                      "gbs": round(byts / us / 1e3, 1), "status": _lib.read_status()}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, required=True)
    ap.add_argument("--n", type=int, required=True)
    ap.add_argument("--k", type=int, required=True)
    ap.add_argument("--dtype", default="fp8", choices=["fp8", "int8"])
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--hint", type=lambda s: int(s, 0), default=0)
    ap.add_argument("--op", default="gemm", choices=["gemm", "quant", "shuffle", "moe1", "moe2", "mx", "mx4"],
                    help="gemm (default), quant: per-token quantiser on [m, k] bf16, shuffle: weight preshuffle of [n, k], "
                    "moe1 / moe2: mixture-of-experts stage 1 / 2 with m tokens, inter_dim n and model_dim k, "
                    "mx / mx4: MXFP8 / MXFP4 block-scaled GEMM")
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--topk", type=int, default=2)
    ap.add_argument("--tile-m", type=int, default=128)
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    if a.op in ("moe1", "moe2"):
        return run_moe(a, dev)
    if a.op in ("mx", "mx4"):
        return run_mx(a, dev)
    if a.op != "gemm":
        from flydsl_b200.utils import pertoken_quant_kernel

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
