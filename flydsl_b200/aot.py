"""Ahead-of-time "compilation" of preshuffle GEMM configurations, after the
reference's tests/python/examples/aot_example.py.

    python -m flydsl_b200.aot [--configs N,K,M,dtype ...] [--manifest out.json] [--run_kernel]

The reference fills a cache directory with JIT-compiled binaries by calling each
launcher once with CPU placeholders under ``COMPILE_ONLY=1``.  Here every kernel
variant is compiled ahead of time into ``libflyb200.so`` by
``python -m flydsl_b200.build``; what remains of the step is (1) making sure
the library is built and loadable, (2) the same ``COMPILE_ONLY=1`` call per
configuration, which resolves the prebuilt variant that configuration will run,
and (3) a manifest of those variants (JSON) in place of the cache directory.
``--run_kernel`` additionally launches every configuration on the GPU and
checks it against the torch dequantise-and-matmul formula, as the reference's
example does.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch

from . import _lib, build, compile_preshuffle_gemm, pertoken_quant, shuffle_weight

# (N, K, M, in_dtype): the reference example's defaults (aot_example.py:190-200)
# plus the decode and prefill shapes this library is tuned for
DEFAULT_CONFIGS = [
    (5120, 8192, 16, "fp8"),
    (5120, 8192, 5120, "fp8"),
    (5120, 8192, 16, "int8"),
    (8192, 8192, 32, "int8"),
    (28672, 8192, 8192, "fp8"),
    (4096, 4096, 128, "fp8"),
    (4096, 4096, 128, "bf16"),
]


def precompile(launch_fn, M, N, K, in_dtype):
    """The reference's pre-compilation call (aot_example.py:38-64): CPU placeholders, COMPILE_ONLY=1."""
    low = in_dtype not in ("fp16", "bf16")
    a_dtype = torch.int8 if low else (torch.float16 if in_dtype == "fp16" else torch.bfloat16)
    prev = os.environ.get("COMPILE_ONLY")
    os.environ["COMPILE_ONLY"] = "1"
    try:
        launch_fn(
            torch.zeros(1, dtype=torch.float16), torch.zeros(1, dtype=a_dtype), torch.zeros(1, dtype=a_dtype),
            torch.zeros(1, dtype=torch.float32) if low else torch.empty(0, dtype=torch.float32),
            torch.zeros(1, dtype=torch.float32) if low else torch.empty(0, dtype=torch.float32),
            torch.empty(0, dtype=torch.float16), M, N, 0,
        )  # fmt: skip
    finally:
        if prev is None:
            os.environ.pop("COMPILE_ONLY", None)
        else:
            os.environ["COMPILE_ONLY"] = prev
    return launch_fn.last_plan


def run_and_verify(launch_fn, M, N, K, in_dtype):
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    a = torch.rand(M, K, device=dev, generator=g)
    b = torch.rand(N, K, device=dev, generator=g)
    if in_dtype in ("fp16", "bf16"):
        dt = torch.float16 if in_dtype == "fp16" else torch.bfloat16
        a_q, b_q = a.to(dt), b.to(dt)
        sa = sb = torch.empty(0, device=dev)
        ref = a_q.float() @ b_q.float().t()
    else:
        qd = torch.int8 if in_dtype == "int8" else torch.float8_e4m3fn
        a_q, sa = pertoken_quant(a, quant_dtype=qd)
        b_q, sb = pertoken_quant(b, quant_dtype=qd)
        ref = (a_q.float() * sa) @ (b_q.float() * sb).t()
    c = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    i8 = (lambda t: t.view(torch.int8)) if in_dtype == "fp8" else (lambda t: t)
    launch_fn(c.view(-1), i8(a_q).view(-1), i8(shuffle_weight(b_q)).view(-1), sa.view(-1), sb.view(-1),
              torch.empty(0, dtype=torch.bfloat16, device=dev), M, N, torch.cuda.current_stream())
    torch.cuda.synchronize()
    err = float((c.float() - ref).abs().max() / ref.abs().max())
    if err > 2e-2:
        raise RuntimeError(f"N={N} K={K} M={M} {in_dtype}: relative error {err:.3g}")
    return err


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--configs", nargs="*", help="N,K,M,dtype (dtype: fp8, int8, fp16, bf16)")
    ap.add_argument("--manifest", default=None, help="write the manifest to this JSON file")
    ap.add_argument("--run_kernel", action="store_true", help="also launch every configuration on the GPU")
    a = ap.parse_args(argv)
    configs = DEFAULT_CONFIGS
    if a.configs:
        configs = []
        for c in a.configs:
            n, k, m, dt = c.split(",")
            configs.append((int(n), int(k), int(m), dt))
    t0 = time.time()
    path = build.build_library()
    _lib.load()
    entries = []
    for n, k, m, dt in configs:
        fn = compile_preshuffle_gemm(N=n, K=k, tile_m=128, tile_n=256, tile_k=128, in_dtype=dt)
        plan = precompile(fn, m, n, k, dt)
        entry = {"N": n, "K": k, "M": m, "in_dtype": dt, "variant": plan}
        if a.run_kernel:
            entry["max_rel_error"] = run_and_verify(fn, m, n, k, dt)
        entries.append(entry)
        print(f"  N={n} K={k} M={m} {dt}: {plan}")
    manifest = {"library": os.path.relpath(path), "library_version": int(_lib.load().flyb200_version()),
                "arch": "sm_100a", "configs": entries, "seconds": round(time.time() - t0, 2)}
    if a.manifest:
        with open(a.manifest, "w") as f:
            json.dump(manifest, f, indent=1)
    print(json.dumps({k: v for k, v in manifest.items() if k != "configs"}))
    return manifest


if __name__ == "__main__":
    sys.exit(0 if main() else 1)
