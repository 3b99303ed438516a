#!/usr/bin/env python3
"""Benchmark of the A8W8 preshuffle GEMM on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c5|c3|...]

Prints ONE JSON line.  A "step" is one pass of the hot path over one batch of
synthetic, seeded input.  Default workload: the column-parallel FP8 GEMM
M=16384, N=57344, K=8192 with N split over the GPUs (N/world output channels
per GPU, strong scaling, no collective on the data path); at one GPU the
whole problem runs on that GPU.  The metric is aggregate TFLOP/s
(2*M*N*K per step / max-over-ranks device time).

`value`     device-timed, operands resident in HBM.
`e2e`       the same step through the Python operator with HOST buffers: the
            step's activations and token scales go pinned-host -> device and
            the output shard comes back device -> pinned-host inside the timed
            region (weights are model state: preshuffled and resident).
`roofline`  the GEMM kernel's own launch time from CUDA events; `roofline.configs`
            holds the single-GPU decode / prefill configurations (HBM- or
            tensor-bound), timed after the main region (not part of `value`),
            and `roofline.cublaslt_fp8_tflops` the library FP8 GEMM
            (torch._scaled_mm) on the same shapes in the same run, for scale.
`cpu_baseline` / `--impl reference`  the reference's torch dequantise-and-matmul
            check on the host cores, on a bounded sample of the same workload.
`config.parity_check`  after the timed regions the outputs are compared with
            the CPU reference on sampled rows and, on several GPUs, the fused
            and the NCCL all-gather paths with each other; a mismatch makes the
            run exit non-zero.
`extras`    side figures (block-scaled and grouped GEMMs).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FP8 = torch.float8_e4m3fn
NOMINAL_FP8_TFLOPS = 4500.0  # dense, datasheet
WORKLOADS = {
    # name: (M, N, K, in_dtype, weight_scale, seed)
    "c5": (16384, 57344, 8192, "fp8", 1.0, 1005),
    "c3": (8192, 28672, 8192, "fp8", 0.02, 1003),
    "c2": (32, 8192, 8192, "int8", 1.0, 1002),
    "c1": (128, 4096, 4096, "fp8", 1.0, 1001),
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"], bf16_sustained=d.get("bf16_tflops_sustained"),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_sustained=1400.0, source="fallback")


def gemm_bytes(m, n, k):
    return m * k + n * k + 2 * m * n + 4 * (m + n)


# ---------------------------------------------------------------------------
# clocks (read-only NVML sampling during the timed region)
# ---------------------------------------------------------------------------
class ClockSampler:
    REASONS = {
        0x8: "hw_slowdown",
        0x40: "hw_thermal_slowdown",
        0x20: "sw_thermal_slowdown",
        0x4: "sw_power_cap",
        0x80: "hw_power_brake_slowdown",
    }

    def __init__(self, device_index: int, period_s: float = 0.005):
        self.samples, self.reasons, self.power = [], set(), []
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self.h = None
        try:
            import pynvml

            self.nv = pynvml
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            try:
                self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception as e:  # NVML missing: report no clocks rather than fail the run
            self.err = repr(e)
            self.h = None
        self.period = period_s

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
                self.power.append(self._power_w())
            except Exception:
                pass
            self._stop.wait(self.period)

    def _power_w(self):
        nv = self.nv
        try:  # instantaneous board power where the driver offers it (the default reading is a running average)
            fv = nv.nvmlDeviceGetFieldValues(self.h, [nv.NVML_FI_DEV_POWER_INSTANT])[0]
            if fv.nvmlReturn == 0 and fv.value.uiVal > 0:
                return fv.value.uiVal / 1000.0
        except Exception:
            pass
        return nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0

    def start(self):
        if self.h is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join()
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {
            "sm_mhz": statistics.median(self.samples),
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
            "power_w_max": max(self.power) if self.power else None,
        }


# ---------------------------------------------------------------------------
# the reference's CPU path (torch dequantise-and-matmul) on a bounded sample
# ---------------------------------------------------------------------------
def cpu_reference_rate(m, n, k, in_dtype, seconds_budget, steps=1, warmup=0):
    """Time oracle.run_torch on a [ms, k] x [ns, k] sample of the workload on all
    host threads.  Returns (TFLOP/s, sample description, seconds per step, threads)."""
    from oracle import a8w8_oracle as oracle

    torch.set_num_threads(os.cpu_count() or 1)
    threads = torch.get_num_threads()
    # calibrate on a small probe, then size the sample for the time budget
    pm, pn = min(m, 256), min(n, 2048)
    a_q, b_q, sa, sb = oracle.make_inputs(pm, pn, k, in_dtype, seed=1)
    oracle.run_torch(a_q, b_q, sa, sb)
    t0 = time.perf_counter()
    oracle.run_torch(a_q, b_q, sa, sb)
    probe = time.perf_counter() - t0
    rate = 2.0 * pm * pn * k / max(probe, 1e-6)
    per_step = seconds_budget / max(1, steps + warmup)
    target_flops = rate * per_step
    ms = min(m, 2048)
    ns = int(min(n, max(256, target_flops / (2.0 * ms * k))))
    ns = max(16, ns // 16 * 16)
    a_q, b_q, sa, sb = oracle.make_inputs(ms, ns, k, in_dtype, seed=2)
    for _ in range(warmup):
        oracle.run_torch(a_q, b_q, sa, sb)
    t0 = time.perf_counter()
    for _ in range(steps):
        oracle.run_torch(a_q, b_q, sa, sb)
    dt = (time.perf_counter() - t0) / steps
    tflops = 2.0 * ms * ns * k / dt / 1e12
    sample = f"rows[0:{ms}] x channels[0:{ns}] x K={k} of the workload, fp32 dequantise + torch.mm, {steps} timed pass(es)"
    return tflops, sample, dt, threads


def run_reference_arm(args, m, n, k, in_dtype, workload):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    tflops, sample, dt, threads = cpu_reference_rate(m, n, k, in_dtype, seconds_budget=90.0, steps=args.steps,
                                                     warmup=args.warmup)
    line = {
        "impl": "reference",
        "metric": "fp8_gemm_tflops",
        "value": tflops,
        "unit": "TFLOP/s",
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": dt * 1e3,
        "higher_is_better": True,
        "scaling": "strong",
        "vs_baseline": None,
        "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": workload, "M": m, "N": n, "K": k, "in_dtype": in_dtype},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
def quantise_rows(x, in_dtype):
    """Per-row symmetric quantisation as the benchmark configurations state it:
    scale = amax / 448 (fp8) or amax / 127 with round-to-nearest (int8)."""
    from flydsl_b200 import pertoken_quant

    if in_dtype == "int8":
        s = x.abs().amax(dim=-1, keepdim=True) / 127.0
        s.masked_fill_(s == 0, 1.0)
        return torch.round(x / s).clamp_(-127, 127).to(torch.int8), s
    return pertoken_quant(x, quant_dtype=FP8)


def quantised_on_gpu(m, n, k, in_dtype, dev, seed, weight_scale):
    """Seeded N(0,1) activations [m, k] and weights [n, k] (times weight_scale),
    quantised per token / per output channel on the GPU."""
    g = torch.Generator(device=dev).manual_seed(seed)
    a_q, sa = quantise_rows(torch.randn(m, k, generator=g, device=dev), in_dtype)
    # weights in row chunks to bound the fp32 temporary
    w_q = torch.empty(n, k, dtype=a_q.dtype, device=dev)
    sb = torch.empty(n, 1, dtype=torch.float32, device=dev)
    step = 8192
    for i in range(0, n, step):
        q, s = quantise_rows(torch.randn(min(step, n - i), k, generator=g, device=dev) * weight_scale, in_dtype)
        w_q[i : i + q.shape[0]] = q
        sb[i : i + q.shape[0]] = s
    return a_q, sa.view(-1), w_q, sb.view(-1)


def settle(seconds=0.3):
    """Let the board leave the power-capped state of the preceding tensor-bound runs
    before a short memory-bound case is timed (idle host time, outside every timed region)."""
    torch.cuda.synchronize()
    time.sleep(seconds)


def time_config(m, n, k, in_dtype, dev, iters=40, hint=0, seed=0, weight_scale=1.0):
    """Device time of one single-GPU configuration: CUDA events around a graph
    replay of `iters` launches whose operand copies rotate, so that consecutive
    launches do not find their weights in L2.  Operands: seeded N(0,1),
    quantised per token / per channel as the configuration states."""
    from flydsl_b200 import compile_preshuffle_gemm, shuffle_weight

    per = m * k + n * k + 2 * m * n
    copies = max(1, min(8, int(400e6 // per) + 1))
    fn = compile_preshuffle_gemm(N=n, K=k, tile_m=128, tile_n=256, tile_k=128, in_dtype=in_dtype, variant_hint=hint)
    a_q, sa, w_q, sb = quantised_on_gpu(m, n, k, in_dtype, dev, seed, weight_scale)
    w_s = shuffle_weight(w_q).view(torch.int8)
    del w_q
    A = [a_q.view(torch.int8)] + [a_q.view(torch.int8).clone() for _ in range(copies - 1)]
    W = [w_s] + [w_s.clone() for _ in range(copies - 1)]
    C = [torch.empty(m, n, dtype=torch.bfloat16, device=dev) for _ in range(copies)]
    bias = torch.empty(0, dtype=torch.bfloat16, device=dev)
    st = torch.cuda.Stream()

    def launch(i):
        j = i % copies
        fn(C[j].view(-1), A[j].view(-1), W[j].view(-1), sa, sb, bias, m, n, st)

    with torch.cuda.stream(st):
        for i in range(3):
            launch(i)
        st.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            for i in range(iters):
                launch(i)
        g.replay()
        st.synchronize()
        best = None
        for _ in range(3):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(st)
            g.replay()
            e1.record(st)
            st.synchronize()
            t = e0.elapsed_time(e1) * 1e3 / iters
            best = t if best is None else min(best, t)
    return best, copies


def time_scaled_mm_graph(m, n, k, dev, iters=20, seed=0):
    """The library FP8 GEMM on a decode-sized shape, timed like time_config: CUDA events around a
    graph replay of `iters` calls whose weight copies rotate past L2.  Returns (us, mode) or (None, reason)."""
    a_q, sa, w_q, sb = quantised_on_gpu(m, n, k, "fp8", dev, seed, 1.0)
    per = m * k + n * k + 2 * m * n
    copies = max(1, min(8, int(400e6 // per) + 1))
    W = [w_q] + [w_q.clone() for _ in range(copies - 1)]
    out = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    s_a, s_b = sa.view(m, 1).contiguous(), sb.view(1, n).contiguous()
    st = torch.cuda.Stream()
    try:
        with torch.cuda.stream(st):
            for i in range(3):
                torch._scaled_mm(a_q, W[i % copies].t(), scale_a=s_a, scale_b=s_b, out_dtype=torch.bfloat16, out=out)
            st.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=st):
                for i in range(iters):
                    torch._scaled_mm(a_q, W[i % copies].t(), scale_a=s_a, scale_b=s_b, out_dtype=torch.bfloat16, out=out)
            g.replay()
            st.synchronize()
            best = None
            for _ in range(3):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(st)
                g.replay()
                e1.record(st)
                st.synchronize()
                t = e0.elapsed_time(e1) * 1e3 / iters
                best = t if best is None else min(best, t)
        return best, "rowwise"
    except Exception as e:
        return None, repr(e)[:120]


def time_scaled_mm(m, n, k, dev, iters=5, seed=0, weight_scale=1.0):
    """The library FP8 GEMM (torch._scaled_mm -> cuBLASLt) on the same operands and
    scales, bf16 output: the FP8 yardstick this machine offers, since no FP8 peak is
    measured.  Returns (us, scaling mode) or (None, reason)."""
    a_q, sa, w_q, sb = quantised_on_gpu(m, n, k, "fp8", dev, seed, weight_scale)
    out = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    modes = (("rowwise", sa.view(m, 1).contiguous(), sb.view(1, n).contiguous()),
             ("tensorwise", sa.max().view(()), sb.max().view(())))
    last = "no mode ran"
    for name, s_a, s_b in modes:
        try:
            def run():
                return torch._scaled_mm(a_q, w_q.t(), scale_a=s_a, scale_b=s_b, out_dtype=torch.bfloat16, out=out)

            for _ in range(2):
                run()
            torch.cuda.synchronize()
            best = None
            for _ in range(3):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(iters):
                    run()
                e1.record()
                torch.cuda.synchronize()
                t = e0.elapsed_time(e1) * 1e3 / iters
                best = t if best is None else min(best, t)
            return best, name
        except Exception as e:  # this build of the library lacks the mode: try the next
            last = f"{name}: {repr(e)[:120]}"
    return None, last


def time_mx(m, n, k, dev, iters=10, fp4=False):
    """Device time of the block-scaled GEMM, MXFP8 or (fp4=True) MXFP4 codes (operands larger than L2,
    back-to-back launches); algorithmic bytes as in the reference's tests
    (tests/kernels/test_preshuffle_gemm.py:695 and :455-459)."""
    from flydsl_b200 import shuffle_weight
    from flydsl_b200.kernels.gemm.mxfp4_preshuffle import compile_mxfp4_preshuffle_gemm
    from flydsl_b200.kernels.gemm.mxfp8_preshuffle import compile_mxfp8_preshuffle_gemm, shuffle_scale

    g = torch.Generator(device=dev).manual_seed(78)
    code_bytes = k // 2 if fp4 else k  # bytes per row of codes

    def codes(rows):
        if fp4:  # random E2M1 pairs
            return torch.randint(0, 256, (rows, code_bytes), generator=g, dtype=torch.uint8, device=dev)
        return (torch.randn(rows, k, generator=g, device=dev) * 64).clamp_(-448, 448).to(FP8).view(torch.uint8)

    a = codes(m)
    byts = (m + n) * code_bytes + 2 * m * n + (m + n) * (k // 32)
    # weights (and their scales) rotate over enough copies that no launch finds them in L2
    copies = max(1, min(6, int(400e6 // byts) + 1))
    ws, sws = [], []
    for _ in range(copies):
        ws.append(shuffle_weight(codes(n)))
        sws.append(shuffle_scale(torch.randint(120, 130, (n, k // 32), generator=g, dtype=torch.uint8, device=dev)))
    sa = shuffle_scale(torch.randint(120, 130, (m, k // 32), generator=g, dtype=torch.uint8, device=dev))
    c = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    fn = compile_mxfp4_preshuffle_gemm(N=n, K=k) if fp4 else compile_mxfp8_preshuffle_gemm(N=n, K=k)
    st = torch.cuda.Stream()

    def launch(i):
        j = i % copies
        fn(c.view(-1), a.view(-1), ws[j].view(torch.uint8).view(-1), sa, sws[j], None, m, n, st)

    with torch.cuda.stream(st):
        for i in range(3):
            launch(i)
        st.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=st):
            for i in range(iters):
                launch(i)
        graph.replay()
        st.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(st)
        graph.replay()
        e1.record(st)
        st.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / iters
    nominal = 2 * NOMINAL_FP8_TFLOPS if fp4 else NOMINAL_FP8_TFLOPS
    return {"us": round(us, 2), "tflops": round(2.0 * m * n * k / us / 1e6, 1), "hbm_gbs": round(byts / us / 1e3, 1),
            ("frac_of_nominal_fp4_9000" if fp4 else "frac_of_nominal_fp8"): round(2.0 * m * n * k / us / 1e6 / nominal, 3),
            "algorithmic_bytes": int(byts), "rotating_copies": copies}


def time_mx_mixed(m, n, k, dev, iters=10):
    """Device time of the MXFP6-activation x MXFP4-weight GEMM through its launcher (the call includes the
    launcher's per-call conversion of the activations from the reference's layout to byte containers);
    algorithmic bytes as in the reference's test (tests/kernels/test_preshuffle_gemm.py:582-583)."""
    from flydsl_b200.kernels.gemm.mxfp4_preshuffle import compile_mxfp4_preshuffle_gemm, shuffle_scale_w4, shuffle_weight_w4

    g = torch.Generator(device=dev).manual_seed(79)
    a_pad = torch.randint(0, 256, (m, k // 32, 32), generator=g, dtype=torch.uint8, device=dev)
    a_pad[:, :, 24:] = 0  # per 32 elements: 24 bytes of packed 6-bit codes + 8 zero bytes
    a_pad = a_pad.view(m, k)
    w = shuffle_weight_w4(torch.randint(0, 256, (n, k // 2), generator=g, dtype=torch.uint8, device=dev), 16, False, False,
                          for_a_dtype="fp6")
    sa = shuffle_scale_w4(torch.randint(120, 130, (m, k // 32), generator=g, dtype=torch.uint8, device=dev), 1, False)
    sw = shuffle_scale_w4(torch.randint(120, 130, (n, k // 32), generator=g, dtype=torch.uint8, device=dev), 1, False)
    c = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    fn = compile_mxfp4_preshuffle_gemm(N=n, K=k, a_dtype="fp6", b_dtype="fp4")
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        for _ in range(3):
            fn(c.view(-1), a_pad.view(-1), w.view(-1), sa, sw, None, m, n, st)
        st.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(st)
        for _ in range(iters):
            fn(c.view(-1), a_pad.view(-1), w.view(-1), sa, sw, None, m, n, st)
        e1.record(st)
        st.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / iters
    byts = m * k + n * k // 2 + 2 * m * n + (m + n) * (k // 32)
    return {"us": round(us, 2), "tflops": round(2.0 * m * n * k / us / 1e6, 1), "algorithmic_bytes": int(byts),
            "note": "eager launches incl. the activation layout conversion; weights travel in byte containers (N*K bytes)"}


def time_moe(tokens, model_dim, inter_dim, experts, topk, tile_m, dev, iters=20):
    """Device time of the two mixture-of-experts GEMM stages (activation gather
    included) on seeded synthetic routing, with the algorithmic bytes of the
    reference's own model: routed activation rows + every expert's weights once +
    output rows (tests/kernels/test_moe_gemm_2stage.py:2001-2025)."""
    from flydsl_b200 import shuffle_weight
    from flydsl_b200.kernels.moe.moe_gemm_2stage import compile_moe_gemm1, compile_moe_gemm2, moe_sorting

    g = torch.Generator(device=dev).manual_seed(77)
    score = torch.rand(tokens, experts, generator=g, device=dev)
    vals, ids = torch.topk(score, k=topk, dim=1)
    srt, wts, e_ids, post = moe_sorting(ids.to(torch.int32), torch.softmax(vals, dim=1), num_experts=experts, block_size=tile_m)
    n_valid, blocks = post[:1].contiguous(), int(e_ids.numel())

    def q8(*shape):
        return (torch.randn(*shape, generator=g, device=dev) * 64).clamp_(-448, 448).to(FP8)

    x, a2 = q8(tokens, model_dim), q8(tokens * topk, inter_dim)
    w1 = shuffle_weight(q8(experts, 2 * inter_dim, model_dim))
    w2 = shuffle_weight(q8(experts, model_dim, inter_dim))
    sx, sa2 = torch.rand(tokens, device=dev) + 0.5, torch.rand(tokens * topk, device=dev) + 0.5
    sw1, sw2 = torch.rand(experts * 2 * inter_dim, device=dev) * 1e-3, torch.rand(experts * model_dim, device=dev) * 1e-3
    out1 = torch.empty(tokens * topk, inter_dim, dtype=torch.bfloat16, device=dev)
    out2 = torch.empty(tokens * topk, model_dim, dtype=torch.bfloat16, device=dev)
    kw = dict(model_dim=model_dim, inter_dim=inter_dim, experts=experts, topk=topk, tile_m=tile_m, tile_n=128, tile_k=128,
              out_dtype="bf16", in_dtype="fp8")
    g1 = compile_moe_gemm1(**kw, doweight_stage1=False)
    g2 = compile_moe_gemm2(**kw, doweight_stage2=True, accumulate=False)
    copies = 4  # the launches of a timed graph rotate over copies of the weights: 4 x (134 + 67) MB > L2
    w1s = [w1] + [w1.clone() for _ in range(copies - 1)]
    w2s = [w2] + [w2.clone() for _ in range(copies - 1)]
    st = torch.cuda.Stream()
    res = {}
    for name, fn, ws, head, tail, flops, byts in (
        ("stage1", g1, w1s, (out1, x.view(-1)), (sx, sw1, srt, e_ids, wts, n_valid, tokens, inter_dim, model_dim, blocks),
         2.0 * tokens * topk * 2 * inter_dim * model_dim,
         tokens * topk * model_dim + experts * 2 * inter_dim * model_dim + tokens * topk * inter_dim * 2),
        ("stage2", g2, w2s, (out2, a2.view(-1)), (sa2, sw2, srt, e_ids, wts, n_valid, tokens, model_dim, inter_dim, blocks),
         2.0 * tokens * topk * model_dim * inter_dim,
         tokens * topk * inter_dim + experts * model_dim * inter_dim + tokens * topk * model_dim * 2),
    ):
        with torch.cuda.stream(st):
            for i in range(3):
                fn(*head, ws[i % copies].view(-1), *tail, st)
            st.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=st):
                for i in range(iters):
                    fn(*head, ws[i % copies].view(-1), *tail, st)
            graph.replay()
            st.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(st)
            graph.replay()
            e1.record(st)
            st.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / iters
        res[name] = {"us": round(us, 2), "tflops": round(flops / us / 1e6, 1), "hbm_gbs": round(byts / us / 1e3, 1),
                     "algorithmic_bytes": int(byts), "launches_per_call": 2}
    res["config"] = {"tokens": tokens, "model_dim": model_dim, "inter_dim": inter_dim, "experts": experts, "topk": topk,
                     "tile_m": tile_m, "blocks": blocks, "l2": "weights rotated over 4 copies (> L2) inside one CUDA graph"}
    return res


def parity_check(op, a_q, sa, w_q_local, sb_local, local, full_ag, full_fused, dev, world, rank):
    """Checker, outside every timed region: (i) on sampled rows this rank's output
    columns against the CPU reference (fp32 dequantise-and-matmul, rtol = atol =
    1e-2, every sampled element must pass), on up to 8192 of its columns (first and
    last 4096); (ii) on several GPUs the all-gathered and the fused full outputs
    against each other (bitwise) and their local columns against the local shard
    (bitwise).  Returns a dict; `ok` is the AND over all ranks."""
    import torch.distributed as dist

    from oracle import a8w8_oracle as oracle

    m = a_q.shape[0]
    nl = w_q_local.shape[0]
    gen = torch.Generator().manual_seed(4242)  # the same rows on every rank
    pick = torch.cat([torch.tensor([0, 1, 127, 128, m - 129, m - 2, m - 1]), torch.randint(0, m, (57,), generator=gen)])
    pick = pick.clamp_(0, m - 1).unique().to(dev)
    cols = torch.arange(nl, device=dev) if nl <= 8192 else torch.cat(
        [torch.arange(0, 4096, device=dev), torch.arange(nl - 4096, nl, device=dev)])
    ref = oracle.run_torch(a_q[pick].cpu(), w_q_local[cols].cpu(), sa[pick].cpu(), sb_local[cols].cpu())
    got = local[pick][:, cols].float().cpu()
    bad = int(oracle.strict_mismatches(got, ref, 1e-2, 1e-2))
    res = {"oracle_rows": int(pick.numel()), "oracle_cols_per_rank": int(cols.numel()), "oracle_mismatches": bad,
           "rtol_atol": 1e-2}
    ok = bad == 0
    if world > 1:
        n0, n1 = op.spec.n0, op.spec.n1
        eq_shard = bool(torch.equal(full_ag[:, n0:n1], local))
        res["allgather_shard_equals_local"] = eq_shard
        ok = ok and eq_shard
        if full_fused is not None:
            eq_fused = bool(torch.equal(full_fused, full_ag))
            res["fused_equals_allgather"] = eq_fused
            ok = ok and eq_fused
        flag = torch.tensor([1 if ok else 0, bad], dtype=torch.int64, device=dev)
        worst = flag.clone()
        dist.all_reduce(worst[:1], op=dist.ReduceOp.MIN)
        dist.all_reduce(flag[1:], op=dist.ReduceOp.SUM)
        ok = bool(worst[0].item() == 1)
        res["oracle_mismatches"] = int(flag[1].item())
        res["ranks_checked"] = world
    res["ok"] = ok
    return res


# DRAM traffic of the dominant kernel, from one ncu capture of a smaller case with the
# same tile order (profiles/gemm_rows_fp8_traffic.md): bytes read + written per launch
# there, and that case's algorithmic bytes.  The weights stream once per group of row
# tiles and the activations once, so the full workload's traffic is estimated group by
# group (see traffic_estimate), not by plain proportion.
NCU_TRAFFIC_CASE = {"m": 4096, "n": 14336, "k": 8192, "group_m": 32, "read": 176.1e6, "write": 95.7e6}


def traffic_estimate(m, n, k, group_m):
    """DRAM bytes per launch of the large-M kernel under its tile order: weights once per
    group of `group_m` row tiles (they do not survive in L2 from one group to the next,
    apart from the turn-around tiles), activations once, output once."""
    groups = -(-((m + 127) // 128) // group_m)
    return groups * n * k + m * k + 2 * m * n + 4 * (m + n)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c5", choices=sorted(WORKLOADS))
    ap.add_argument("--hint", type=lambda v: int(v, 0), default=0, help="variant_hint of the main workload (tuning sweeps)")
    ap.add_argument("--no-extras", action="store_true", help="skip the single-GPU decode/prefill side measurements")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-fused", action="store_true", help="skip the fused GEMM + all-gather measurement (N > 1)")
    ap.add_argument("--no-parity", action="store_true", help="skip the parity check after the timed regions")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    m, n, k, in_dtype, wscale, seed = WORKLOADS[args.workload]
    workload = f"{args.workload}: {in_dtype} A8W8 preshuffle GEMM M={m} N={n} K={k}, N split over GPUs"

    if args.impl == "reference":
        run_reference_arm(args, m, n, k, in_dtype, workload)
        return

    import torch.distributed as dist

    from flydsl_b200 import _lib
    from flydsl_b200.column_parallel import ColumnParallelGemm, pinned_near

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU path")
    _lib.load()  # fail loudly if the CUDA library is missing

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    cpu_group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        cpu_group = dist.new_group(backend="gloo")

    peaks = measured_peaks()
    op = ColumnParallelGemm(n, k, in_dtype=in_dtype, rank=rank, world=world, cpu_group=cpu_group, variant_hint=args.hint)
    nl = op.spec.n_local
    # every rank: replicated activations, its own weight shard (seeded per shard)
    a_q, sa, w_q, sb = quantised_on_gpu(m, nl, k, in_dtype, dev, seed + 17 * rank, wscale)
    if world > 1:  # identical activations on all ranks
        dist.broadcast(a_q.view(torch.int8), src=0)
        dist.broadcast(sa, src=0)
    op.load_weight_shard(w_q, sb)
    c = torch.empty(m, nl, dtype=torch.bfloat16, device=dev)
    stream = torch.cuda.current_stream()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, reps, warm=2):
        """max over ranks of the device time per call of fn, CUDA events on the launching stream."""
        for _ in range(warm):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            fn()
        e1.record(stream)
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) / reps

    # ---- device-timed region: K steps, inputs resident ---------------------
    for _ in range(args.warmup):
        op.forward(a_q, sa, out=c)
    barrier()
    # More untimed steps right up to the timed region (about half a second of them): the
    # board's power and clock telemetry lags by tens of milliseconds, and the timed steps
    # should run - and be sampled - at the clocks a long job sees, not at a cold burst.
    w0, w1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0.record(stream)
    op.forward(a_q, sa, out=c)
    w1.record(stream)
    torch.cuda.synchronize()
    preroll = max(0, min(400, int(0.5 / max(w0.elapsed_time(w1) * 1e-3, 1e-5))))
    for _ in range(preroll):
        op.forward(a_q, sa, out=c)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    barrier()
    evs[0].record(stream)
    for i in range(args.steps):
        op.forward(a_q, sa, out=c)
        evs[i + 1].record(stream)
    barrier()
    total_ms = evs[0].elapsed_time(evs[-1])
    kernel_ms = [evs[i].elapsed_time(evs[i + 1]) for i in range(args.steps)]
    clocks = sampler.stop() if sampler else None
    status = _lib.read_status()
    t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    flops_step = 2.0 * m * n * k
    value = flops_step / (ms_per_step * 1e-3) / 1e12

    # ---- end to end: host buffers in, host buffer out ------------------------
    # pinned buffers on the GPU's own NUMA node; on several GPUs each rank uploads
    # 1/world of the activations and the ranks all-gather them over NVLink
    a_host = pinned_near(dev, tuple(a_q.shape), torch.int8)
    a_host.copy_(a_q.view(torch.int8))
    sa_host = pinned_near(dev, (m,), torch.float32)
    sa_host.copy_(sa)
    c_host = pinned_near(dev, (m, nl), torch.bfloat16)
    e2e_steps = max(3, min(args.steps, 10))
    e2e_ms = timed(lambda: op.forward_host(a_host, sa_host, c_host, chunks=8), e2e_steps)
    e2e_value = flops_step / (e2e_ms * 1e-3) / 1e12
    h2d = int(op.last_h2d_bytes)
    d2h = c_host.numel() * 2
    e2e_ok = bool(torch.equal(c_host, c.cpu())) if not args.no_parity else None
    del a_host, c_host

    # ---- optional: with the all-gather of the shards (full output on every rank)
    gathered = None
    if world > 1:
        reps = max(3, min(args.steps, 10))
        g_ms = timed(lambda: op.forward_full(a_q, sa, row_major=False), reps)
        gathered = {"ms_per_step": g_ms, "tflops": flops_step / (g_ms * 1e-3) / 1e12,
                    "what": "GEMM shard + NCCL all-gather of bf16 shards (shard-major result)"}

    # ---- optional: the same full output from the GEMM fused with the exchange
    #      (tiles TMA-stored straight into every rank's full-width buffer)
    fused = None
    fused_ready = False
    if world > 1 and not args.no_fused:
        try:
            op.enable_fused_gather(m_max=m)
            fused_ready = True
            reps = max(3, min(args.steps, 10))
            f_ms = timed(lambda: op.forward_full_fused(a_q, sa), reps)
            fused = {"ms_per_step": f_ms, "tflops": flops_step / (f_ms * 1e-3) / 1e12,
                     "what": "one GEMM kernel per rank whose epilogue TMA-stores every tile into all ranks' "
                             "full-width buffers (peer memory), then a one-element NCCL all-reduce as barrier"}
        except Exception as e:  # symmetric memory unavailable: report, keep the main numbers
            fused = {"unavailable": repr(e)[:200]}

    # ---- parity, after every timed region --------------------------------------
    parity = None
    if not args.no_parity:
        local = op.forward(a_q, sa, out=c)
        full_ag = op.forward_full(a_q, sa, row_major=True) if world > 1 else None
        full_fused = op.forward_full_fused(a_q, sa) if fused_ready else None
        barrier()
        parity = parity_check(op, a_q, sa, w_q, sb, local, full_ag, full_fused, dev, world, rank)
        parity["e2e_output_equals_device_output"] = e2e_ok
        parity["ok"] = bool(parity["ok"] and e2e_ok)
        del full_ag, full_fused
    del w_q

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        if parity is not None and not parity["ok"]:
            sys.exit(3)
        return

    # ---- rank 0: roofline, extras, CPU baseline, the JSON line ----------------
    med_ms = statistics.median(kernel_ms)
    flops_launch = 2.0 * m * nl * k
    achieved = flops_launch / (med_ms * 1e-3) / 1e12
    fp8_peak = 2.0 * peaks["bf16_tflops"]  # burst: the denominator of the short cases in roofline.configs
    # the timed steps run after half a second at the power cap: the matching measured figure is the sustained one
    fp8_peak_sustained = 2.0 * (peaks["bf16_sustained"] or peaks["bf16_tflops"])
    plan = op.launch.plan(m)
    group_m = (args.hint >> 16) & 0xFF or 32
    traffic = None
    traffic_note = "no ncu capture recorded for this build"
    if NCU_TRAFFIC_CASE:
        tc = NCU_TRAFFIC_CASE
        model_small = traffic_estimate(tc["m"], tc["n"], tc["k"], tc["group_m"])
        traffic = (tc["read"] + tc["write"]) / model_small * traffic_estimate(m, nl, k, group_m)
        traffic_note = (f"ncu dram__bytes_read+write of {tc['m']}x{tc['n']}x{tc['k']} (same tile order, group {tc['group_m']}): "
                        f"{(tc['read'] + tc['write']) / 1e6:.0f} MB per launch = {(tc['read'] + tc['write']) / model_small:.2f} x the "
                        "tile-order model (weights once per group of row tiles + activations + output), scaled to this "
                        "launch by that model; profiles/gemm_rows_fp8_traffic.md")
    roofline = {
        "bound": "tensor",
        "kernel": f"gemm_rows_kernel<fp8> (tcgen05 kind::f8f6f4, 128x{plan['bn']} tiles, persistent, {plan['stages']} stages)",
        "achieved": achieved,
        "peak": fp8_peak_sustained,
        "unit": "TFLOP/s",
        "frac": achieved / fp8_peak_sustained,
        "peak_source": f"2 x {peaks['source']} dense bf16 SUSTAINED ({peaks['bf16_sustained']} TFLOP/s; the kernel is timed after "
                       f"~0.5 s at the power cap): no FP8 figure is measured.  Against 2 x the bf16 burst figure "
                       f"({peaks['bf16_tflops']}): frac_of_2x_bf16_burst",
        "frac_of_2x_bf16_burst": achieved / fp8_peak,
        "frac_of_nominal_4500": achieved / NOMINAL_FP8_TFLOPS,
        "traffic": traffic,
        "traffic_note": traffic_note,
        "algorithmic_bytes": gemm_bytes(m, nl, k),
        "launch_ms_median": med_ms,
    }
    extras = {}
    if not args.no_extras and world == 1:  # single-GPU side measurements: not repeated in the multi-GPU runs
        del c, a_q
        torch.cuda.empty_cache()
        PDLW = 3 << 28  # small-M kernel: dependent launch with early prefetch of the (static) weights
        cases = [
            # name, M, N, K, dtype, weight scale, seed, bound, also time with static-weight prefetch
            ("c1_fp8_128x4096x4096", 128, 4096, 4096, "fp8", 1.0, 1001, "hbm", True),
            ("c2_int8_32x8192x8192", 32, 8192, 8192, "int8", 1.0, 1002, "hbm", True),
            ("c4_fp8_1x8192x8192", 1, 8192, 8192, "fp8", 1.0, 1040, "hbm", True),
            ("c4_fp8_16x8192x8192", 16, 8192, 8192, "fp8", 1.0, 1041, "hbm", True),
            ("c4_fp8_64x8192x8192", 64, 8192, 8192, "fp8", 1.0, 1042, "hbm", False),
            ("c4_fp8_256x8192x8192", 256, 8192, 8192, "fp8", 1.0, 1043, "hbm", False),
            ("c4_fp8_1024x8192x8192", 1024, 8192, 8192, "fp8", 1.0, 1044, "tensor", False),
            ("c4_fp8_4096x8192x8192", 4096, 8192, 8192, "fp8", 1.0, 1045, "tensor", False),
            ("c4_fp8_16384x8192x8192", 16384, 8192, 8192, "fp8", 1.0, 1046, "tensor", False),
            ("c3_fp8_8192x28672x8192", 8192, 28672, 8192, "fp8", 0.02, 1003, "tensor", False),
        ]
        configs = {}
        for name, em, en, ek, edt, ews, eseed, bound, static_too in cases:
            iters = 20 if em <= 4096 and en <= 8192 else 5
            settle()  # every case starts from the same idle state, not from the throttled end of the previous one
            us, copies = time_config(em, en, ek, edt, dev, iters=iters, seed=eseed, weight_scale=ews)
            by = gemm_bytes(em, en, ek)
            tf = 2.0 * em * en * ek / us / 1e6
            row = {"us": round(us, 2), "bound": bound}
            if bound == "hbm":
                row["gbs"] = round(by / us / 1e3, 0)
                row["frac"] = round(by / us / 1e3 / peaks["hbm_gbs"], 3)
            else:
                row["tflops"] = round(tf, 0)
                row["frac"] = round(tf / fp8_peak, 3)
                row["frac_nominal"] = round(tf / NOMINAL_FP8_TFLOPS, 3)
            if static_too:
                us2, _ = time_config(em, en, ek, edt, dev, iters=iters, hint=PDLW, seed=eseed, weight_scale=ews)
                row["us_weights_static"] = round(us2, 2)
                row["frac_weights_static"] = round(by / us2 / 1e3 / peaks["hbm_gbs"], 3)
            configs[name] = row
            torch.cuda.empty_cache()
        roofline["configs"] = configs
        roofline["configs_note"] = (f"hbm rows: algorithmic bytes / time over the measured copy bandwidth {peaks['hbm_gbs']} GB/s; "
                                    f"tensor rows: over {fp8_peak:.0f} TFLOP/s (2 x measured bf16) and over nominal 4500; CUDA events "
                                    "around a graph replay, operand copies rotated past L2, seeded N(0,1) inputs quantised per "
                                    "token / per channel; *_weights_static = builder kwarg weights_static=True")
        lib_fp8 = {}
        for name, em, en, ek, ews, eseed in (("c3_8192x28672x8192", 8192, 28672, 8192, 0.02, 1003),
                                            ("c5_16384x57344x8192", m, n, k, wscale, seed)):
            us, mode = time_scaled_mm(em, en, ek, dev, iters=5, seed=eseed, weight_scale=ews)
            lib_fp8[name] = ({"tflops": round(2.0 * em * en * ek / us / 1e6, 0), "us": round(us, 1), "scaling": mode}
                             if us else {"unavailable": mode})
            torch.cuda.empty_cache()
        # ... and on two decode-sized shapes (FP8 both: the library has no INT8 counterpart with these scales)
        for name, em, en, ek, eseed in (("c1_128x4096x4096", 128, 4096, 4096, 1001), ("m32_32x8192x8192", 32, 8192, 8192, 1002)):
            settle()
            us, mode = time_scaled_mm_graph(em, en, ek, dev, seed=eseed)
            lib_fp8[name] = ({"us": round(us, 2), "hbm_frac": round(gemm_bytes(em, en, ek) / us / 1e3 / peaks["hbm_gbs"], 3),
                              "scaling": mode} if us else {"unavailable": mode})
            torch.cuda.empty_cache()
        roofline["cublaslt_fp8_tflops"] = lib_fp8
        # the MXFP8 block-scaled GEMM on the prefill shape of configuration 3 (halved N to bound the run)
        settle()
        extras["mxfp8_8192x14336x8192"] = time_mx(8192, 14336, 8192, dev, iters=5)
        # ... and on the reference's own MXFP8 test shapes (tests/kernels/test_preshuffle_gemm.py:590-598)
        for mm in (32, 64, 128, 1024):
            settle()
            r = time_mx(mm, 8192, 8192, dev, iters=20)
            r["hbm_frac_of_measured"] = round(r["hbm_gbs"] / peaks["hbm_gbs"], 3)
            extras[f"mxfp8_{mm}x8192x8192"] = r
        # the MXFP4 block-scaled GEMM (two codes per byte): prefill shape and two of the reference's test shapes
        settle()
        extras["mxfp4_8192x14336x8192"] = time_mx(8192, 14336, 8192, dev, iters=5, fp4=True)
        for mm in (64, 1024):
            settle()
            r = time_mx(mm, 8192, 8192, dev, iters=20, fp4=True)
            r["hbm_frac_of_measured"] = round(r["hbm_gbs"] / peaks["hbm_gbs"], 3)
            extras[f"mxfp4_{mm}x8192x8192"] = r
        settle()
        extras["mxfp6_x_mxfp4_4096x8192x8192"] = time_mx_mixed(4096, 8192, 8192, dev)
        # the grouped (mixture-of-experts) stages: a decode-sized and a prefill-sized batch
        for name, mt, mtile in (("moe_fp8_decode_32tok", 32, 16), ("moe_fp8_prefill_4096tok", 4096, 128)):
            settle()
            r = time_moe(mt, 4096, 2048, 8, 2, mtile, dev)
            for stage in ("stage1", "stage2"):
                r[stage]["hbm_frac_of_measured"] = round(r[stage]["hbm_gbs"] / peaks["hbm_gbs"], 3)
                r[stage]["frac_of_nominal_fp8"] = round(r[stage]["tflops"] / NOMINAL_FP8_TFLOPS, 3)
            extras[name] = r
    cpu = None
    if not args.no_cpu_baseline and world == 1:
        tf, sample, dt, threads = cpu_reference_rate(m, n, k, in_dtype, seconds_budget=15.0, steps=1, warmup=0)
        cpu = {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample}

    line = {
        "metric": "fp8_gemm_tflops",
        "value": value,
        "unit": "TFLOP/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": ms_per_step,
        "higher_is_better": True,
        "scaling": "strong",
        "vs_baseline": None,
        "dtype": "fp8_e4m3 x fp8_e4m3 -> f32 accumulate -> bf16" if in_dtype == "fp8" else "s8 x s8 -> s32 -> bf16",
        "data": "synthetic",
        "config": {
            "workload": workload,
            "M": m, "N": n, "K": k, "n_per_gpu": nl, "in_dtype": in_dtype, "out_dtype": "bf16",
            "parallelism": f"column-parallel x{world} (no collective on the data path)",
            "l2": "operands per GPU exceed L2 (126 MB); no flush needed",
            "per_gpu_tflops": value / world,
            "per_gpu_frac_of_nominal_fp8_4500": value / world / NOMINAL_FP8_TFLOPS,
            "variant_hint": args.hint,
            "parity_check": parity,
        },
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms, "steps": e2e_steps,
                "note": "bytes per rank; on several GPUs a rank uploads 1/world of the activations and NCCL all-gathers them"},
        "gpu_launches": args.steps,
        "untimed_steps_before": args.warmup + 1 + preroll,
        "clocks": clocks,
        "roofline": roofline,
        "cpu_baseline": cpu,
        "device_status": status,
    }
    if gathered:
        line["with_allgather"] = gathered
    if fused:
        line["with_fused_allgather"] = fused
    if extras:
        line["extras"] = extras
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if parity is not None and not parity["ok"]:
        sys.exit(3)


if __name__ == "__main__":
    main()
