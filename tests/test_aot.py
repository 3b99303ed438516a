"""The ahead-of-time step (flydsl_b200.aot), after the reference's tests/python/examples/aot_example.py."""

import json
import os

import pytest
import torch

from flydsl_b200 import aot, compile_preshuffle_gemm


def test_compile_only_call_with_cpu_placeholders(monkeypatch):
    """COMPILE_ONLY=1 + CPU dummies, exactly the reference's pre-compilation call: nothing is launched,
    the prebuilt variant of the configuration is resolved."""
    fn = compile_preshuffle_gemm(N=8192, K=8192, tile_m=16, tile_n=64, tile_k=256, in_dtype="int8")
    plan = aot.precompile(fn, 32, 8192, 8192, "int8")
    assert plan["kernel"] == 1 and plan["bn"] == 32 and plan["split_k"] == 2 and plan["reduce"] == 2
    assert os.environ.get("COMPILE_ONLY") is None  # restored
    assert aot.precompile(fn, 4096, 8192, 8192, "int8")["kernel"] == 2
    # without COMPILE_ONLY the same CPU tensors are refused: there is no CPU path
    with pytest.raises(ValueError):
        fn(torch.zeros(1, dtype=torch.bfloat16), torch.zeros(1, dtype=torch.int8), torch.zeros(1, dtype=torch.int8),
           torch.zeros(1), torch.zeros(1), torch.empty(0, dtype=torch.bfloat16), 32, 8192, 0)


def test_manifest(tmp_path):
    out = tmp_path / "manifest.json"
    m = aot.main(["--configs", "5120,8192,16,fp8", "4096,4096,128,bf16", "--manifest", str(out)])
    on_disk = json.loads(out.read_text())
    assert on_disk["arch"] == "sm_100a" and len(on_disk["configs"]) == 2
    assert on_disk["configs"] == m["configs"]
    assert on_disk["configs"][0]["variant"]["kernel"] == 1


@pytest.mark.gpu
def test_manifest_with_kernel_runs():
    m = aot.main(["--configs", "1024,2048,16,fp8", "1024,2048,300,int8", "512,1024,64,bf16", "--run_kernel"])
    assert all(c["max_rel_error"] <= 2e-2 for c in m["configs"])
