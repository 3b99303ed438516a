"""Build libflyb200.so (CUDA kernels + C ABI) in-tree for sm_100a.

    python -m flydsl_b200.build [--force]

nvcc cross-compiles without a GPU.  The library is written next to its
sources so that a snapshot of the tree carries it to the GPU machine.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys

CSRC = os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc")
LIB_PATH = os.path.join(CSRC, "libflyb200.so")
SOURCES = ["flyb200.cu", "flyb200_moe.cu", "flyb200_mx.cu"]
HEADERS = ["ptx.cuh", "gemm_kernels.cuh", "decode_kernel.cuh", "rows2_kernel.cuh", "quant_kernel.cuh", "moe_kernel.cuh", "mx_kernel.cuh", "host_common.h", os.path.join("..", "..", "include", "flyb200.h")]

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-shared",
    "-Xcompiler",
    "-fPIC",
]


def find_nvcc() -> str | None:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    if os.path.exists(cand):
        return cand
    return shutil.which("nvcc")


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    for f in SOURCES + HEADERS:
        p = os.path.join(CSRC, f)
        if os.path.exists(p) and os.path.getmtime(p) > built:
            return True
    return False


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if it is missing or older than its sources."""
    if not force and not is_stale():
        return LIB_PATH
    nvcc = find_nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build libflyb200.so")
    cmd = [nvcc, *NVCC_FLAGS, "-o", LIB_PATH + ".tmp", *SOURCES]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, cwd=CSRC, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed ({res.returncode}):\n{res.stdout}\n{res.stderr}")
    os.replace(LIB_PATH + ".tmp", LIB_PATH)
    if verbose:
        print(res.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
