"""Build libflyb200.so (CUDA kernels + C ABI) in-tree for sm_100a.

    python -m flydsl_b200.build [--force] [-v]

nvcc cross-compiles without a GPU.  The library is written next to its
sources so that a snapshot of the tree carries it to the GPU machine.  Every
translation unit is compiled to an object file of its own (in parallel, and
only when it is older than what it includes), then the objects are linked.
Concurrent callers (the ranks of a multi-process run that all find the
library missing) are serialised by a file lock; the loser of the race finds a
fresh library and builds nothing.
"""

from __future__ import annotations

import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

CSRC = os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc")
LIB_PATH = os.path.join(CSRC, "libflyb200.so")
STAMP_PATH = os.path.join(CSRC, "libflyb200.stamp")  # digest of the inputs the library was built from
OBJ_DIR = os.path.join(CSRC, "build")
SOURCES = [
    "flyb200.cu",
    "flyb200_rows.cu",
    "flyb200_decode.cu",
    "flyb200_decode_wide.cu",
    "flyb200_decode2.cu",
    "flyb200_moe.cu",
    "flyb200_mx.cu",
]
HEADERS = [
    "ptx.cuh",
    "gemm_kernels.cuh",
    "decode_kernel.cuh",
    "rows2_kernel.cuh",
    "rows_tall_kernel.cuh",
    "decode2_kernel.cuh",
    "quant_kernel.cuh",
    "moe_kernel.cuh",
    "mx_kernel.cuh",
    "launch.h",
    "decode_launch.h",
    "host_common.h",
    os.path.join("..", "..", "include", "flyb200.h"),
]

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-Xcompiler",
    "-fPIC",
]


def find_nvcc() -> str | None:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    if os.path.exists(cand):
        return cand
    return shutil.which("nvcc")


def _input_digest() -> str:
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    for f in SOURCES + HEADERS:
        p = os.path.join(CSRC, f)
        h.update(f.encode())
        if os.path.exists(p):
            with open(p, "rb") as fh:
                h.update(fh.read())
    return h.hexdigest()


def is_stale() -> bool:
    """The library is current when the digest of its inputs matches the stamp
    written at build time (file times do not survive a copy of the tree)."""
    if not os.path.exists(LIB_PATH) or not os.path.exists(STAMP_PATH):
        return True
    with open(STAMP_PATH) as fh:
        return fh.read().strip() != _input_digest()


def _object_stale(src: str, obj: str) -> bool:
    if not os.path.exists(obj):
        return True
    built = os.path.getmtime(obj)
    if os.path.getmtime(os.path.join(CSRC, src)) > built:
        return True
    # headers are shared by all translation units: any newer header rebuilds everything
    return any(
        os.path.exists(os.path.join(CSRC, h)) and os.path.getmtime(os.path.join(CSRC, h)) > built for h in HEADERS
    )


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if it is missing or older than its sources."""
    if not force and not is_stale():
        return LIB_PATH
    nvcc = find_nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build libflyb200.so")
    os.makedirs(OBJ_DIR, exist_ok=True)
    with open(os.path.join(OBJ_DIR, ".lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and not is_stale():  # another process built it while this one waited
                return LIB_PATH
            todo = []
            for src in SOURCES:
                obj = os.path.join(OBJ_DIR, src[:-3] + ".o")
                if force or _object_stale(src, obj):
                    todo.append((src, obj))

            def compile_one(item):
                src, obj = item
                cmd = [nvcc, *NVCC_FLAGS, "-c", "-o", obj + f".{os.getpid()}.tmp", src]
                if verbose:
                    cmd[1:1] = ["-Xptxas", "-v"]
                res = subprocess.run(cmd, cwd=CSRC, capture_output=True, text=True)
                if res.returncode != 0:
                    raise RuntimeError(f"nvcc failed on {src} ({res.returncode}):\n{res.stdout}\n{res.stderr}")
                os.replace(obj + f".{os.getpid()}.tmp", obj)
                return res.stderr

            with ThreadPoolExecutor(max_workers=min(len(todo), os.cpu_count() or 1) or 1) as pool:
                logs = list(pool.map(compile_one, todo))
            if verbose:
                print("\n".join(logs))
            objs = [os.path.join(OBJ_DIR, s[:-3] + ".o") for s in SOURCES]
            tmp = LIB_PATH + f".{os.getpid()}.tmp"
            res = subprocess.run([nvcc, "-shared", "-o", tmp, *objs, "-lcudart"], cwd=CSRC, capture_output=True,
                                 text=True)
            if res.returncode != 0:
                raise RuntimeError(f"link failed ({res.returncode}):\n{res.stdout}\n{res.stderr}")
            os.replace(tmp, LIB_PATH)
            with open(STAMP_PATH + f".{os.getpid()}.tmp", "w") as fh:
                fh.write(_input_digest() + "\n")
            os.replace(STAMP_PATH + f".{os.getpid()}.tmp", STAMP_PATH)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return LIB_PATH


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
