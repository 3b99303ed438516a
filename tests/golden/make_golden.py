"""Generate the golden fixtures in this directory from the reference's own code.

Run once, in a container where the reference checkout is mounted:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's pure-torch helper module ``tests/utils.py`` by file
path (the reference's GPU kernel cannot run here; its helpers and its torch
check can), feeds it seeded inputs and stores inputs and outputs as small
``.npz`` files.  The test-suite then checks the oracle and the shipped host
helpers against these files without needing the reference.

Fixtures written:
  quant_fp8.npz / quant_int8.npz   pertoken_quant (tests/utils.py:29-73) incl.
                                   zero rows, NaN/Inf inputs, amax ties
  shuffle_ref_i8.npz / _f16.npz    shuffle_weight (tests/utils.py:76-96)
  gemm_fp8.npz / gemm_int8.npz     quantise -> dequantise-and-matmul check
                                   (tests/kernels/test_preshuffle_gemm.py:103-113,
                                   formula applied to the reference helper's outputs)
"""

import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_ref_utils(ref_root):
    path = os.path.join(ref_root, "tests", "utils.py")
    spec = importlib.util.spec_from_file_location("_ref_tests_utils", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def u8(t):
    return t.contiguous().view(torch.uint8).numpy()


def main(ref_root):
    ref = load_ref_utils(ref_root)
    g = torch.Generator(device="cpu").manual_seed(20240611)

    # --- quantiser ---------------------------------------------------------
    x = torch.randn(37, 256, generator=g, dtype=torch.float32) * 3.0
    x[3] = 0.0  # zero row -> scale 1
    x[5, 7] = float("nan")
    x[6, 9] = float("inf")
    x[7, 11] = float("-inf")
    x[8] = x[8].abs()  # all-positive row
    x[9] = -x[9].abs()  # all-negative row
    for name, qd in (("fp8", torch.float8_e4m3fn), ("int8", torch.int8)):
        y, s = ref.pertoken_quant(x, quant_dtype=qd)
        np.savez_compressed(os.path.join(HERE, f"quant_{name}.npz"), x=x.numpy(), y=u8(y), scale=s.numpy())

    # --- reference weight layout ------------------------------------------
    w8 = torch.randint(-128, 128, (64, 256), generator=g, dtype=torch.int32).to(torch.int8)
    np.savez_compressed(
        os.path.join(HERE, "shuffle_ref_i8.npz"), x=w8.numpy(), y=ref.shuffle_weight(w8, layout=(16, 16)).numpy()
    )
    w16 = torch.randn(32, 128, generator=g, dtype=torch.float32).to(torch.float16)
    np.savez_compressed(
        os.path.join(HERE, "shuffle_ref_f16.npz"),
        x=u8(w16),
        y=u8(ref.shuffle_weight(w16, layout=(16, 16))),
    )

    # --- quantise + dequantise-and-matmul ------------------------------------
    m, n, k = 19, 48, 256
    a = torch.randn(m, k, generator=g, dtype=torch.float32)
    w = torch.randn(n, k, generator=g, dtype=torch.float32)
    for name, qd in (("fp8", torch.float8_e4m3fn), ("int8", torch.int8)):
        a_q, sa = ref.pertoken_quant(a, quant_dtype=qd)
        b_q, sb = ref.pertoken_quant(w, quant_dtype=qd)
        a_f = a_q.to(torch.float32) * sa.view(-1, 1)
        b_f = b_q.to(torch.float32) * sb.view(-1, 1)
        c = torch.mm(a_f, b_f.T)
        extra = {}
        if name == "int8":
            extra["acc"] = (a_q.to(torch.int32) @ b_q.to(torch.int32).T).numpy()
        np.savez_compressed(
            os.path.join(HERE, f"gemm_{name}.npz"),
            a=a.numpy(),
            w=w.numpy(),
            a_q=u8(a_q),
            b_q=u8(b_q),
            sa=sa.numpy(),
            sb=sb.numpy(),
            c=c.numpy(),
            b_shuf_ref=u8(ref.shuffle_weight(b_q, layout=(16, 16))),
            **extra,
        )
    print("wrote fixtures to", HERE)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <reference checkout>")
    main(sys.argv[1])
