"""Generate the MXFP8 golden fixture from the reference's own utilities.

    python tests/golden/make_golden_mx.py /path/to/reference

Imports tests/kernels/utils/gemm_common_utils.py of the reference by file path
(pure torch for the functions used here) and stores seeded inputs with the
outputs of ``per_1x32_f8_quant``, ``e8m0_to_f32`` and the dequantise-and-matmul
reference of tests/kernels/test_preshuffle_gemm.py:651-654.

Fixture written:  mx_fp8.npz
"""

import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def main(ref_root):
    path = os.path.join(ref_root, "tests", "kernels", "utils", "gemm_common_utils.py")
    spec = importlib.util.spec_from_file_location("_ref_gemm_common_utils", path)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    g = torch.Generator(device="cpu").manual_seed(20241105)
    m, n, k = 40, 48, 256
    a = torch.randn(m, k, generator=g, dtype=torch.float32)
    b = torch.randn(n, k, generator=g, dtype=torch.float32)
    a[3] = 0.0  # an all-zero row: clamp_min path
    a[5, :32] *= 1e-20  # a tiny block
    b[7, 32:64] *= 1e6  # a huge block
    a_q, sa = ref.per_1x32_f8_quant(a)
    b_q, sb = ref.per_1x32_f8_quant(b)
    a_deq = a_q.float() * ref.e8m0_to_f32(sa.repeat_interleave(32, dim=1))
    b_deq = b_q.float() * ref.e8m0_to_f32(sb.repeat_interleave(32, dim=1))
    c = torch.mm(a_deq, b_deq.T).to(torch.float32)
    all_bytes = torch.arange(256, dtype=torch.uint8)
    np.savez_compressed(
        os.path.join(HERE, "mx_fp8.npz"),
        a=a.numpy(), b=b.numpy(), a_q=a_q.view(torch.uint8).numpy(), b_q=b_q.view(torch.uint8).numpy(),
        sa=sa.view(torch.uint8).numpy(), sb=sb.view(torch.uint8).numpy(), c=c.numpy(),
        e8m0_table=ref.e8m0_to_f32(all_bytes).view(torch.int32).numpy(),
    )
    print("written: a_q", tuple(a_q.shape), "sa", tuple(sa.shape), "c", tuple(c.shape))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden_mx.py /path/to/reference")
    main(sys.argv[1])
