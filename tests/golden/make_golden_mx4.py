"""Generate the MXFP4 golden fixture from the reference's own utilities.

    python tests/golden/make_golden_mx4.py /path/to/reference

Imports tests/kernels/utils/gemm_common_utils.py of the reference by file path
and stores seeded inputs with the outputs of ``per_1x32_f4_quant``,
``mxfp4_to_f32`` and the dequantise-and-matmul reference of
tests/kernels/test_preshuffle_gemm.py:404-411, plus the E2M1 code of a sweep of
values around every rounding boundary.

Fixture written:  mx_fp4.npz
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
    g = torch.Generator(device="cpu").manual_seed(20241107)
    m, n, k = 40, 48, 256
    a = torch.randn(m, k, generator=g, dtype=torch.float32)
    b = torch.randn(n, k, generator=g, dtype=torch.float32)
    a[3] = 0.0  # an all-zero row
    a[5, :32] *= 1e-20  # a tiny block
    b[7, 32:64] *= 1e6  # a huge block
    a_q, sa, _ = ref.per_1x32_f4_quant(a)
    b_q, sb, _ = ref.per_1x32_f4_quant(b)
    a_q, b_q = a_q.view(torch.uint8), b_q.view(torch.uint8)
    sa, sb = sa.view(torch.uint8), sb.view(torch.uint8)
    a_deq = ref.mxfp4_to_f32(a_q.clone()) * ref.e8m0_to_f32(sa.repeat_interleave(32, dim=1))
    b_deq = ref.mxfp4_to_f32(b_q.clone()) * ref.e8m0_to_f32(sb.repeat_interleave(32, dim=1))
    c = torch.mm(a_deq, b_deq.T).to(torch.float32)
    # every rounding boundary of E2M1, its neighbours one ulp away, both signs, and values beyond the range
    mids = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, 0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 7.0, 100.0])
    probe = torch.cat([mids, torch.nextafter(mids, torch.tensor(10.0)), torch.nextafter(mids, torch.tensor(-10.0))])
    probe = torch.cat([probe, -probe])
    probe = probe[: probe.numel() // 2 * 2]
    probe_codes = ref._f32_to_floatx_unpacked(probe.clone(), 2, 1)
    np.savez_compressed(
        os.path.join(HERE, "mx_fp4.npz"),
        a=a.numpy(), b=b.numpy(), a_q=a_q.numpy(), b_q=b_q.numpy(), sa=sa.numpy(), sb=sb.numpy(), c=c.numpy(),
        probe=probe.numpy(), probe_codes=probe_codes.numpy(),
        table=ref.mxfp4_to_f32(torch.arange(256, dtype=torch.uint8).view(1, 256)).numpy(),
    )
    print("written: a_q", tuple(a_q.shape), "sa", tuple(sa.shape), "c", tuple(c.shape), "probe", probe.numel())


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden_mx4.py /path/to/reference")
    main(sys.argv[1])
