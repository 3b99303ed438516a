"""Generate the MXFP6-activation golden fixture from the reference's own utilities.

    python tests/golden/make_golden_mx6.py /path/to/reference

Imports tests/kernels/utils/gemm_common_utils.py of the reference by file path and stores seeded
inputs with the outputs of ``per_1x32_f6_quant`` (padded packed codes, scales, unpacked codes),
``fp6_e2m3_to_f32`` on all 64 codes, the E2M3 code of a sweep through every rounding boundary,
``per_1x32_f4_quant`` of the weights and the A6W4 reference of
tests/kernels/test_preshuffle_gemm.py:530-538.

Fixture written:  mx_fp6.npz
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
    g = torch.Generator(device="cpu").manual_seed(20241109)
    m, n, k = 40, 48, 256
    a = torch.randn(m, k, generator=g, dtype=torch.float32)
    b = torch.randn(n, k, generator=g, dtype=torch.float32)
    a[3] = 0.0
    a[5, :32] *= 1e-20
    a[6, 32:64] *= 1e5
    a_pad, sa, a_codes = ref.per_1x32_f6_quant(a)
    b_q, sb, _ = ref.per_1x32_f4_quant(b)
    b_q, sa, sb = b_q.view(torch.uint8), sa.view(torch.uint8), sb.view(torch.uint8)
    a_deq = ref.fp6_e2m3_to_f32(a_codes) * ref.e8m0_to_f32(sa.repeat_interleave(32, dim=1))
    b_deq = ref.mxfp4_to_f32(b_q.clone()) * ref.e8m0_to_f32(sb.repeat_interleave(32, dim=1))
    c = torch.mm(a_deq, b_deq.T).to(torch.float32)
    vals = ref.fp6_e2m3_to_f32(torch.arange(32, dtype=torch.uint8))
    mids = (vals[:-1] + vals[1:]) / 2
    base = torch.cat([vals, mids, torch.tensor([7.5, 7.75, 8.0, 100.0])])
    probe = torch.cat([base, torch.nextafter(base, torch.tensor(1000.0)), torch.nextafter(base, torch.tensor(-1000.0))])
    probe = torch.cat([probe, -probe])
    probe_codes = ref._f32_to_floatx_unpacked(probe.clone(), 2, 3)
    np.savez_compressed(
        os.path.join(HERE, "mx_fp6.npz"),
        a=a.numpy(), b=b.numpy(), a_pad=a_pad.numpy(), a_codes=a_codes.numpy(), sa=sa.numpy(), b_q=b_q.numpy(), sb=sb.numpy(),
        c=c.numpy(), probe=probe.numpy(), probe_codes=probe_codes.numpy(),
        table=ref.fp6_e2m3_to_f32(torch.arange(64, dtype=torch.uint8)).numpy(),
    )
    print("written: a_pad", tuple(a_pad.shape), "c", tuple(c.shape), "probe", probe.numel())


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden_mx6.py /path/to/reference")
    main(sys.argv[1])
