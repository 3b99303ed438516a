"""Generate the mixture-of-experts golden fixtures from the reference's own code.

    python tests/golden/make_golden_moe.py /path/to/reference

The reference's torch definitions of the two stages (``torch_moe_gemm1`` /
``torch_moe_gemm2``, tests/kernels/test_ref.py:91-260) are imported by file
path and run on CPU.  They are written for a GPU box in two places only: the
result tensor is created with ``device="cuda"`` and stage 2 asserts
``is_cuda``; this script redirects the first to the CPU and wraps the inputs
in a tensor subclass that answers the second, changing nothing of the
arithmetic.  The routing-table builder ``_moe_sorting_torch_native``
(tests/kernels/test_moe_gemm_2stage.py:99-137) sits in a test module that
imports the reference's compiler at top level, so its source text is cut out
of the file and executed on its own.

Fixtures written (inputs seeded here, outputs from the reference):
  moe_fp8.npz / moe_int8.npz   routing table, quantised inputs of both stages,
                               stage-1 and stage-2 reference outputs; the int8 file
                               also holds per-route ("int8smooth") stage-1 activations
                               and their reference output
"""

import ast
import importlib.util
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


class OnGpuLookalike(torch.Tensor):
    """A CPU tensor that answers ``is_cuda`` with True."""

    @property
    def is_cuda(self):  # noqa: D401
        return True


def load_test_ref(ref_root):
    path = os.path.join(ref_root, "tests", "kernels", "test_ref.py")
    spec = importlib.util.spec_from_file_location("_ref_test_ref", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    real_zeros = torch.zeros

    class TorchOnCpu:
        """torch with zeros(..., device="cuda") created on the CPU."""

        def __getattr__(self, name):
            return getattr(torch, name)

        @staticmethod
        def zeros(*a, **k):
            k.pop("device", None)
            return real_zeros(*a, **k)

    mod.torch = TorchOnCpu()
    return mod


def load_sorting(ref_root):
    path = os.path.join(ref_root, "tests", "kernels", "test_moe_gemm_2stage.py")
    src = open(path).read()
    tree = ast.parse(src)
    fn = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "_moe_sorting_torch_native")
    ns = {"torch": torch, "Tuple": tuple}
    exec(compile(ast.Module(body=[fn], type_ignores=[]), path, "exec"), ns)
    return ns["_moe_sorting_torch_native"]


def pertoken_quant_ref(ref_root):
    path = os.path.join(ref_root, "tests", "utils.py")
    spec = importlib.util.spec_from_file_location("_ref_tests_utils", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.pertoken_quant


def u8(t):
    return t.contiguous().view(torch.uint8).numpy()


def main(ref_root):
    ref = load_test_ref(ref_root)
    sorting = load_sorting(ref_root)
    quant = pertoken_quant_ref(ref_root)
    tokens, model_dim, inter_dim, experts, topk, block = 24, 128, 64, 4, 2, 16
    for name, qd in (("fp8", torch.float8_e4m3fn), ("int8", torch.int8)):
        g = torch.Generator(device="cpu").manual_seed(20240917)
        score = torch.rand((tokens, experts), generator=g, dtype=torch.float32)
        vals, ids = torch.topk(score, k=topk, dim=1)
        topk_weights = torch.softmax(vals, dim=1).to(torch.float32)
        topk_ids = ids.to(torch.int32)
        x = torch.randn((tokens, model_dim), generator=g, dtype=torch.float32)
        w1 = torch.randn((experts, 2 * inter_dim, model_dim), generator=g, dtype=torch.float32) / math.sqrt(model_dim)
        w2 = torch.randn((experts, model_dim, inter_dim), generator=g, dtype=torch.float32) / math.sqrt(inter_dim)
        x_q, scale_x = quant(x, quant_dtype=qd)
        w1_q, scale_w1 = quant(w1, quant_dtype=qd)
        w2_q, scale_w2 = quant(w2, quant_dtype=qd)
        sorted_ids, sorted_w, sorted_e, post_pad = sorting(topk_ids, topk_weights, num_experts=experts, block_size=block)
        n_valid = int(post_pad[0])
        out1 = ref.torch_moe_gemm1(
            x_q, w1_q.view(experts * 2 * inter_dim, model_dim), scale_x, scale_w1.view(-1, 1), topk_ids.to(torch.int64),
            topk_weights, inter_dim=inter_dim, doweight_stage1=False,
        )
        out1_w = ref.torch_moe_gemm1(
            x_q, w1_q.view(experts * 2 * inter_dim, model_dim), scale_x, scale_w1.view(-1, 1), topk_ids.to(torch.int64),
            topk_weights, inter_dim=inter_dim, doweight_stage1=True,
        )
        a2_q, scale_a2 = quant(out1, quant_dtype=qd)
        out2 = ref.torch_moe_gemm2(
            a2_q.as_subclass(OnGpuLookalike), w2_q.as_subclass(OnGpuLookalike), scale_a2, scale_w2,
            topk_ids.to(torch.int64), topk_weights, model_dim=model_dim, doweight_stage2=True,
        )
        out2_nw = ref.torch_moe_gemm2(
            a2_q.as_subclass(OnGpuLookalike), w2_q.as_subclass(OnGpuLookalike), scale_a2, scale_w2,
            topk_ids.to(torch.int64), topk_weights, model_dim=model_dim, doweight_stage2=False,
        )
        extra = {}
        if name == "int8":
            # per-route activations (token-major [tokens, topk, K]) as in the reference's int8smooth test
            smooth = 0.75 + 0.5 * torch.rand((experts, model_dim), generator=g, dtype=torch.float32)
            x_route = x[:, None, :].expand(tokens, topk, model_dim) * smooth[topk_ids.to(torch.int64)]
            sx_r = torch.amax(torch.abs(x_route), dim=-1, keepdim=True) / 127.0
            sx_r[sx_r == 0] = 1.0
            xq_r = (x_route / sx_r).to(torch.int8)
            out1_r = ref.torch_moe_gemm1(
                xq_r, w1_q.view(experts * 2 * inter_dim, model_dim), sx_r, scale_w1.view(-1, 1), topk_ids.to(torch.int64),
                topk_weights, inter_dim=inter_dim, doweight_stage1=False,
            )
            extra = dict(x_route_q=u8(xq_r), scale_x_route=sx_r.numpy(), out1_route=out1_r.numpy())
        np.savez_compressed(
            os.path.join(HERE, f"moe_{name}.npz"),
            dims=np.array([tokens, model_dim, inter_dim, experts, topk, block], dtype=np.int64),
            topk_ids=topk_ids.numpy(), topk_weights=topk_weights.numpy(),
            sorted_ids=sorted_ids.numpy(), sorted_weights_valid=sorted_w.numpy()[:n_valid] * (sorted_ids.numpy()[:n_valid] & 0xFFFFFF < tokens),
            sorted_expert_ids=sorted_e.numpy(), post_pad=post_pad.numpy(),
            x_q=u8(x_q), scale_x=scale_x.numpy(), w1_q=u8(w1_q), scale_w1=scale_w1.numpy(),
            w2_q=u8(w2_q), scale_w2=scale_w2.numpy(), a2_q=u8(a2_q), scale_a2=scale_a2.numpy(),
            out1=out1.numpy(), out1_weighted=out1_w.numpy(),
            out2=out2.as_subclass(torch.Tensor).numpy(), out2_unweighted=out2_nw.as_subclass(torch.Tensor).numpy(),
            **extra,
        )
        print(name, "written: out1", tuple(out1.shape), "out2", tuple(out2.shape), "rows in use", n_valid)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden_moe.py /path/to/reference")
    main(sys.argv[1])
