"""TEST INFRASTRUCTURE — CPU restatement of the reference's definition of the
two-stage mixture-of-experts GEMM.  Only tests, the smoke check and the
benchmark's CPU-baseline leg may import this module; the product never does.

Parity status: PINNED.  ``tests/golden/moe_*.npz`` were produced by the
reference's own torch functions (``torch_moe_gemm1`` / ``torch_moe_gemm2`` in
tests/kernels/test_ref.py:91-260 and ``_moe_sorting_torch_native`` in
tests/kernels/test_moe_gemm_2stage.py:99-137) run on CPU by
``tests/golden/make_golden_moe.py``; ``tests/test_moe_oracle_golden.py`` checks
every function below against them.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

QUANT_DTYPES = {"fp8": torch.float8_e4m3fn, "int8": torch.int8, "int4": torch.int8}  # int4 = W4A8: int8 activations


def moe_sorting(topk_ids, topk_weights, num_experts, block_size):
    """Routing table, expert by expert (tests/kernels/test_moe_gemm_2stage.py:99-137):
    returns (sorted_ids, sorted_weights, sorted_expert_ids, num_tokens_post_pad).
    Padding entries of sorted_weights are zero here (uninitialised in the reference)."""
    tokens, topk = topk_ids.shape
    max_padded = int(topk_ids.numel() + num_experts * block_size - topk)
    max_blocks = (max_padded + block_size - 1) // block_size
    sorted_ids = torch.full((max_padded,), (topk << 24) | tokens, dtype=torch.int32)
    sorted_weights = torch.zeros((max_padded,), dtype=torch.float32)
    sorted_expert_ids = torch.full((max_blocks,), -1, dtype=torch.int32)
    row, blk = 0, 0
    for e in range(num_experts):
        token_id, slot_id = torch.where(topk_ids == e)  # ascending (token, slot)
        n = int(token_id.numel())
        nblk = (n + block_size - 1) // block_size
        sorted_ids[row : row + n] = (slot_id.to(torch.int32) << 24) | token_id.to(torch.int32)
        sorted_weights[row : row + n] = topk_weights[token_id, slot_id].to(torch.float32)
        sorted_expert_ids[blk : blk + nblk] = e
        row += nblk * block_size
        blk += nblk
    return sorted_ids, sorted_weights, sorted_expert_ids, torch.tensor([row, tokens], dtype=torch.int32)


def _dequant(x_q, scale):
    """tests/kernels/test_ref.py:77-88, the per-token / per-row scalar-scale case."""
    return x_q.to(torch.float32) * scale


def moe_gemm1(x_q, w1_q_flat, scale_x, scale_w1_flat, topk_ids, topk_weights, inter_dim, doweight_stage1=False):
    """[tokens, topk, inter_dim] fp32: silu(gate) * up per routed (token, slot)
    (tests/kernels/test_ref.py:91-162)."""
    tokens, topk = topk_ids.shape
    model_dim = x_q.shape[-1]
    experts = w1_q_flat.shape[0] // (2 * inter_dim)
    x = _dequant(x_q, scale_x)  # [tokens, K], or [tokens, topk, K] with one activation row per route
    w1 = _dequant(w1_q_flat, scale_w1_flat).view(experts, 2 * inter_dim, model_dim)
    out = torch.zeros((tokens, topk, inter_dim), dtype=torch.float32)
    for e in range(experts):
        idx = (topk_ids == e).nonzero(as_tuple=False)
        if idx.numel() == 0:
            continue
        t_idx, s_idx = idx[:, 0], idx[:, 1]
        y2 = F.linear(x[t_idx, :] if x.dim() == 2 else x[t_idx, s_idx, :], w1[e])
        y = F.silu(y2[:, :inter_dim]) * y2[:, inter_dim:]
        if doweight_stage1:
            y = y * topk_weights[t_idx, s_idx].unsqueeze(-1)
        out[t_idx, s_idx, :] = y
    return out


def moe_gemm2(a2_q, w2_q, scale_a2, scale_w2, topk_ids, topk_weights, model_dim, doweight_stage2=True):
    """[tokens, model_dim] fp32: down projection of every routed row, summed over
    the top-k slots (tests/kernels/test_ref.py:165-260).  a2_q is [tokens, topk, inter_dim]."""
    tokens, topk = topk_ids.shape
    inter_dim = a2_q.shape[-1]
    experts = w2_q.shape[0] if w2_q.dim() == 3 else w2_q.shape[0] // model_dim
    a2 = _dequant(a2_q, scale_a2)
    w2 = _dequant(w2_q, scale_w2).view(experts, model_dim, inter_dim)
    out = torch.zeros((tokens, model_dim), dtype=torch.float32)
    for e in range(experts):
        idx = (topk_ids == e).nonzero(as_tuple=False)
        if idx.numel() == 0:
            continue
        t_idx, s_idx = idx[:, 0], idx[:, 1]
        y = F.linear(a2[t_idx, s_idx, :], w2[e])
        if doweight_stage2:
            y = y * topk_weights[t_idx, s_idx].unsqueeze(-1)
        out.index_add_(0, t_idx, y)
    return out


def moe_gemm2_per_slot(a2_q, w2_q, scale_a2, scale_w2, topk_ids, topk_weights, model_dim, doweight_stage2=True):
    """[tokens, topk, model_dim] fp32: the rows stage 2 writes with accumulate=False,
    before the top-k reduction (same arithmetic as moe_gemm2 without the final sum)."""
    tokens, topk = topk_ids.shape
    inter_dim = a2_q.shape[-1]
    experts = w2_q.shape[0] if w2_q.dim() == 3 else w2_q.shape[0] // model_dim
    a2 = _dequant(a2_q, scale_a2)
    w2 = _dequant(w2_q, scale_w2).view(experts, model_dim, inter_dim)
    out = torch.zeros((tokens, topk, model_dim), dtype=torch.float32)
    for e in range(experts):
        idx = (topk_ids == e).nonzero(as_tuple=False)
        if idx.numel() == 0:
            continue
        t_idx, s_idx = idx[:, 0], idx[:, 1]
        y = F.linear(a2[t_idx, s_idx, :], w2[e])
        if doweight_stage2:
            y = y * topk_weights[t_idx, s_idx].unsqueeze(-1)
        out[t_idx, s_idx, :] = y
    return out


def cosine_sim(a, b):
    """tests/kernels/test_moe_gemm_2stage.py:82-88."""
    a = a.to(torch.float32).flatten()
    b = b.to(torch.float32).flatten()
    return float(torch.dot(a, b) / (a.norm() * b.norm() + 1e-12))


def pertoken_quant(x, quant_dtype, dtype_max=None):
    """tests/utils.py:29-73 for finite inputs (the general restatement is in a8w8_oracle).  ``dtype_max=7``
    quantises to the signed 4-bit range held in int8, as the reference's W4A8 tests do
    (tests/kernels/test_moe_gemm_2stage.py:214-215)."""
    qmax = float(dtype_max) if dtype_max is not None else (448.0 if quant_dtype == torch.float8_e4m3fn else 127.0)
    amax = x.abs().amax(dim=-1, keepdim=True).to(torch.float32)
    scale = amax / qmax
    scale = torch.where(scale == 0, torch.ones_like(scale), scale)
    return (x / scale).to(quant_dtype), scale


def smooth_stage1_inputs(x, w1, topk_ids, generator):
    """Per-route ("int8smooth") stage-1 activations as the reference's test builds them
    (tests/kernels/test_moe_gemm_2stage.py:487-519): x times a per-expert smoothing vector,
    quantised per (token, slot).  Returns the token-major tensors the torch definition takes
    and the slot-major ones the kernel takes."""
    tokens, model_dim = x.shape
    topk = topk_ids.shape[1]
    experts = w1.shape[0]
    smooth = 0.75 + 0.5 * torch.rand((experts, model_dim), generator=generator, dtype=torch.float32)
    x_route = x[:, None, :].expand(tokens, topk, model_dim) * smooth[topk_ids.to(torch.int64)]
    amax = torch.amax(torch.abs(x_route), dim=-1, keepdim=True)
    scale_x = amax / 127.0
    scale_x[scale_x == 0] = 1.0
    x_q = (x_route / scale_x).to(torch.int8)
    return dict(
        x_ref=x_q.contiguous(), sx_ref=scale_x.contiguous(),
        x_slot_major=x_q.permute(1, 0, 2).contiguous().view(tokens * topk, model_dim),
        sx_slot_major=scale_x.permute(1, 0, 2).contiguous().view(-1),
    )


def make_routing(tokens, experts, topk, generator):
    """Scores -> top-k -> softmax weights (tests/kernels/test_moe_gemm_2stage.py:152-158), seeded on CPU."""
    score = torch.rand((tokens, experts), generator=generator, dtype=torch.float32)
    vals, ids = torch.topk(score, k=topk, dim=1)
    return ids.to(torch.int32), torch.softmax(vals, dim=1).to(torch.float32)


def make_inputs(tokens, model_dim, inter_dim, experts, topk, in_dtype, seed):
    """Seeded inputs of both stages with the recipe of the reference's tests
    (tests/kernels/test_moe_gemm_2stage.py:196-215, 268-325): unit-variance x,
    weights scaled by 1/sqrt(fan-in), per-token / per-row quantisation; the
    stage-2 input is the quantised stage-1 reference output."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    qd = QUANT_DTYPES[in_dtype]
    topk_ids, topk_weights = make_routing(tokens, experts, topk, g)
    x = torch.randn((tokens, model_dim), generator=g, dtype=torch.float32)
    w1 = torch.randn((experts, 2 * inter_dim, model_dim), generator=g, dtype=torch.float32) / math.sqrt(model_dim)
    w2 = torch.randn((experts, model_dim, inter_dim), generator=g, dtype=torch.float32) / math.sqrt(inter_dim)
    x_q, scale_x = pertoken_quant(x, qd)
    wmax = 7 if in_dtype == "int4" else None  # W4A8: weights in [-8, 7]
    w1_q, scale_w1 = pertoken_quant(w1, qd, wmax)
    w2_q, scale_w2 = pertoken_quant(w2, qd, wmax)
    out1 = moe_gemm1(
        x_q, w1_q.view(experts * 2 * inter_dim, model_dim), scale_x, scale_w1.view(-1, 1), topk_ids.long(), topk_weights,
        inter_dim, False,
    )
    a2_q, scale_a2 = pertoken_quant(out1, qd)
    return dict(
        topk_ids=topk_ids, topk_weights=topk_weights, x_q=x_q, scale_x=scale_x, w1_q=w1_q, scale_w1=scale_w1,
        w2_q=w2_q, scale_w2=scale_w2, out1=out1, a2_q=a2_q, scale_a2=scale_a2,
    )
