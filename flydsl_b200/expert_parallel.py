"""Expert-parallel use of the two-stage mixture-of-experts GEMM across the GPUs
of one machine.

The experts are split into contiguous, equal groups, one per rank; every rank
holds the activations and the router's choice (replicated) and the weights of
its own experts only.  A rank builds the routing table of the routes that go
to ITS experts (the others are dropped by the sort), runs stage 1, the
per-token quantiser and stage 2 (accumulating into ``[tokens, model_dim]``) on
them, and the partial outputs of the ranks are summed with one NCCL
all-reduce: the path has a real exchange step, because a token's top-k experts
live on different ranks.

The reference has no multi-GPU form of these kernels (its expert-parallel hook
is the expert mask of the top-k reduction, kernels/moe/moe_gemm_2stage/moe_reduce.py:164-205);
one process per GPU as in tests/kernels/test_allreduce.py:267,629-644.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from .column_parallel import check_agreement


@dataclass(frozen=True)
class ExpertShard:
    experts_total: int
    world: int
    rank: int

    @property
    def experts_local(self) -> int:
        return self.experts_total // self.world

    @property
    def e0(self) -> int:
        return self.rank * self.experts_local

    @property
    def e1(self) -> int:
        return self.e0 + self.experts_local


def expert_shard(experts_total: int, world: int, rank: int) -> ExpertShard:
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world: {rank}/{world}")
    if experts_total % world != 0:
        raise ValueError(f"{experts_total} experts cannot be split evenly over {world} ranks")
    return ExpertShard(experts_total, world, rank)


def local_routing(topk_ids: torch.Tensor, shard: ExpertShard) -> torch.Tensor:
    """The router's choice in the numbering of this rank's experts: expert e of
    the shard becomes e - e0, every other expert becomes -1 (which the routing
    sort ignores).  Works on CPU and CUDA tensors."""
    local = topk_ids.to(torch.int32) - shard.e0
    return torch.where((local >= 0) & (local < shard.experts_local), local, torch.full_like(local, -1))


class ExpertParallelMoe:
    """One rank's part of an expert-parallel MoE layer (fp8 or int8 weights)."""

    def __init__(self, *, model_dim, inter_dim, experts, topk, tile_m=64, in_dtype="fp8", rank=None, world=None, group=None):
        from .kernels.moe.moe_gemm_2stage import compile_moe_gemm1, compile_moe_gemm2

        self.group = group
        self.rank = dist.get_rank(group) if rank is None else rank
        self.world = dist.get_world_size(group) if world is None else world
        self.shard = expert_shard(experts, self.world, self.rank)
        self.model_dim, self.inter_dim, self.topk, self.tile_m, self.in_dtype = model_dim, inter_dim, topk, tile_m, in_dtype
        kw = dict(model_dim=model_dim, inter_dim=inter_dim, experts=self.shard.experts_local, topk=topk, tile_m=tile_m,
                  tile_n=128, tile_k=128, in_dtype=in_dtype)
        self._g1 = compile_moe_gemm1(**kw, doweight_stage1=False, out_dtype="bf16")
        self._g2 = compile_moe_gemm2(**kw, doweight_stage2=True, out_dtype="f32", accumulate=True)
        self._w1 = self._w2 = self._sw1 = self._sw2 = None

    def describe(self) -> dict:
        return dict(model_dim=self.model_dim, inter_dim=self.inter_dim, experts=self.shard.experts_total, topk=self.topk,
                    tile_m=self.tile_m, in_dtype=self.in_dtype, world=self.world)

    def load_expert_weights(self, w1_q, scale_w1, w2_q, scale_w2):
        """Quantised weights of THIS rank's experts: w1 [E/w, 2*inter, model], w2 [E/w, model, inter]
        and their per-row scales; preshuffled here, expert by expert."""
        from . import shuffle_weight

        el = self.shard.experts_local
        if w1_q.shape != (el, 2 * self.inter_dim, self.model_dim) or w2_q.shape != (el, self.model_dim, self.inter_dim):
            raise ValueError("weight shapes do not match this rank's expert shard")
        self._w1, self._w2 = shuffle_weight(w1_q), shuffle_weight(w2_q)
        self._sw1 = scale_w1.reshape(-1).float().contiguous()
        self._sw2 = scale_w2.reshape(-1).float().contiguous()

    def forward_local(self, x_q, scale_x, topk_ids, topk_weights):
        """This rank's partial output [tokens, model_dim] fp32 (routes to other ranks' experts contribute nothing)."""
        from . import pertoken_quant
        from .kernels.moe.moe_gemm_2stage import moe_sorting

        if self._w1 is None:
            raise RuntimeError("load_expert_weights has not been called")
        tokens = x_q.shape[0]
        dev = x_q.device
        ids = local_routing(topk_ids, self.shard)
        srt, wts, e_ids, post = moe_sorting(ids, topk_weights, num_experts=self.shard.experts_local, block_size=self.tile_m)
        blocks = int(e_ids.numel())
        st = torch.cuda.current_stream(dev)
        # rows of routes that belong to other ranks are never written nor read: zero keeps the quantiser finite
        out1 = torch.zeros(tokens * self.topk, self.inter_dim, dtype=torch.bfloat16, device=dev)
        self._g1(out1, x_q.reshape(-1), self._w1.reshape(-1), scale_x.reshape(-1), self._sw1, srt, e_ids, wts, post, tokens,
                 self.inter_dim, self.model_dim, blocks, st)
        qd = torch.float8_e4m3fn if self.in_dtype == "fp8" else torch.int8
        a2, sa2 = pertoken_quant(out1, quant_dtype=qd)
        y = torch.zeros(tokens, self.model_dim, dtype=torch.float32, device=dev)
        self._g2(y, a2.reshape(-1), self._w2.reshape(-1), sa2.reshape(-1), self._sw2, srt, e_ids, wts, post, tokens,
                 self.model_dim, self.inter_dim, blocks, st)
        return y

    def forward(self, x_q, scale_x, topk_ids, topk_weights, handshake_group=None):
        """The layer's output [tokens, model_dim] fp32 on every rank: local part, then one all-reduce (sum)."""
        if handshake_group is not None:
            check_agreement(dict(self.describe(), tokens=int(x_q.shape[0])), group=handshake_group)
        y = self.forward_local(x_q, scale_x, topk_ids, topk_weights)
        if self.world > 1:
            dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
        return y
