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

    def __init__(self, *, model_dim, inter_dim, experts, topk, tile_m=64, in_dtype="fp8", out_dtype="bf16", rank=None,
                 world=None, group=None):
        """``out_dtype`` "bf16": stage 2 writes one bf16 row per route, the rows of a token are summed
        (fp32, one rounding) and the ranks exchange bf16.  "f32": stage 2 accumulates with fp32 atomics
        into a zero-filled fp32 output and the ranks exchange fp32 (twice the bytes, no bf16 rounding
        between the partial sums)."""
        from .kernels.moe.moe_gemm_2stage import compile_moe_gemm1, compile_moe_gemm2, compile_moe_reduction

        if out_dtype not in ("bf16", "f32"):
            raise ValueError(f"out_dtype must be 'bf16' or 'f32', got {out_dtype!r}")
        self.out_dtype = out_dtype

        self.group = group
        self.rank = dist.get_rank(group) if rank is None else rank
        self.world = dist.get_world_size(group) if world is None else world
        self.shard = expert_shard(experts, self.world, self.rank)
        self.model_dim, self.inter_dim, self.topk, self.tile_m, self.in_dtype = model_dim, inter_dim, topk, tile_m, in_dtype
        kw = dict(model_dim=model_dim, inter_dim=inter_dim, experts=self.shard.experts_local, topk=topk, tile_m=tile_m,
                  tile_n=128, tile_k=128, in_dtype=in_dtype)
        self._g1 = compile_moe_gemm1(**kw, doweight_stage1=False, out_dtype="bf16")
        if out_dtype == "f32":
            self._g2 = compile_moe_gemm2(**kw, doweight_stage2=True, out_dtype="f32", accumulate=True)
        else:
            self._g2 = compile_moe_gemm2(**kw, doweight_stage2=True, out_dtype="bf16", accumulate=False)
            self._reduce = compile_moe_reduction(topk=topk, model_dim=model_dim, dtype_str="bf16", use_mask=True,
                                                 num_experts=experts)
            self._mask = None  # 1 for this rank's experts, built on first use on the layer's device
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
        """This rank's partial output [tokens, model_dim] (routes to other ranks' experts contribute nothing)."""
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
        if self.out_dtype == "f32":
            y = torch.zeros(tokens, self.model_dim, dtype=torch.float32, device=dev)
            self._g2(y, a2.reshape(-1), self._w2.reshape(-1), sa2.reshape(-1), self._sw2, srt, e_ids, wts, post, tokens,
                     self.model_dim, self.inter_dim, blocks, st)
            return y
        # rows of routes that belong to other ranks are never written; the masked reduction skips them
        out2 = torch.empty(tokens * self.topk, self.model_dim, dtype=torch.bfloat16, device=dev)
        self._g2(out2, a2.reshape(-1), self._w2.reshape(-1), sa2.reshape(-1), self._sw2, srt, e_ids, wts, post, tokens,
                 self.model_dim, self.inter_dim, blocks, st)
        if self._mask is None or self._mask.device != dev:
            mask = torch.zeros(self.shard.experts_total, dtype=torch.int32, device=dev)
            mask[self.shard.e0 : self.shard.e1] = 1
            self._mask = mask
        y = torch.empty(tokens, self.model_dim, dtype=torch.bfloat16, device=dev)
        self._reduce(out2, y, self._mask, topk_ids.to(torch.int32).contiguous(), tokens, st)
        return y

    def forward(self, x_q, scale_x, topk_ids, topk_weights, handshake_group=None):
        """The layer's output [tokens, model_dim] on every rank: local part, then one all-reduce (sum)."""
        if handshake_group is not None:
            check_agreement(dict(self.describe(), tokens=int(x_q.shape[0])), group=handshake_group)
        y = self.forward_local(x_q, scale_x, topk_ids, topk_weights)
        if self.world > 1:
            dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
        return y


def _bench_main():
    """Timing driver: ``python -m torch.distributed.run --nproc-per-node W -m flydsl_b200.expert_parallel
    [--tokens T]``: one rank per GPU, seeded synthetic weights and routing, device time of the whole
    layer (routing table, both stages, quantiser, all-reduce) as the max over ranks; rank 0 prints one JSON line."""
    import argparse
    import json
    import os

    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--model-dim", type=int, default=4096)
    ap.add_argument("--inter-dim", type=int, default=2048)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--topk", type=int, default=2)
    ap.add_argument("--tile-m", type=int, default=128)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--out-dtype", default="bf16", choices=["bf16", "f32"])
    ap.add_argument("--graph", action="store_true", help="one GPU only: capture the layer into one CUDA graph and time replays")
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    if a.graph and world > 1:
        # capturing the NCCL all-reduce of this layer did not complete on the test machine: single GPU only
        raise SystemExit("--graph times the single-GPU layer only")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    op = ExpertParallelMoe(model_dim=a.model_dim, inter_dim=a.inter_dim, experts=a.experts, topk=a.topk, tile_m=a.tile_m,
                           in_dtype="fp8", out_dtype=a.out_dtype, rank=rank, world=world)
    g = torch.Generator(device=dev).manual_seed(1234)  # the same routing and activations on every rank
    fp8 = torch.float8_e4m3fn

    def q8(*shape):
        return (torch.randn(*shape, generator=g, device=dev) * 64).clamp_(-448, 448).to(fp8)

    x, sx = q8(a.tokens, a.model_dim), torch.rand(a.tokens, generator=g, device=dev) * 1e-2
    vals, ids = torch.topk(torch.rand(a.tokens, a.experts, generator=g, device=dev), k=a.topk, dim=1)
    wts = torch.softmax(vals, dim=1)
    el = op.shard.experts_local
    gw = torch.Generator(device=dev).manual_seed(99 + rank)
    w1 = (torch.randn(el, 2 * a.inter_dim, a.model_dim, generator=gw, device=dev) * 64).clamp_(-448, 448).to(fp8)
    w2 = (torch.randn(el, a.model_dim, a.inter_dim, generator=gw, device=dev) * 64).clamp_(-448, 448).to(fp8)
    op.load_expert_weights(w1, torch.full((el, 2 * a.inter_dim), 1e-3, device=dev), w2, torch.full((el, a.model_dim), 1e-3, device=dev))
    for _ in range(3):
        op.forward(x, sx, ids.int(), wts)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ids32 = ids.int()
    if a.graph:
        st = torch.cuda.Stream()
        with torch.cuda.stream(st):
            op.forward(x, sx, ids32, wts)
            st.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=st):
                op.forward(x, sx, ids32, wts)
            graph.replay()
            st.synchronize()
            e0.record(st)
            for _ in range(a.iters):
                graph.replay()
            e1.record(st)
            st.synchronize()
    else:
        e0.record()
        for _ in range(a.iters):
            op.forward(x, sx, ids32, wts)
        e1.record()
        torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / a.iters], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        flops = 2.0 * a.tokens * a.topk * 3 * a.inter_dim * a.model_dim  # gate, up and down projections of every route
        print(json.dumps({"layer": "expert-parallel MoE", "n_gpus": world, "tokens": a.tokens, "experts": a.experts,
                          "topk": a.topk, "model_dim": a.model_dim, "inter_dim": a.inter_dim, "tile_m": a.tile_m, "out_dtype": a.out_dtype, "cuda_graph": bool(a.graph),
                          "ms_per_layer": round(float(t[0]), 4), "tflops": round(flops / float(t[0]) / 1e9, 1)}), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    _bench_main()
