"""Host logic of the expert-parallel MoE layer on CPU: shard arithmetic, routing in local numbering,
and (two gloo ranks) that the ranks' local routing tables together cover every route exactly once."""

import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from flydsl_b200.expert_parallel import expert_shard, local_routing
from flydsl_b200.kernels.moe.moe_gemm_2stage import moe_sorting
from oracle import moe_oracle


def test_expert_shard():
    s = expert_shard(8, 4, 2)
    assert (s.experts_local, s.e0, s.e1) == (2, 4, 6)
    with pytest.raises(ValueError):
        expert_shard(6, 4, 0)
    with pytest.raises(ValueError):
        expert_shard(8, 2, 2)


def test_local_routing_and_sorting_drop_foreign_routes():
    g = torch.Generator().manual_seed(3)
    ids, wts = moe_oracle.make_routing(50, 8, 2, g)
    seen = torch.zeros(50, 2, dtype=torch.int32)
    for rank in range(4):
        sh = expert_shard(8, 4, rank)
        loc = local_routing(ids, sh)
        assert torch.equal(loc >= 0, (ids >= sh.e0) & (ids < sh.e1))
        srt, w, e_ids, post = moe_sorting(loc, wts, num_experts=sh.experts_local, block_size=16)
        want = moe_oracle.moe_sorting(loc, wts, sh.experts_local, 16)
        assert torch.equal(srt, want[0]) and torch.equal(e_ids, want[2]) and torch.equal(post, want[3])
        valid = srt[: int(post[0])]
        valid = valid[(valid & 0xFFFFFF) < 50]
        seen[(valid & 0xFFFFFF).long(), (valid >> 24).long()] += 1
    assert torch.all(seen == 1)  # every (token, slot) is handled by exactly one rank


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # the sum over ranks of the oracle restricted to a rank's experts is the whole layer
        d = moe_oracle.make_inputs(24, 128, 128, 4, 2, "int8", seed=9)
        sh = expert_shard(4, world, rank)
        loc = local_routing(d["topk_ids"], sh)
        part = moe_oracle.moe_gemm2(d["a2_q"], d["w2_q"][sh.e0:sh.e1], d["scale_a2"], d["scale_w2"][sh.e0:sh.e1],
                                    loc.long(), d["topk_weights"], 128, True)
        dist.all_reduce(part)
        full = moe_oracle.moe_gemm2(d["a2_q"], d["w2_q"], d["scale_a2"], d["scale_w2"], d["topk_ids"].long(),
                                    d["topk_weights"], 128, True)
        q.put((rank, bool(torch.allclose(part, full, rtol=1e-5, atol=1e-5)), ""))
    except Exception as e:
        q.put((rank, False, repr(e)))
    finally:
        dist.destroy_process_group()


def test_partial_outputs_sum_to_the_layer_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert all(ok for _, ok, _ in res), res
