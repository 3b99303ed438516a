"""Expert-parallel MoE layer on two GPUs (skipped with fewer): one process per GPU, NCCL all-reduce
of the ranks' partial outputs, every rank checks the full result against the CPU oracle of the whole layer."""

import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import torch.distributed as dist

    from flydsl_b200 import _lib
    from flydsl_b200.expert_parallel import ExpertParallelMoe
    from oracle import moe_oracle

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    ok, msg = True, ""
    try:
        for in_dtype, tokens, tile_m, out_dtype in (("fp8", 200, 64, "bf16"), ("int8", 40, 16, "f32"), ("fp8", 300, 128, "f32")):
            model_dim, inter_dim, experts, topk = 512, 256, 8, 2
            d = moe_oracle.make_inputs(tokens, model_dim, inter_dim, experts, topk, in_dtype, seed=17 + tokens)  # same on every rank
            op = ExpertParallelMoe(model_dim=model_dim, inter_dim=inter_dim, experts=experts, topk=topk, tile_m=tile_m,
                                   in_dtype=in_dtype, out_dtype=out_dtype, rank=rank, world=world)
            sl = slice(op.shard.e0, op.shard.e1)
            op.load_expert_weights(d["w1_q"][sl].to(dev), d["scale_w1"][sl].to(dev), d["w2_q"][sl].to(dev), d["scale_w2"][sl].to(dev))
            y = op.forward(d["x_q"].to(dev), d["scale_x"].to(dev), d["topk_ids"].to(dev), d["topk_weights"].to(dev))
            torch.cuda.synchronize()
            ref = moe_oracle.moe_gemm2(d["a2_q"], d["w2_q"], d["scale_a2"], d["scale_w2"], d["topk_ids"].long(),
                                       d["topk_weights"], model_dim, True)
            err = float((y.float().cpu() - ref).abs().max())
            if err > 5e-2 * float(ref.abs().max()):
                ok, msg = False, f"{in_dtype}: max abs error {err} on rank {rank}"
            if _lib.read_status() != 0:
                ok, msg = False, "device status set"
        dist.barrier()
    except Exception as e:  # report instead of hanging the peer
        ok, msg = False, repr(e)
    finally:
        q.put((rank, ok, msg))
        dist.destroy_process_group()


def test_expert_parallel_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert all(ok for _, ok, _ in res), res
