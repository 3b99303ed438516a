"""GEMM fused with the all-gather of its output shards, on two GPUs.

Needs two CUDA devices (skipped otherwise).  One process per GPU, NCCL; every
rank checks the full [M, N] result it received against the CPU oracle and
against the unfused path (local shard + NCCL all-gather)."""

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
    from flydsl_b200.column_parallel import ColumnParallelGemm
    from oracle import a8w8_oracle as oracle

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    ok, msg = True, ""
    try:
        for in_dtype, m, n, k in (("fp8", 300, 1056, 1024), ("int8", 1000, 2048, 2048)):
            a_q, b_q, sa, sb = oracle.make_inputs(m, n, k, in_dtype, seed=11 + m)  # same on every rank
            op = ColumnParallelGemm(n, k, in_dtype=in_dtype, rank=rank, world=world)
            sl = slice(op.spec.n0, op.spec.n1)
            op.load_weight_shard(b_q[sl].to(dev), sb[sl].to(dev))
            op.enable_fused_gather(m_max=1024)
            ref = oracle.run_torch(a_q, b_q, sa, sb)
            a_d, sa_d = a_q.to(dev), sa.to(dev)
            for it in range(3):  # alternates the two symmetric buffers
                full = op.forward_full_fused(a_d, sa_d)
                torch.cuda.synchronize()
                bad = oracle.strict_mismatches(full.float().cpu(), ref, 1e-2, 1e-2)
                if bad:
                    ok, msg = False, f"{in_dtype} it{it}: {bad} mismatches vs oracle on rank {rank}"
            unfused = op.forward_full(a_d, sa_d, row_major=True)
            torch.cuda.synchronize()
            if not torch.equal(unfused, full):
                ok, msg = False, f"{in_dtype}: fused and unfused results differ on rank {rank}"
            if _lib.read_status() != 0:
                ok, msg = False, "device status set"
        dist.barrier()
    except Exception as e:  # report instead of hanging the peer
        ok, msg = False, repr(e)
    finally:
        q.put((rank, ok, msg))
        dist.destroy_process_group()


def test_fused_gemm_allgather_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=300) for _ in procs)
    for p in procs:
        p.join(timeout=120)
    for rank, ok, msg in results:
        assert ok, msg
