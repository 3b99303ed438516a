"""Host logic of the column-parallel path on two CPU ranks (gloo)."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flydsl_b200.column_parallel import check_agreement, gather_columns, shard_spec


def test_shard_spec():
    s = shard_spec(57344, 8, 3)
    assert (s.n_local, s.n0, s.n1) == (7168, 21504, 28672)
    assert [shard_spec(57344, w, 0).n_local for w in (1, 2, 4, 8)] == [57344, 28672, 14336, 7168]
    with pytest.raises(ValueError):
        shard_spec(1000, 8, 0)  # 125 channels per shard: not a multiple of 16
    with pytest.raises(ValueError):
        shard_spec(1024, 3, 0)
    with pytest.raises(ValueError):
        shard_spec(1024, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, mismatch, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n, m = 64, 5
        desc = dict(rank=rank, N=n if not (mismatch and rank == 1) else n + 16, K=256, in_dtype="fp8")
        try:
            check_agreement(desc)
            agreed = True
        except RuntimeError as e:
            agreed = False
            assert "disagrees" in str(e)
        spec = shard_spec(n, world, rank)
        full = torch.arange(m * n, dtype=torch.float32).view(m, n).to(torch.bfloat16)
        local = full[:, spec.n0 : spec.n1].contiguous()
        got = gather_columns(local, world, row_major=True)
        shard_major = gather_columns(local, world, row_major=False)
        ok = torch.equal(got, full) and torch.equal(shard_major[rank], local) and shard_major.shape == (world, m, n // world)
        results.put((rank, agreed, ok))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mismatch", [False, True])
def test_handshake_and_gather_two_ranks(mismatch):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, mismatch, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, agreed, ok in out:
        assert agreed == (not mismatch)
        assert ok


def test_row_shard_and_numa_lookup(tmp_path):
    from flydsl_b200.column_parallel import numa_cpus_of_pci_device, row_shard

    assert [row_shard(2048, 8, r) for r in (0, 3, 7)] == [(0, 256), (768, 1024), (1792, 2048)]
    with pytest.raises(ValueError):
        row_shard(100, 8, 0)
    # a fake sysfs: the GPU at 0000:1b:00.0 sits on node 1, whose CPUs are 32-63 and 96-127
    dev = tmp_path / "bus/pci/devices/0000:1b:00.0"
    dev.mkdir(parents=True)
    (dev / "numa_node").write_text("1\n")
    node = tmp_path / "devices/system/node/node1"
    node.mkdir(parents=True)
    (node / "cpulist").write_text("32-63,96-127\n")
    cpus = numa_cpus_of_pci_device("0000:1B:00.0", sysfs_root=str(tmp_path))
    assert cpus == list(range(32, 64)) + list(range(96, 128))
    # unknown node (-1) or a device that is not there: no opinion
    (dev / "numa_node").write_text("-1\n")
    assert numa_cpus_of_pci_device("0000:1b:00.0", sysfs_root=str(tmp_path)) == []
    assert numa_cpus_of_pci_device("0000:ff:00.0", sysfs_root=str(tmp_path)) == []


def _sharded_upload_worker(rank, world, port, results):
    """What forward_host does with the activations on several ranks, on CPU tensors: each rank
    fills only its rows of a block, the in-place all-gather completes the block on every rank."""
    from flydsl_b200.column_parallel import row_shard

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m, k, rows = 16, 8, 8
        a_host = torch.arange(m * k, dtype=torch.float32).view(m, k)
        a_dev = torch.full((m, k), -1.0)
        for r0 in range(0, m, rows):
            p0, p1 = row_shard(rows, world, rank)
            a_dev[r0 + p0 : r0 + p1].copy_(a_host[r0 + p0 : r0 + p1])
            parts = [torch.empty(p1 - p0, k) for _ in range(world)]
            dist.all_gather(parts, a_dev[r0 + p0 : r0 + p1].contiguous())
            a_dev[r0 : r0 + rows] = torch.cat(parts)
        results.put((rank, torch.equal(a_dev, a_host)))
    finally:
        dist.destroy_process_group()


def test_sharded_upload_reassembles_activations_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_sharded_upload_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert out == [(0, True), (1, True)]
