"""Column-parallel use of the preshuffle GEMM across the GPUs of one machine.

The output channels (N) are split into contiguous, equal shards, one per
rank; every rank holds the activations A (replicated), its own weight shard
preshuffled locally, and computes C[:, n0:n1] with the single-GPU kernel.
There is no reduction across ranks (K is never split), so the data path has no
collective unless the caller asks for the full output, in which case the bf16
shards are all-gathered with NCCL.

The reference has no multi-GPU form of this operator; the only collective in
its tree that matches is the ``all_gather_into_tensor`` fallback of
kernels/comm/custom_all_reduce.py:929-938.  One process per GPU, as in
tests/kernels/test_allreduce.py:267,629-644.
"""

from __future__ import annotations

import contextlib
import os
from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class ShardSpec:
    n_total: int
    world: int
    rank: int

    @property
    def n_local(self) -> int:
        return self.n_total // self.world

    @property
    def n0(self) -> int:
        return self.rank * self.n_local

    @property
    def n1(self) -> int:
        return self.n0 + self.n_local


def shard_spec(n_total: int, world: int, rank: int) -> ShardSpec:
    """Equal contiguous shards of the output channels; each must itself be a
    valid weight image (a multiple of 16 channels)."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world: {rank}/{world}")
    if n_total % world != 0 or (n_total // world) % 16 != 0:
        raise ValueError(f"N={n_total} cannot be split into {world} shards that are multiples of 16 channels")
    return ShardSpec(n_total, world, rank)


def check_agreement(desc: dict, group=None, timeout_s: float = 60.0) -> None:
    """Host-side handshake before any GPU collective: every rank publishes its
    view of the problem (shape, dtypes, shard) and all must match, so a missing
    or mismatched rank surfaces as a Python error on the CPU instead of a hung
    NCCL kernel.  Uses the object collectives of ``group`` (pass a gloo group
    to keep the handshake off the GPU)."""
    world = dist.get_world_size(group)
    gathered = [None] * world
    dist.all_gather_object(gathered, desc, group=group)
    ref = {k: v for k, v in gathered[0].items() if k != "rank"}
    for r, d in enumerate(gathered):
        if d is None:
            raise RuntimeError(f"rank {r} did not answer the handshake")
        other = {k: v for k, v in d.items() if k != "rank"}
        if other != ref:
            raise RuntimeError(f"rank {r} disagrees on the problem: {other} vs {ref}")
    ranks = sorted(d["rank"] for d in gathered)
    if ranks != list(range(world)):
        raise RuntimeError(f"ranks present {ranks}, expected 0..{world - 1}")


def gather_columns(local: torch.Tensor, world: int, group=None, row_major: bool = True) -> torch.Tensor:
    """All-gather the [M, N/world] shards.  NCCL concatenates along dim 0, so
    the natural result is shard-major [world, M, N/world]; ``row_major=True``
    adds one local copy into [M, N]."""
    m, nl = local.shape
    out = torch.empty(world, m, nl, dtype=local.dtype, device=local.device)
    try:
        dist.all_gather_into_tensor(out, local.contiguous(), group=group)
    except (RuntimeError, NotImplementedError):  # backends without the fused form (old gloo)
        parts = [torch.empty_like(local) for _ in range(world)]
        dist.all_gather(parts, local.contiguous(), group=group)
        out = torch.stack(parts)
    if not row_major:
        return out
    return out.permute(1, 0, 2).reshape(m, world * nl)


def _parse_cpulist(text: str) -> list[int]:
    cpus: list[int] = []
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.extend(range(int(lo), int(hi or lo) + 1))
    return cpus


def numa_cpus_of_pci_device(pci_address: str, sysfs_root: str = "/sys") -> list[int]:
    """CPUs of the NUMA node a PCI device (``dddd:bb:dd.f``) hangs off, read from
    sysfs; empty when the node is unknown (-1) or sysfs is not there."""
    try:
        with open(os.path.join(sysfs_root, "bus/pci/devices", pci_address.lower(), "numa_node")) as f:
            node = int(f.read().strip())
        if node < 0:
            return []
        with open(os.path.join(sysfs_root, "devices/system/node", f"node{node}", "cpulist")) as f:
            return _parse_cpulist(f.read())
    except (OSError, ValueError):
        return []


@contextlib.contextmanager
def near_device(device: torch.device, sysfs_root: str = "/sys"):
    """Run the body on the CPUs next to ``device``: pinned host buffers allocated
    (and first touched) inside land on the GPU's own NUMA node, so the copies of
    the eight GPUs of a two-socket machine do not all cross to one socket.  Best
    effort: without the information, or when the process may not use those CPUs,
    nothing changes."""
    old = None
    try:
        props = torch.cuda.get_device_properties(device)
        addr = f"{getattr(props, 'pci_domain_id', 0):04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        cpus = set(numa_cpus_of_pci_device(addr, sysfs_root)) & set(os.sched_getaffinity(0))
        if cpus:
            old = os.sched_getaffinity(0)
            os.sched_setaffinity(0, cpus)
    except (AttributeError, OSError, RuntimeError):
        old = None
    try:
        yield
    finally:
        if old is not None:
            try:
                os.sched_setaffinity(0, old)
            except OSError:
                pass


def pinned_near(device: torch.device, shape, dtype) -> torch.Tensor:
    """A pinned host tensor whose pages sit on the NUMA node of ``device``."""
    with near_device(device):
        t = torch.empty(shape, dtype=dtype).pin_memory()
        t.view(torch.uint8).zero_()  # first touch
    return t


def row_shard(m: int, world: int, rank: int) -> tuple[int, int]:
    """Rows [r0, r1) of an M-row matrix that rank ``rank`` uploads when the rows
    are split evenly (M must be a multiple of ``world``)."""
    if m % world != 0:
        raise ValueError(f"M={m} is not a multiple of the group size {world}")
    per = m // world
    return rank * per, (rank + 1) * per


class ColumnParallelGemm:
    """One rank's share of C = A . W^T split on the output channels."""

    def __init__(self, N: int, K: int, in_dtype: str = "fp8", out_dtype: str = "bf16", group=None, cpu_group=None,
                 rank: int | None = None, world: int | None = None, variant_hint: int = 0):
        from .kernels.gemm.preshuffle_gemm import compile_preshuffle_gemm

        self.group = group
        self.world = world if world is not None else (dist.get_world_size(group) if dist.is_initialized() else 1)
        self.rank = rank if rank is not None else (dist.get_rank(group) if dist.is_initialized() else 0)
        self.spec = shard_spec(N, self.world, self.rank)
        self.N, self.K, self.in_dtype, self.out_dtype = N, K, in_dtype, out_dtype
        if dist.is_initialized() and self.world > 1:
            check_agreement(
                dict(rank=self.rank, N=N, K=K, in_dtype=in_dtype, out_dtype=out_dtype, n_local=self.spec.n_local),
                group=cpu_group if cpu_group is not None else group,
            )
        self.launch = compile_preshuffle_gemm(
            N=self.spec.n_local, K=K, tile_m=128, tile_n=256, tile_k=128, in_dtype=in_dtype, out_dtype=out_dtype,
            variant_hint=variant_hint,
        )
        self.w_shuf = None
        self.sb = None
        self._bias = None

    def load_weight_shard(self, w_q_local: torch.Tensor, sb_local: torch.Tensor) -> None:
        """Take this rank's rows [n0, n1) of the quantised weights (row-major)
        and preshuffle them locally: the weight image is not contiguous in N,
        so shards are shuffled after the split, never before."""
        from .utils import shuffle_weight

        if tuple(w_q_local.shape) != (self.spec.n_local, self.K):
            raise ValueError(f"weight shard must be [{self.spec.n_local}, {self.K}], got {tuple(w_q_local.shape)}")
        self.w_shuf = shuffle_weight(w_q_local).view(torch.int8 if w_q_local.element_size() == 1 else w_q_local.dtype)
        self.sb = sb_local.contiguous().view(-1)
        self._bias = torch.empty(0, dtype=torch.bfloat16 if self.out_dtype == "bf16" else torch.float16,
                                 device=w_q_local.device)

    def forward(self, a_q: torch.Tensor, sa: torch.Tensor, out: torch.Tensor | None = None, stream=None):
        """C[:, n0:n1] for this rank (bf16 [M, N/world]); asynchronous."""
        m = a_q.shape[0]
        if out is None:
            out = torch.empty(m, self.spec.n_local, dtype=self._bias.dtype, device=a_q.device)
        a = a_q.view(torch.int8) if a_q.element_size() == 1 else a_q
        self.launch(out.view(-1), a.view(-1), self.w_shuf.view(-1), sa.view(-1), self.sb, self._bias, m,
                    self.spec.n_local, stream if stream is not None else torch.cuda.current_stream())
        return out

    # ---- host buffers in, host buffer out ---------------------------------------
    def forward_host(self, a_host: torch.Tensor, sa_host: torch.Tensor, out_host: torch.Tensor, chunks: int = 8,
                     shard_upload: bool | None = None):
        """This rank's shard computed from pinned HOST activations into a pinned
        HOST output, with the legs pipelined over row blocks: while block i is
        multiplied, block i+1 is uploaded and block i-1 downloaded (separate
        streams; PCIe is full duplex).

        In a group of several GPUs every rank needs all of A.  With
        ``shard_upload`` (default whenever the group has more than one rank and
        the block size divides evenly) a rank uploads only ITS 1/world of each
        row block over PCIe and the ranks exchange the pieces with an NCCL
        all-gather over NVLink, so the host side sees A once per step instead of
        once per GPU.  Returns after enqueueing; the caller synchronises
        ``torch.cuda.current_stream()``."""
        m = a_host.shape[0]
        dev = self.w_shuf.device
        if getattr(self, "_host_state", None) is None or self._host_state[0] < m:
            a_dev = torch.empty((m, a_host.shape[1]), dtype=a_host.dtype, device=dev)
            sa_dev = torch.empty(m, dtype=torch.float32, device=dev)
            c_dev = torch.empty((m, self.spec.n_local), dtype=self._bias.dtype, device=dev)
            self._host_state = (m, a_dev, sa_dev, c_dev, torch.cuda.Stream(dev), torch.cuda.Stream(dev))
        _, a_dev, sa_dev, c_dev, s_in, s_out = self._host_state
        cur = torch.cuda.current_stream(dev)
        s_in.wait_stream(cur)
        s_out.wait_stream(cur)
        w = self.world
        rows = max(128, ((m + chunks - 1) // chunks + 127) // 128 * 128)
        if shard_upload is None:
            shard_upload = w > 1 and dist.is_initialized()
        if shard_upload and (rows % w != 0 or m % rows != 0):
            shard_upload = False  # ragged blocks: every rank uploads everything
        self.last_h2d_bytes = 0
        with torch.cuda.stream(s_in):
            sa_dev[:m].copy_(sa_host.view(-1)[:m], non_blocking=True)
        self.last_h2d_bytes += m * 4
        for r0 in range(0, m, rows):
            r1 = min(m, r0 + rows)
            with torch.cuda.stream(s_in):
                if shard_upload:
                    p0, p1 = row_shard(r1 - r0, w, self.rank)
                    a_dev[r0 + p0 : r0 + p1].copy_(a_host[r0 + p0 : r0 + p1], non_blocking=True)
                    self.last_h2d_bytes += (p1 - p0) * a_host.shape[1] * a_host.element_size()
                    # in place: rank r's piece already sits at its position in the block
                    dist.all_gather_into_tensor(a_dev[r0:r1], a_dev[r0 + p0 : r0 + p1], group=self.group)
                else:
                    a_dev[r0:r1].copy_(a_host[r0:r1], non_blocking=True)
                    self.last_h2d_bytes += (r1 - r0) * a_host.shape[1] * a_host.element_size()
                ready = torch.cuda.Event()
                ready.record(s_in)
            cur.wait_event(ready)
            self.forward(a_dev[r0:r1], sa_dev[r0:r1], out=c_dev[r0:r1], stream=cur)
            done = torch.cuda.Event()
            done.record(cur)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                out_host[r0:r1].copy_(c_dev[r0:r1], non_blocking=True)
        cur.wait_stream(s_out)
        return out_host

    # ---- GEMM fused with the all-gather of its output shards -------------------
    def enable_fused_gather(self, m_max: int) -> None:
        """Allocate (once) two full-width [m_max, N] output buffers in symmetric
        memory, i.e. mapped into every rank of the group, for
        :meth:`forward_full_fused`.  Collective: every rank must call it."""
        import ctypes
        import os

        import torch.distributed._symmetric_memory as symm_mem

        if self.world > 8:
            raise ValueError("the fused gather writes to at most 8 output buffers")
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer stores only
        dev = self.w_shuf.device
        group = self.group if self.group is not None else dist.group.WORLD
        self._sym = []
        for _ in range(2):
            buf = symm_mem.empty((m_max, self.N), dtype=self._bias.dtype, device=dev)
            hdl = symm_mem.rendezvous(buf, group)
            ptrs = (ctypes.c_void_p * self.world)(*[int(hdl.buffer_ptrs[r]) for r in range(self.world)])
            self._sym.append((buf, hdl, ptrs))
        self._flip = 0
        self._flag = torch.zeros(1, dtype=torch.int32, device=dev)
        self._m_max = m_max

    def forward_full_fused(self, a_q: torch.Tensor, sa: torch.Tensor, stream=None) -> torch.Tensor:
        """Full [M, N] output on every rank from ONE GEMM kernel per rank: each
        output tile is TMA-stored into the full-width buffer of every rank
        (columns [rank*N/w, (rank+1)*N/w)), so the exchange over NVLink overlaps
        the math; a one-element NCCL all-reduce on the SAME stream then orders
        the stores against the readers.  The returned tensor is valid for work
        enqueued on that stream (or ordered after it) until this rank issues
        its NEXT call: the two buffers alternate only so that a peer that is one
        call ahead never writes into the buffer this rank is still reading
        (a peer cannot pass the all-reduce of call i+1 before this rank has
        issued call i+1, and call i+2 is the first that reuses call i's buffer)."""
        from . import _lib

        m = a_q.shape[0]
        if m > self._m_max:
            raise ValueError(f"M={m} exceeds the buffers allocated by enable_fused_gather({self._m_max})")
        buf, _hdl, ptrs = self._sym[self._flip]
        self._flip ^= 1
        lib = _lib.load()
        s = stream if stream is not None else torch.cuda.current_stream()
        a = a_q.view(torch.int8) if a_q.element_size() == 1 else a_q
        eight = self.in_dtype in ("fp8", "int8")
        rc = lib.flyb200_gemm_a8w8_scatter(
            ptrs, self.world, self.rank, self.N, self.spec.n0,
            a.data_ptr(), self.w_shuf.data_ptr(), sa.data_ptr() if eight else None, self.sb.data_ptr() if eight else None,
            None, m, self.spec.n_local, self.K, _lib.IN_DTYPES[self.in_dtype], _lib.OUT_DTYPES[self.out_dtype],
            _lib.EPI_NONE, 0, s.cuda_stream,
        )  # fmt: skip
        _lib.check(rc, "gemm_a8w8_scatter")
        if self.world > 1:
            # all ranks' stores have landed before anyone reads; issued on the kernel's stream
            with torch.cuda.stream(s):
                dist.all_reduce(self._flag, group=self.group)
        return buf[:m]

    def forward_full(self, a_q, sa, row_major: bool = True):
        """Full [M, N] on every rank: local shard, then an NCCL all-gather."""
        local = self.forward(a_q, sa)
        if self.world == 1:
            return local
        return gather_columns(local, self.world, self.group, row_major=row_major)
