"""Column-parallel sharding of the quantized GEMMs across the GPUs of one node.

Every output column of these GEMMs depends on one weight column (and its scales) and on all
of the activations, so rank ``r`` of ``P`` owns columns ``[r*N/P, (r+1)*N/P)`` of the weights,
computes the ``[M, N/P]`` output shard with the ordinary single-GPU entry points, and one
all-gather of the shards rebuilds ``[M, N]`` on every rank.  There is no reference counterpart:
KAIO is single-device.

The helpers below are layout logic only (they run on CPU tensors too, which is how the
``gloo`` tests exercise them); the collective is ``torch.distributed`` (NCCL over NVLink on
GPUs).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_bounds(n: int, world: int, rank: int, multiple: int = 16) -> tuple[int, int]:
    """Column range of ``rank``.  ``n`` must split into ``world`` equal shards whose width is a
    multiple of ``multiple`` (16 keeps every shard on the TMA paths)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    if n % (world * multiple) != 0:
        raise ValueError(f"N={n} does not split into {world} shards of a multiple of {multiple} columns")
    w = n // world
    return rank * w, (rank + 1) * w


def shard_int8_weights(b: torch.Tensor, k: int, n: int, world: int, rank: int) -> torch.Tensor:
    """Row-major ``[K, N]`` s8 weights -> contiguous ``[K, N/P]`` (flat)."""
    lo, hi = shard_bounds(n, world, rank)
    return b.view(k, n)[:, lo:hi].contiguous().view(-1)


def shard_packed_int4(packed: torch.Tensor, k: int, n: int, world: int, rank: int) -> torch.Tensor:
    """Packed s4 weights: word ``k/8`` of column ``j`` lives at ``(k/8) + j*(K/8)``, so a column
    range is one contiguous slice of the flat buffer (a view, no copy)."""
    lo, hi = shard_bounds(n, world, rank)
    kw = k // 8
    return packed.view(-1)[lo * kw:hi * kw]


def shard_group_scales(scales: torch.Tensor, k: int, n: int, world: int, rank: int,
                       group_size: int = 128) -> torch.Tensor:
    """f16 ``[K/group, N]`` row-major group scales -> contiguous ``[K/group, N/P]`` (flat)."""
    lo, hi = shard_bounds(n, world, rank)
    return scales.view(k // group_size, n)[:, lo:hi].contiguous().view(-1)


def shard_column_vector(v: torch.Tensor, n: int, world: int, rank: int) -> torch.Tensor:
    """Per-column vector (e.g. f32 weight scales) -> this rank's slice."""
    lo, hi = shard_bounds(n, world, rank)
    return v.view(-1)[lo:hi].contiguous()


class ColumnGather:
    """All-gather of ``[M, N/P]`` output shards into a row-major ``[M, N]`` on every rank.

    NCCL gathers into ``[P, M, N/P]``; the un-shard step interleaves the shards back into rows.
    Buffers are allocated once per (M, N, dtype)."""

    def __init__(self, m: int, n: int, dtype: torch.dtype, device, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.m, self.n, self.n_loc = m, n, n // self.world
        shard_bounds(n, self.world, 0, multiple=1)
        self.gathered = torch.empty(self.world * m * self.n_loc, dtype=dtype, device=device)
        self.full = torch.empty(m, n, dtype=dtype, device=device)

    def __call__(self, shard: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            self.full.view(-1).copy_(shard.view(-1)[: self.m * self.n])
            return self.full
        dist.all_gather_into_tensor(self.gathered, shard.view(-1)[: self.m * self.n_loc].contiguous(),
                                    group=self.group)
        self.unshard()
        return self.full

    def unshard(self) -> torch.Tensor:
        """``gathered[p, i, j]`` -> ``full[i, p*N/P + j]``."""
        src = self.gathered.view(self.world, self.m, self.n_loc).transpose(0, 1)
        self.full.view(self.m, self.world, self.n_loc).copy_(src)
        return self.full


class PanelPipeline:
    """Sharded W4A16 GEMM whose all-gather overlaps the GEMM: the rank's ``N/P`` columns are cut
    into ``panels`` column panels; panel ``i`` is gathered (NCCL, on ``comm_stream``) while panel
    ``i+1`` is computed.  Packed INT4 weights are column-major, so a column panel of the shard is
    a contiguous slice; the group scales of each panel are copied once at construction.

    After ``run()`` every rank holds the row-major ``[M, N]`` product in ``self.full``.
    """

    def __init__(self, ops, device, a, w_packed_shard, scales_shard, m, n, k, world, rank, comm_stream,
                 panels: int = 4, group=None):
        self.ops, self.device, self.a = ops, device, a
        self.m, self.n, self.k, self.world, self.group = m, n, k, world, group
        self.n_loc = n // world
        while panels > 1 and self.n_loc % (panels * 16) != 0:
            panels -= 1
        self.panels, self.pw = panels, self.n_loc // panels
        kw, groups = k // 8, k // 128
        self.w = [w_packed_shard.view(-1)[i * self.pw * kw:(i + 1) * self.pw * kw] for i in range(panels)]
        sc2d = scales_shard.view(groups, self.n_loc)
        self.sc = [sc2d[:, i * self.pw:(i + 1) * self.pw].contiguous().view(-1) for i in range(panels)]
        dev_t = a.device
        self.c = [torch.empty(m * self.pw, dtype=torch.float16, device=dev_t) for _ in range(panels)]
        self.gathered = [torch.empty(world * m * self.pw, dtype=torch.float16, device=dev_t) for _ in range(panels)]
        self.full = torch.empty(m, n, dtype=torch.float16, device=dev_t)
        self.comm_stream = comm_stream
        self.events = [torch.cuda.Event() for _ in range(panels)]

    def run(self):
        main = torch.cuda.current_stream()
        # full[i, p*n_loc + q*pw + j] <- gathered[q][p, i, j]
        full5 = self.full.view(self.m, self.world, self.panels, self.pw)
        for q in range(self.panels):
            self.ops.matmul_int4(self.device, self.a, self.w[q], self.sc[q], self.c[q], self.m, self.pw, self.k, 128)
            self.events[q].record(main)
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_event(self.events[q])
                dist.all_gather_into_tensor(self.gathered[q], self.c[q], group=self.group)
                full5[:, :, q, :].copy_(self.gathered[q].view(self.world, self.m, self.pw).transpose(0, 1))
        main.wait_stream(self.comm_stream)
        return self.full


class FusedGatherGemm:
    """Sharded W4A16 GEMM whose epilogue writes into every rank's output buffer (peer memory):
    one kernel per rank does the GEMM and the all-gather, tile by tile over NVLink.

    The ``[M, N]`` f16 output lives in torch symmetric memory so that every rank holds a mapping
    of every other rank's buffer.  ``run()`` launches the kernel and then meets the other ranks
    at the symmetric-memory barrier; after it returns (and the stream is synchronised or ordered),
    ``self.out`` holds the full product on every rank.
    """

    def __init__(self, ops, device, m, n, k, world, rank, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.ops, self.device = ops, device
        self.m, self.n, self.k, self.world, self.rank = m, n, k, world, rank
        self.flat = symm_mem.empty(m * n, dtype=torch.float16, device=f"cuda:{device.ordinal}")
        self.handle = symm_mem.rendezvous(self.flat, group if group is not None else dist.group.WORLD)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.out = self.flat.view(m, n)

    def run(self, a, w_packed_shard, scales_shard):
        self.ops.matmul_int4_allgather(self.device, a, w_packed_shard, scales_shard, self.ptrs,
                                       self.m * self.n, self.world, self.rank, self.m, self.n, self.k)
        self.handle.barrier()  # every rank's stores have landed before anyone reads
        return self.out
