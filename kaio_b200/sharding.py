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

import os

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
        # Where torch binds the symmetric buffers to an NVLink multicast object the large-m kernel
        # writes each output block once through it (KAIO_B200_MULTICAST=0 keeps per-rank stores).
        self.multicast = 0
        if os.environ.get("KAIO_B200_MULTICAST", "1") != "0":
            self.multicast = int(getattr(self.handle, "multicast_ptr", 0) or 0)

    def run(self, a, w_packed_shard, scales_shard):
        if self.multicast:
            self.ops.matmul_int4_allgather_multicast(self.device, a, w_packed_shard, scales_shard, self.ptrs,
                                                     self.m * self.n, self.multicast, self.world, self.rank,
                                                     self.m, self.n, self.k)
        else:
            self.ops.matmul_int4_allgather(self.device, a, w_packed_shard, scales_shard, self.ptrs,
                                           self.m * self.n, self.world, self.rank, self.m, self.n, self.k)
        self.handle.barrier()  # every rank's stores have landed before anyone reads
        return self.out
