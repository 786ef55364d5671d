"""Column-parallel sharding on CPU: layout helpers, and a 2-rank gloo run in which each rank
computes its output shard with the CPU oracle and the all-gather rebuilds the full product."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kaio_b200 import sharding


def test_shard_bounds():
    assert sharding.shard_bounds(64, 2, 1) == (32, 64)
    assert sharding.shard_bounds(11008, 8, 3) == (4128, 5504)
    with pytest.raises(ValueError):
        sharding.shard_bounds(100, 8, 0)
    with pytest.raises(ValueError):
        sharding.shard_bounds(64, 2, 2)


def test_packed_int4_shard_is_a_contiguous_slice(oracle):
    k, n, world = 256, 64, 2
    w = oracle.lcg_s4(5, k * n).reshape(k, n)
    packed = torch.from_numpy(oracle.pack_s4(w, k, n).view(np.int32))
    for rank in range(world):
        lo, hi = sharding.shard_bounds(n, world, rank)
        mine = sharding.shard_packed_int4(packed, k, n, world, rank)
        want = oracle.pack_s4(np.ascontiguousarray(w[:, lo:hi]), k, hi - lo).view(np.int32)
        assert np.array_equal(mine.numpy(), want)
        assert mine.data_ptr() == packed.data_ptr() + lo * (k // 8) * 4  # a view, not a copy


def test_strided_shards(oracle):
    k, n, world = 256, 64, 4
    b = torch.from_numpy(oracle.lcg_i8(1, k * n))
    s = torch.arange((k // 128) * n, dtype=torch.float32).to(torch.float16)
    for rank in range(world):
        lo, hi = sharding.shard_bounds(n, world, rank)
        assert torch.equal(sharding.shard_int8_weights(b, k, n, world, rank).view(k, -1), b.view(k, n)[:, lo:hi])
        assert torch.equal(sharding.shard_group_scales(s, k, n, world, rank).view(k // 128, -1),
                           s.view(k // 128, n)[:, lo:hi])


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, m, n, k, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle as orc
        a = orc.lcg_i8(11, m * k)
        b = orc.lcg_i8(12, k * n)
        sa = np.linspace(0.001, 0.01, m).astype(np.float32)
        sw = np.linspace(0.01, 0.001, n).astype(np.float32)
        b_loc = sharding.shard_int8_weights(torch.from_numpy(b), k, n, world, rank).numpy()
        sw_loc = sharding.shard_column_vector(torch.from_numpy(sw), n, world, rank).numpy()
        n_loc = n // world
        shard = orc.matmul_int8_scaled(a, b_loc, sa, sw_loc, m, n_loc, k)
        gather = sharding.ColumnGather(m, n, torch.float32, "cpu")
        full = gather(torch.from_numpy(shard)).numpy()
        want = orc.matmul_int8_scaled(a, b, sa, sw, m, n, k)
        ret[rank] = bool(np.array_equal(full, want))
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_all_gather_rebuilds_full_output(oracle):
    m, n, k, world = 24, 64, 64, 2
    mgr = mp.Manager()
    ret = mgr.dict()
    port = _free_port()
    mp.spawn(_worker, args=(world, port, m, n, k, ret), nprocs=world, join=True)
    assert dict(ret) == {0: True, 1: True}
