"""Two-rank run of the fused GEMM + all-gather (needs 2 GPUs; skipped otherwise).

Each rank computes its column shard of a W4A16 GEMM; the kernel's epilogue writes the shard into
both ranks' [M, N] buffers (torch symmetric memory = peer mappings).  Both ranks must end with the
oracle's full product.  No rank faults or exits mid-step; NVLS is not involved.
"""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
G = 128


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, shapes, ret):
    import torch.distributed as dist

    from kaio_b200 import ops, sharding
    from oracle import oracle as orc
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    ok = True
    try:
        dev = ops.KaioDevice(rank)
        for (m, n, k) in shapes:
            rng = np.random.default_rng(m + n + k)
            w = rng.integers(-8, 8, (k, n), dtype=np.int8)
            a = rng.standard_normal(m * k).astype(np.float16)
            sc = rng.uniform(0.005, 0.02, (k // G) * n).astype(np.float16)
            packed = orc.pack_s4(w, k, n)
            want = orc.matmul_int4(a, packed, sc, m, n, k, f16_out=True).astype(np.float32)
            pk = torch.from_numpy(packed.view(np.int32)).cuda()
            w_loc = sharding.shard_packed_int4(pk, k, n, world, rank)
            sc_loc = sharding.shard_group_scales(torch.from_numpy(sc).cuda(), k, n, world, rank)
            fused = sharding.FusedGatherGemm(ops, dev, m, n, k, world, rank)
            for _ in range(2):  # twice: the second call overwrites buffers the peer has read
                fused.flat.fill_(float("nan"))
                dist.barrier()
                out = fused.run(torch.from_numpy(a).cuda(), w_loc, sc_loc)
                torch.cuda.synchronize()
                got = out.float().cpu().numpy()
                rel = np.max(np.abs(got - want) / np.maximum(np.abs(want), 1.0))
                ok = ok and bool(np.all(np.isfinite(got))) and rel < 2e-2
            # the NCCL form behind the C ABI (kaio_b200_allgather_cols) on the same shard: the
            # gathered matrix must equal the fused one bit for bit
            n_loc = n // world
            shard = torch.empty(m * n_loc, device="cuda", dtype=torch.float16)
            ops.matmul_int4(dev, torch.from_numpy(a).cuda(), w_loc, sc_loc, shard, m, n_loc, k, G)
            full = torch.full((m * n,), float("nan"), device="cuda", dtype=torch.float16)
            comm = dist.distributed_c10d._get_default_group()._get_backend(torch.device("cuda"))._comm_ptr()
            ops.allgather_cols(dev, shard, full, m, n, world, comm)
            torch.cuda.synchronize()
            ok = ok and ops.last_variant() == "allgather_cols_nccl"
            ok = ok and bool(torch.equal(full.view(torch.int16), out.reshape(-1).view(torch.int16)))
            assert ops.device_status(dev)[0] == 0
        ret[rank] = ok
    finally:
        dist.destroy_process_group()


def test_fused_gather_two_ranks():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    world = 2
    # the last two run the paired GEMM (m > 512), whose epilogue writes through the NVLink multicast
    # object where there is one; ragged rows and a shard width that is not a multiple of the tile
    shapes = [(16, 1024, 512), (300, 2048, 1024), (640, 2048, 1024), (700, 2080, 512)]
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), shapes, ret), nprocs=world, join=True)
    assert dict(ret) == {0: True, 1: True}
