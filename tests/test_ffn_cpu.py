"""The W4A16 feed-forward chain on CPU: the oracle's SiLU-gate against known answers, the
row-parallel (K-shard) layout helpers, and a 2-rank gloo run of ``FfnInt4`` in which the three
launches of each rank are played by the CPU oracle and the partial outputs are summed by the
collective (all-reduce and reduce-scatter)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kaio_b200 import ffn


# ---------------------------------------------------------------- oracle pins

def test_silu_gate_oracle_known_answers(oracle):
    # sigmoid(0) = 1/2 exactly; a zero gate or a zero x gives zero; for large x the sigmoid is 1
    # to f32 precision and the result is x*gate; for large negative x it underflows to -0.
    x = np.array([0.0, 1.0, 3.0, 40.0, -200.0, 2.0], dtype=np.float32)
    g = np.array([5.0, 0.0, 1.0, 0.25, 1.0, -1.0], dtype=np.float32)
    out = oracle.silu_gate_f32(x, g)
    assert out[0] == 0.0 and out[1] == 0.0
    assert out[3] == 10.0
    assert out[4] == 0.0
    assert out[2] == np.float32(3.0 / (1.0 + np.exp(-3.0)))
    assert out[5] == np.float32(-2.0 / (1.0 + np.exp(-2.0)))


def test_silu_gate_oracle_on_the_example_data(oracle):
    # the example's closed-form inputs (examples/fused_silu_gate/src/main.rs:45-51), checked
    # against the same formula written independently in numpy float64
    n = 1 << 14
    i = np.arange(n)
    x = ((i % 97).astype(np.float32) / np.float32(97.0)) - np.float32(0.5)
    g = ((i % 113).astype(np.float32) / np.float32(113.0)) - np.float32(0.5)
    want = (x.astype(np.float64) / (1.0 + np.exp(-x.astype(np.float64))) * g.astype(np.float64)).astype(np.float32)
    got = oracle.silu_gate_f32(x, g)
    # x*sig*g and x/(1+e)*g differ in the last f64 bit at most; after narrowing to f32 they agree
    # except on rare ties
    assert np.max(np.abs(got - want)) <= 1e-9


def test_silu_gate_f16_oracle_strides(oracle):
    rng = np.random.default_rng(3)
    rows, cols = 5, 24
    both = (rng.standard_normal((rows, 2 * cols)) * 3).astype(np.float16)
    got = oracle.silu_gate_f16(both.reshape(-1), both.reshape(-1)[cols:], rows, cols, x_ld=2 * cols, gate_ld=2 * cols)
    want32 = oracle.silu_gate_f32(both[:, :cols].astype(np.float32).reshape(-1),
                                  both[:, cols:].astype(np.float32).reshape(-1))
    assert np.array_equal(got.reshape(-1), want32.astype(np.float16))


# ---------------------------------------------------------------- layout helpers

def test_k_shard_bounds():
    assert ffn.k_shard_bounds(28672, 8, 3) == (10752, 14336)
    with pytest.raises(ValueError):
        ffn.k_shard_bounds(1024, 3, 0)
    with pytest.raises(ValueError):
        ffn.k_shard_bounds(256, 4, 0)  # 64-wide shards would split a scale group


def test_k_shard_matches_packing_the_row_slice(oracle):
    k, n, world = 512, 24, 2
    w = oracle.lcg_s4(9, k * n).reshape(k, n)
    packed = torch.from_numpy(oracle.pack_s4(w, k, n).view(np.int32))
    sc = torch.arange((k // 128) * n, dtype=torch.float32).to(torch.float16)
    for rank in range(world):
        lo, hi = ffn.k_shard_bounds(k, world, rank)
        mine = ffn.k_shard_packed_int4(packed, k, n, world, rank)
        want = oracle.pack_s4(np.ascontiguousarray(w[lo:hi]), hi - lo, n).view(np.int32)
        assert np.array_equal(mine.numpy(), want)
        s_mine = ffn.k_shard_group_scales(sc, k, n, world, rank)
        assert torch.equal(s_mine.view(-1, n), sc.view(k // 128, n)[lo // 128:hi // 128])


def test_concat_gate_up_is_the_packing_of_the_concatenated_matrix(oracle):
    k, n = 256, 16
    wg = oracle.lcg_s4(1, k * n).reshape(k, n)
    wu = oracle.lcg_s4(2, k * n).reshape(k, n)
    sg = torch.arange((k // 128) * n, dtype=torch.float32).to(torch.float16)
    su = (torch.arange((k // 128) * n, dtype=torch.float32) + 100).to(torch.float16)
    packed, scales = ffn.concat_gate_up(torch.from_numpy(oracle.pack_s4(wg, k, n).view(np.int32)), sg,
                                        torch.from_numpy(oracle.pack_s4(wu, k, n).view(np.int32)), su, k, n)
    want = oracle.pack_s4(np.ascontiguousarray(np.concatenate([wg, wu], axis=1)), k, 2 * n).view(np.int32)
    assert np.array_equal(packed.numpy(), want)
    assert torch.equal(scales.view(k // 128, 2 * n), torch.cat([sg.view(-1, n), su.view(-1, n)], dim=1))


def test_interleave_gate_up_is_the_packing_of_the_interleaved_matrix(oracle):
    """Blocks of 64 gate columns alternate with the same columns of up: the layout of the fused
    gate|up + SiLU-gate GEMM."""
    k, n = 256, 128
    wg = oracle.lcg_s4(3, k * n).reshape(k, n)
    wu = oracle.lcg_s4(4, k * n).reshape(k, n)
    sg = torch.arange((k // 128) * n, dtype=torch.float32).to(torch.float16)
    su = (torch.arange((k // 128) * n, dtype=torch.float32) + 1000).to(torch.float16)
    w_gu, s_gu = ffn.concat_gate_up(torch.from_numpy(oracle.pack_s4(wg, k, n).view(np.int32)), sg,
                                    torch.from_numpy(oracle.pack_s4(wu, k, n).view(np.int32)), su, k, n)
    packed, scales = ffn.interleave_gate_up(w_gu, s_gu, k, n)
    dense = np.concatenate([np.concatenate([wg[:, b:b + 64], wu[:, b:b + 64]], axis=1) for b in range(0, n, 64)], axis=1)
    assert np.array_equal(packed.numpy(), oracle.pack_s4(np.ascontiguousarray(dense), k, 2 * n).view(np.int32))
    sgm, sum_ = sg.view(-1, n), su.view(-1, n)
    want_s = torch.cat([torch.cat([sgm[:, b:b + 64], sum_[:, b:b + 64]], dim=1) for b in range(0, n, 64)], dim=1)
    assert torch.equal(scales.view(k // 128, 2 * n), want_s)
    idx = ffn.interleave_index(n)
    assert sorted(idx.tolist()) == list(range(2 * n))
    with pytest.raises(ValueError):
        ffn.interleave_index(96)


# ---------------------------------------------------------------- the chain over gloo

class OracleOps:
    """Stands in for ``kaio_b200.ops`` on CPU tensors: each launch is the CPU oracle's function."""

    def __init__(self, orc):
        self.orc = orc

    def matmul_int4(self, device, a, b_packed, scales, c, m, n, k, group_size):
        out = self.orc.matmul_int4(a.numpy()[: m * k], b_packed.numpy().view(np.uint32)[: (k // 8) * n],
                                   scales.numpy()[: (k // 128) * n], m, n, k, f16_out=(c.dtype == torch.float16))
        c.view(-1)[: m * n].copy_(torch.from_numpy(np.ascontiguousarray(out).reshape(-1)))

    def silu_gate_f16(self, device, x, gate, out, rows, cols, x_ld=None, gate_ld=None, out_ld=None):
        res = self.orc.silu_gate_f16(x.numpy(), gate.numpy(), rows, cols, x_ld=x_ld, gate_ld=gate_ld)
        out.view(-1)[: rows * cols].copy_(torch.from_numpy(res.reshape(-1)))


def make_ffn_case(orc, hidden, inter, m, seed=0):
    rng = np.random.default_rng(seed)
    pk = lambda k, n: torch.from_numpy(
        orc.pack_s4(rng.integers(-8, 8, (k, n), dtype=np.int8), k, n).view(np.int32))
    sc = lambda k, n: torch.from_numpy(rng.uniform(0.005, 0.02, (k // 128) * n).astype(np.float16))
    x = torch.from_numpy((rng.standard_normal(m * hidden)).astype(np.float16))
    return dict(x=x, w_gate=pk(hidden, inter), s_gate=sc(hidden, inter), w_up=pk(hidden, inter),
                s_up=sc(hidden, inter), w_down=pk(inter, hidden), s_down=sc(inter, hidden))


def ffn_oracle(orc, case, hidden, inter, m):
    """The unsharded chain, stage by stage, on the CPU oracle."""
    u32 = lambda t: t.numpy().view(np.uint32)
    g = orc.matmul_int4(case["x"].numpy(), u32(case["w_gate"]), case["s_gate"].numpy(), m, inter, hidden, f16_out=True)
    u = orc.matmul_int4(case["x"].numpy(), u32(case["w_up"]), case["s_up"].numpy(), m, inter, hidden, f16_out=True)
    act = orc.silu_gate_f16(np.ascontiguousarray(g).reshape(-1), np.ascontiguousarray(u).reshape(-1), m, inter)
    return np.asarray(orc.matmul_int4(act.reshape(-1), u32(case["w_down"]), case["s_down"].numpy(), m, hidden, inter,
                                      f16_out=False)).reshape(m, hidden)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, hidden, inter, m, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle as orc
        case = make_ffn_case(orc, hidden, inter, m)
        want = ffn_oracle(orc, case, hidden, inter, m)
        weights = [case[n] for n in ("w_gate", "s_gate", "w_up", "s_up", "w_down", "s_down")]
        ok = {}
        for reduce in ("all", "scatter"):
            chain = ffn.FfnInt4(OracleOps(orc), "cpu", hidden, inter, *weights, world=world, rank=rank,
                                max_m=m, reduce=reduce)
            got = chain.run(case["x"], m).numpy()
            ref = want if reduce == "all" else want[rank * (m // world):(rank + 1) * (m // world)]
            err = np.max(np.abs(got - ref) / np.maximum(np.abs(ref), 1.0))
            ok[reduce] = bool(got.shape == ref.shape and err < 1e-5)
        ret[rank] = ok
    finally:
        dist.destroy_process_group()


def test_single_rank_chain_equals_the_stagewise_oracle(oracle):
    hidden, inter, m = 256, 384, 6
    case = make_ffn_case(oracle, hidden, inter, m)
    weights = [case[n] for n in ("w_gate", "s_gate", "w_up", "s_up", "w_down", "s_down")]
    chain = ffn.FfnInt4(OracleOps(oracle), "cpu", hidden, inter, *weights, max_m=8)
    got = chain.run(case["x"], m).numpy()
    assert np.array_equal(got, ffn_oracle(oracle, case, hidden, inter, m))


def test_two_rank_gloo_chain_sums_the_partials(oracle):
    hidden, inter, m, world = 256, 512, 8, 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), hidden, inter, m, ret), nprocs=world, join=True)
    assert dict(ret) == {0: {"all": True, "scatter": True}, 1: {"all": True, "scatter": True}}
