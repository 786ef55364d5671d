"""GPU parity of kaio_b200_matmul_int4 (+ f16-output extension) against the CPU oracle.

Cases restate kaio-ops/tests/matmul_int4_e2e.rs.  Tolerance: relative error
|g-w|/max(|w|,1) < 1e-3 for f32 output, < 2e-2 for f16 output; the generic kernel keeps
the reference's operation order and must match bit for bit.
"""
import numpy as np
import pytest
import torch

from kaio_b200 import InvalidConfig, ops
from helpers import dev, device, host, max_rel

pytestmark = pytest.mark.gpu
G = 128


def run(oracle, m, n, k, w, a, scales, f16_out=False):
    packed = oracle.pack_s4(w, k, n)
    want = oracle.matmul_int4(a, packed, scales, m, n, k, f16_out=f16_out)
    c = torch.full((m * n,), float("nan"), device="cuda",
                   dtype=torch.float16 if f16_out else torch.float32)
    ops.matmul_int4(device(), dev(a), dev(packed), dev(scales), c, m, n, k, G)
    variant = ops.last_variant()
    assert ops.device_status(device())[0] == 0
    got = host(c, (m, n))
    if variant == "w4a16_generic":
        assert np.array_equal(got, want), variant
    else:
        assert max_rel(got, want) < (2e-2 if f16_out else 1e-3), variant
    return got, want, variant


def ones(m, k):
    return np.ones(m * k, np.float16)


def const_scales(groups, n, v):
    return np.full(groups * n, v, np.float16)


def test_all_ones_is_128(oracle):
    got, _, _ = run(oracle, 16, 8, 128, np.ones(128 * 8, np.int8), ones(16, 128), const_scales(1, 8, 1.0))
    assert np.all(np.abs(got - 128.0) < 1.0)


def test_sign_extend_negative_eights(oracle):
    """matmul_int4_e2e.rs:230-246."""
    for (m, n) in [(16, 8), (16, 64), (1, 256)]:
        got, _, _ = run(oracle, m, n, 128, np.full(128 * n, -8, np.int8), ones(m, 128),
                        const_scales(1, n, 1.0))
        assert np.all(np.abs(got + 1024.0) < 2.0)


def test_sign_extend_mixed_positions(oracle):
    """matmul_int4_e2e.rs:253-278."""
    for n in (8, 64):
        m, k = 16, 128
        w = np.zeros((k, n), np.int8)
        w[0::2, 0] = 7
        w[1::2, 0] = -8
        got, _, _ = run(oracle, m, n, k, w, ones(m, k), const_scales(1, n, 1.0))
        assert np.all(np.abs(got[:, 0] + 64.0) < 2.0) and np.all(np.abs(got[:, 1:]) < 2.0)


def test_nibble_position_canary(oracle):
    """Each k carries a distinct weight/activation pair so any k-permutation mismatch between
    the weight and activation paths changes the result (extends the mixed-position canary)."""
    m, n, k = 16, 64, 256
    w = ((np.arange(k)[:, None] * 5 + np.arange(n)[None, :] * 3) % 16 - 8).astype(np.int8)
    a = ((np.arange(m)[:, None] + 1) * ((np.arange(k)[None, :] % 13) - 6) / 8.0).astype(np.float16)
    run(oracle, m, n, k, w, a.reshape(-1), const_scales(2, n, 0.25))


def test_multi_group_k256(oracle):
    """matmul_int4_e2e.rs:289-308."""
    m, n, k = 32, 32, 256
    scales = np.concatenate([np.full(n, 1.0), np.full(n, 2.0)]).astype(np.float16)
    got, _, _ = run(oracle, m, n, k, np.ones(k * n, np.int8), ones(m, k), scales)
    assert np.all(np.abs(got - 384.0) < 2.0)


@pytest.mark.parametrize("m,n,k,ws,as_,sc", [
    (64, 64, 128, 0xCAFEBABEDEADBEEF, 0x123456789ABCDEF0, 0.1),
    (128, 128, 256, 0xF00DFACED00D1337, 0xA5A55A5AD00DFEED, 0.05),
    (256, 256, 512, 0x0123456789ABCDEF, 0xFEDCBA9876543210, 0.02),
    (17, 8, 128, 0xDEAD0001BEEF0002, 0xFACE0003BEEF0004, 0.1),
    (16, 13, 128, 0x55555555AAAAAAAA, 0x1111222233334444, 0.1),
])
def test_reference_shapes(oracle, m, n, k, ws, as_, sc):
    """matmul_int4_e2e.rs:314-397 (seeded shapes incl. edge M=17 / N=13)."""
    run(oracle, m, n, k, oracle.lcg_s4(ws, k * n), oracle.lcg_f16_pm1(as_, m * k), const_scales(k // G, n, sc))


@pytest.mark.parametrize("m", [1, 2, 8, 16])
@pytest.mark.parametrize("n,k", [(64, 128), (256, 512), (200, 1024), (1000, 384), (11008, 4096)])
@pytest.mark.parametrize("f16_out", [False, True])
def test_decode_shapes(oracle, m, n, k, f16_out):
    """Decode shapes (M <= 16): random group scales, both output forms."""
    rng = np.random.default_rng(m * 131 + n + k)
    w = rng.integers(-8, 8, k * n, dtype=np.int8)
    a = rng.standard_normal(m * k).astype(np.float16)
    scales = rng.uniform(0.005, 0.02, (k // G) * n).astype(np.float16)
    run(oracle, m, n, k, w, a, scales, f16_out=f16_out)


@pytest.mark.parametrize("m", [17, 32, 33, 64, 100, 128, 129, 256, 257, 500])
@pytest.mark.parametrize("n,k", [(200, 384), (1000, 1024), (4096, 2048), (1024, 4096)])
def test_fused_dequant_shapes(oracle, m, n, k):
    """16 < M <= 512 runs the kernel that dequantises inside the GEMM: every row-tile width
    (32 / 64 / 128 / 256 rows, one and several row tiles), ragged rows and columns."""
    rng = np.random.default_rng(m * 7 + n + k)
    w = rng.integers(-8, 8, k * n, dtype=np.int8)
    a = rng.standard_normal(m * k).astype(np.float16)
    scales = rng.uniform(0.005, 0.02, (k // G) * n).astype(np.float16)
    run(oracle, m, n, k, w, a, scales, f16_out=(m % 2 == 0))
    assert ops.last_variant() in ("w4a16_fused_dequant", "w4a16_fused_dequant_splitk")


def test_decode_is_repeatable():
    """The split-K decode kernel sums its partial tiles in a fixed order, so repeated launches
    must agree bit for bit.  Hundreds of launches with varying gaps between them: a stage of the
    weight ring released too early once showed up as a few wrong columns in about one launch
    of 400 on this shape."""
    m, n, k = 16, 11008, 4096
    g = torch.Generator(device="cuda").manual_seed(5)
    w = torch.randint(-2**31, 2**31 - 1, (k // 8 * n,), dtype=torch.int32, device="cuda", generator=g)
    scales = (torch.rand(k // G * n, device="cuda", generator=g) * 0.015 + 0.005).half()
    a = torch.randn(m * k, device="cuda", generator=g).half()
    first = None
    for it in range(600):
        c = torch.full((m * n,), float("nan"), device="cuda")
        if it % 3 == 1:
            torch.cuda.synchronize()
        if it % 5 == 2:
            torch.randn(1 << 20, device="cuda").sum()
        ops.matmul_int4(device(), a, w, scales, c, m, n, k, G)
        if first is None:
            first = c
        else:
            assert torch.equal(c, first), f"launch {it} differs from launch 0"
    assert ops.device_status(device())[0] == 0


@pytest.mark.parametrize("m,n,k", [(48, 512, 1024), (300, 384, 640), (1024, 256, 4096)])
def test_prefill_shapes(oracle, m, n, k):
    rng = np.random.default_rng(n + k)
    w = rng.integers(-8, 8, k * n, dtype=np.int8)
    a = rng.standard_normal(m * k).astype(np.float16)
    scales = rng.uniform(0.005, 0.02, (k // G) * n).astype(np.float16)
    run(oracle, m, n, k, w, a, scales)
    run(oracle, m, n, k, w, a, scales, f16_out=True)


def test_decode_determinism(oracle):
    """Split-K must reduce in a fixed order: 100 launches, identical bits."""
    m, n, k = 16, 2048, 4096
    rng = np.random.default_rng(1)
    packed = dev(oracle.pack_s4(rng.integers(-8, 8, k * n, dtype=np.int8), k, n))
    a = dev(rng.standard_normal(m * k).astype(np.float16))
    s = dev(rng.uniform(0.005, 0.02, (k // G) * n).astype(np.float16))
    first = None
    for _ in range(100):
        c = torch.zeros(m * n, device="cuda", dtype=torch.float32)
        ops.matmul_int4(device(), a, packed, s, c, m, n, k, G)
        if first is None:
            first = c
        else:
            assert torch.equal(first, c)


def test_rejects_bad_arguments():
    d = device()
    a = torch.zeros(16 * 128, device="cuda", dtype=torch.float16)
    b = torch.zeros(16 * 8, device="cuda", dtype=torch.int32)
    s = torch.zeros(8, device="cuda", dtype=torch.float16)
    c = torch.zeros(16 * 8, device="cuda", dtype=torch.float32)
    with pytest.raises(InvalidConfig, match="K must be a multiple of group_size"):
        ops.matmul_int4(d, a, b, s, c, 16, 8, 127, 128)
    with pytest.raises(InvalidConfig, match="group_size must be 128"):
        ops.matmul_int4(d, a, b, s, c, 16, 8, 128, 64)
    with pytest.raises(InvalidConfig):
        ops.matmul_int4(d, a, b, s, c, 0, 8, 128, 128)
    with pytest.raises(InvalidConfig, match="scales buffer too small"):
        ops.matmul_int4(d, a, b, s[:3], c, 16, 8, 128, 128)


@pytest.mark.parametrize("m", [8, 200])
def test_allgather_form_with_local_destinations(oracle, m):
    """The sharded all-gather entry point on one GPU: two local buffers stand in for the ranks'
    output buffers; 'rank 1 of 2' must write its shard into columns [N/2, N) of both and touch
    nothing else."""
    n, k, world, rank = 512, 512, 2, 1
    rng = np.random.default_rng(m)
    w = rng.integers(-8, 8, (k, n), dtype=np.int8)
    a = rng.standard_normal(m * k).astype(np.float16)
    sc = rng.uniform(0.005, 0.02, (k // G) * n).astype(np.float16)
    n_loc = n // world
    lo = rank * n_loc
    w_loc = np.ascontiguousarray(w[:, lo:lo + n_loc])
    sc_loc = np.ascontiguousarray(sc.reshape(-1, n)[:, lo:lo + n_loc]).reshape(-1)
    want = oracle.matmul_int4(a, oracle.pack_s4(w_loc, k, n_loc), sc_loc, m, n_loc, k, f16_out=True)
    bufs = [torch.full((m * n,), 7.0, device="cuda", dtype=torch.float16) for _ in range(world)]
    ops.matmul_int4_allgather(device(), dev(a), dev(oracle.pack_s4(w_loc, k, n_loc)), dev(sc_loc),
                              [b.data_ptr() for b in bufs], m * n, world, rank, m, n, k)
    assert ops.device_status(device())[0] == 0
    for b in bufs:
        got = host(b, (m, n)).astype(np.float32)
        assert np.all(got[:, :lo] == 7.0)
        assert max_rel(got[:, lo:], want.astype(np.float32)) < 2e-2
