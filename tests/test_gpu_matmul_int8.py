"""GPU parity of kaio_b200_matmul_int8 (+ extensions) against the CPU oracle.

Cases restate kaio-ops/tests/matmul_int8_e2e.rs; accumulators are compared bit for bit and,
because the epilogue is one cast and one (or two) f32 multiplies, so are the f32 outputs.
"""
import numpy as np
import pytest
import torch

from kaio_b200 import InvalidConfig, ops
from helpers import dev, device, host

pytestmark = pytest.mark.gpu

SHAPES = [
    # (m, n, k, scale, seed) -- matmul_int8_e2e.rs:72-146
    (16, 8, 32, 1.0, 0xA5A55A5AD00DFEED),
    (64, 64, 32, 0.5, 0x123456789ABCDEF0),
    (64, 64, 128, 0.125, 0xCAFEBABEDEADBEEF),
    (128, 128, 128, 0.01, 0x0123456789ABCDEF),
    (256, 256, 256, 0.001, 0xF00DFACED00D1337),
    (17, 8, 32, 1.0, 0xDEAD0001BEEF0002),
    (16, 13, 32, 1.0, 0xFACE0003BEEF0004),
    # shapes that exercise the tcgen05 path's edges: ragged M/N tiles, K not a multiple of 128,
    # more tiles than SMs, several K blocks around the 4-stage ring
    (17, 16, 32, 1.0, 1), (128, 256, 128, 0.5, 2), (129, 272, 160, 0.25, 3),
    (300, 528, 1056, 0.01, 4), (1024, 1024, 1024, 0.01, 42), (2000, 4112, 96, 0.02, 5),
    # 90 tiles on 74 pairs: the 16 left-over tiles run as 32 half-width tiles; ragged last column
    (2304, 2560, 256, 0.01, 77), (2304, 2448, 384, 0.01, 78),
]


def run_case(oracle, m, n, k, scale, seed):
    data = oracle.lcg_i8(seed, m * k + k * n)
    a, b = data[:m * k], data[m * k:]
    want, want_acc = oracle.matmul_int8(a, b, scale, m, n, k, want_acc=True)
    d = device()
    ad, bd = dev(a), dev(b)
    c = torch.full((m * n,), float("nan"), device="cuda", dtype=torch.float32)
    acc = torch.full((m * n,), -7, device="cuda", dtype=torch.int32)
    ops.matmul_int8(d, ad, bd, c, scale, m, n, k)
    variant = ops.last_variant()
    ops.matmul_int8_acc(d, ad, bd, acc, m, n, k)
    assert ops.device_status(d)[0] == 0
    assert np.array_equal(host(acc, (m, n)), want_acc), variant
    assert np.array_equal(host(c, (m, n)), want), variant
    return variant


@pytest.mark.parametrize("m,n,k,scale,seed", SHAPES)
def test_round_trip(oracle, m, n, k, scale, seed):
    variant = run_case(oracle, m, n, k, scale, seed)
    expect = ("w8a8_tcgen05_2cta" if m > 128 else "w8a8_tcgen05") if n % 16 == 0 else "int8_generic"
    assert variant == expect


def test_boundary_values(oracle):
    """matmul_int8_e2e.rs:169-202, run at N=16 so the tcgen05 path sees it too."""
    for n in (8, 16):
        m, k = 16, 32
        a = np.zeros((m, k), np.int8)
        a[0, :5] = [-128, 127, -1, 0, 1]
        a[0, 5:] = np.arange(k - 5)
        a[3, :] = -128
        b = np.zeros((k, n), np.int8)
        b[:, 0] = 1
        b[:, 1] = np.where(np.arange(k) % 2 == 0, 1, -1)
        b[:, 2] = -128
        want, want_acc = oracle.matmul_int8(a, b, 1.0, m, n, k, want_acc=True)
        c = torch.zeros(m * n, device="cuda", dtype=torch.float32)
        ops.matmul_int8(device(), dev(a), dev(b), c, 1.0, m, n, k)
        assert np.array_equal(host(c, (m, n)), want)
        assert want_acc[3, 2] == 128 * 128 * k


def test_rowcol_scaled_extension(oracle):
    rng = np.random.default_rng(4242)
    for (m, n, k) in [(50, 48, 64), (300, 528, 1056), (33, 13, 32)]:
        a = rng.integers(-127, 128, (m, k), dtype=np.int8)
        b = rng.integers(-127, 128, (k, n), dtype=np.int8)
        sa = rng.uniform(0.001, 0.01, m).astype(np.float32)
        sw = rng.uniform(0.001, 0.01, n).astype(np.float32)
        want = oracle.matmul_int8_scaled(a, b, sa, sw, m, n, k)
        c = torch.zeros(m * n, device="cuda", dtype=torch.float32)
        ops.matmul_int8_scaled(device(), dev(a), dev(b), c, dev(sa), dev(sw), m, n, k)
        assert np.array_equal(host(c, (m, n)), want), ops.last_variant()


def test_oversized_buffers_and_untouched_tail(oracle):
    """Buffers may be longer than the shape needs; only [0, m*n) of C is written."""
    m, n, k = 40, 32, 64
    data = oracle.lcg_i8(9, m * k + k * n)
    a, b = data[:m * k], data[m * k:]
    pad = 1000
    ad = dev(np.concatenate([a, np.full(pad, 77, np.int8)]))
    bd = dev(np.concatenate([b, np.full(pad, 77, np.int8)]))
    c = torch.full((m * n + pad,), 123.0, device="cuda", dtype=torch.float32)
    ops.matmul_int8(device(), ad, bd, c, 0.5, m, n, k)
    got = host(c)
    assert np.array_equal(got[:m * n].reshape(m, n), oracle.matmul_int8(a, b, 0.5, m, n, k))
    assert np.all(got[m * n:] == 123.0)


def test_rejects_bad_arguments():
    d = device()
    z8 = torch.zeros(16 * 32, device="cuda", dtype=torch.int8)
    c = torch.zeros(16 * 8, device="cuda", dtype=torch.float32)
    with pytest.raises(InvalidConfig, match="K must be a multiple of 32"):
        ops.matmul_int8(d, z8, z8, c, 1.0, 16, 8, 31)
    with pytest.raises(InvalidConfig, match="dimensions must be non-zero"):
        ops.matmul_int8(d, z8, z8, c, 1.0, 0, 8, 32)
    with pytest.raises(InvalidConfig, match="A buffer too small"):
        ops.matmul_int8(d, z8[:10], z8, c, 1.0, 16, 8, 32)
    with pytest.raises(InvalidConfig, match="C buffer too small"):
        ops.matmul_int8(d, z8, z8, c[:5], 1.0, 16, 8, 32)


def test_determinism_100_launches(oracle):
    """Cross-launch bit-exactness (the reference's stress, qkv_project_int8_e2e.rs:397-492)."""
    m, n, k = 512, 768, 1024
    data = oracle.lcg_i8(77, m * k + k * n)
    ad, bd = dev(data[:m * k]), dev(data[m * k:])
    first = None
    for _ in range(100):
        c = torch.zeros(m * n, device="cuda", dtype=torch.float32)
        ops.matmul_int8(device(), ad, bd, c, 0.01, m, n, k)
        if first is None:
            first = c
        else:
            assert torch.equal(first, c)
