"""GPU parity of the fused QKV projections against the CPU oracle.

Cases restate kaio-ops/tests/qkv_project_int8_e2e.rs and qkv_project_int4_e2e.rs; tolerance
is the reference's: |g-w|/max(|w|,1) < 1e-3 on the f16 outputs (tighter than the 2e-2 the
f16 output form is allowed).
"""
import numpy as np
import pytest
import torch

from kaio_b200 import InvalidConfig, ops
from helpers import dev, device, host, max_rel

pytestmark = pytest.mark.gpu
G = 128
TOL = 1e-3


def outs(m, n):
    return [torch.full((m * n,), float("nan"), device="cuda", dtype=torch.float16) for _ in range(3)]


def run_int8(oracle, m, n, k, x, ws, scales):
    o = outs(m, n)
    col = isinstance(scales[0], np.ndarray)
    sc = [dev(s) for s in scales] if col else list(scales)
    ops.qkv_project_int8(device(), dev(x), *[dev(w) for w in ws], *sc, *o, m, n, k)
    variant = ops.last_variant()
    assert ops.device_status(device())[0] == 0
    got = [host(t, (m, n)) for t in o]
    for g, w, s in zip(got, ws, scales):
        want = oracle.qkv_int8(x, w, 0.0 if col else s, m, n, k, col_scale=s if col else None)
        if variant.endswith("generic"):
            assert np.array_equal(g, want), variant
        else:
            assert max_rel(g, want) < TOL, variant
    return got


def run_int4(oracle, m, n, k, x, ws, scales):
    o = outs(m, n)
    packed = [oracle.pack_s4(w, k, n) for w in ws]
    ops.qkv_project_int4(device(), dev(x), *[dev(p) for p in packed], *[dev(s) for s in scales], *o,
                         m, n, k, G)
    variant = ops.last_variant()
    assert ops.device_status(device())[0] == 0
    got = [host(t, (m, n)) for t in o]
    for g, p, s in zip(got, packed, scales):
        want = oracle.qkv_int4(x, p, s, m, n, k)
        if variant.endswith("generic"):
            assert np.array_equal(g, want), variant
        else:
            assert max_rel(g, want) < TOL, variant
    return got


INT8_CASES = [  # qkv_project_int8_e2e.rs:196-236
    (64, 16, 16, 0xDEADBEEF), (64, 16, 128, 0xCAFEBABE), (64, 64, 64, 0xFEEDFACE),
    (128, 64, 64, 0xBEEFF00D), (64, 32, 512, 0xDEADF00D), (256, 128, 256, 0xABCDEF01),
    # larger / ragged shapes for the tcgen05 path
    (200, 256, 1024, 0x1234), (1024, 512, 2048, 0x77), (130, 136, 144, 0x99),
]


@pytest.mark.parametrize("m,n,k,seed", INT8_CASES)
def test_int8_correctness(oracle, m, n, k, seed):
    x = oracle.lcg_f16_pm_half(seed, m * k)
    ws = [oracle.lcg_i8_div4(seed + i, k * n) for i in (1, 2, 3)]
    run_int8(oracle, m, n, k, x, ws, [1.0 / k] * 3)


def test_int8_differentiation_canary(oracle):
    m, n, k = 64, 32, 128
    x = np.ones(m * k, np.float16)
    got = run_int8(oracle, m, n, k, x, [np.full(k * n, v, np.int8) for v in (1, 2, 3)], [1.0 / k] * 3)
    for g, e in zip(got, (1.0, 2.0, 3.0)):
        assert np.all(np.abs(g.astype(np.float32) - e) < 1e-2)


@pytest.mark.parametrize("m,n,k", [(64, 16, 32), (64, 16, 48), (256, 256, 384)])
def test_int8_slot_mapping_canary(oracle, m, n, k):
    """qkv_project_int8_e2e.rs:308-372: exactly K, 2K, 3K."""
    x = np.ones(m * k, np.float16)
    got = run_int8(oracle, m, n, k, x, [np.full(k * n, v, np.int8) for v in (1, 2, 3)], [1.0] * 3)
    for g, e in zip(got, (k, 2 * k, 3 * k)):
        assert np.all(g.astype(np.float32) == float(e))


def test_int8_colscale_extension(oracle):
    rng = np.random.default_rng(8)
    for (m, n, k) in [(64, 32, 64), (300, 256, 1024)]:
        x = rng.standard_normal(m * k).astype(np.float16)
        ws = [rng.integers(-127, 128, k * n, dtype=np.int8) for _ in range(3)]
        scales = [rng.uniform(0.001, 0.01, n).astype(np.float32) for _ in range(3)]
        run_int8(oracle, m, n, k, x, ws, scales)


INT4_CASES = [  # qkv_project_int4_e2e.rs:263-310
    (64, 16, 128, 0xA1), (64, 16, 256, 0xA2), (64, 16, 1024, 0xA3), (64, 64, 128, 0xA4),
    (128, 32, 128, 0xA5), (128, 128, 256, 0xA6),
    (200, 256, 1024, 0xA7), (1024, 512, 2048, 0xA8), (130, 136, 384, 0xA9),
    # decode-like fused QKV: few column tiles and a long K (the fused-dequant kernel runs stream-K)
    (64, 512, 4096, 0xAA), (24, 256, 8192, 0xAB),
]


@pytest.mark.parametrize("m,n,k,seed", INT4_CASES)
def test_int4_correctness(oracle, m, n, k, seed):
    x = oracle.lcg_f16_pm_half(seed, m * k)
    ws = [oracle.lcg_s4(seed + i, k * n) for i in (1, 2, 3)]
    scales = [oracle.lcg_small_scales(seed + i, (k // G) * n) for i in (4, 5, 6)]
    run_int4(oracle, m, n, k, x, ws, scales)


def test_int4_canaries(oracle):
    m, n, k = 64, 16, 128
    x = np.ones(m * k, np.float16)
    one = np.ones(n, np.float16)
    got = run_int4(oracle, m, n, k, x, [np.full(k * n, -8, np.int8)] * 3, [one] * 3)
    for g in got:
        assert np.all(np.abs(g.astype(np.float32) + 1024.0) < 4.0)
    inv_k = np.full(n, 1.0 / k, np.float16)
    got = run_int4(oracle, m, 32, k, np.ones(m * k, np.float16),
                   [np.full(k * 32, v, np.int8) for v in (1, 2, 3)], [np.full(32, 1.0 / k, np.float16)] * 3)
    for g, e in zip(got, (1.0, 2.0, 3.0)):
        assert np.all(np.abs(g.astype(np.float32) - e) < 1e-2)
    del inv_k


def test_determinism_100_launches(oracle):
    """qkv_project_int8_e2e.rs:397-492 (short shape)."""
    m, n, k = 256, 512, 1024
    x = dev(oracle.lcg_f16_pm_half(0xDEADBEEF, m * k))
    ws = [dev(oracle.lcg_i8_div4(s, k * n)) for s in (0x11111111, 0x22222222, 0x33333333)]
    first = None
    for _ in range(100):
        o = outs(m, n)
        ops.qkv_project_int8(device(), x, *ws, 1.0 / k, 1.0 / k, 1.0 / k, *o, m, n, k)
        if first is None:
            first = o
        else:
            for a, b in zip(first, o):
                assert torch.equal(a.view(torch.int16), b.view(torch.int16))


def test_rejects_bad_arguments():
    d = device()
    x = torch.zeros(64 * 16, device="cuda", dtype=torch.float16)
    w = torch.zeros(16 * 16, device="cuda", dtype=torch.int8)
    o = outs(64, 16)
    with pytest.raises(InvalidConfig, match="N must be even"):
        ops.qkv_project_int8(d, x, w, w, w, 1.0, 1.0, 1.0, *o, 64, 15, 16)
    with pytest.raises(InvalidConfig, match="K must be a multiple of K_TILE_SHARED"):
        ops.qkv_project_int8(d, x, w, w, w, 1.0, 1.0, 1.0, *o, 64, 16, 24)
    with pytest.raises(InvalidConfig, match="distinct"):
        ops.qkv_project_int8(d, x, w, w, w, 1.0, 1.0, 1.0, o[0], o[0], o[2], 64, 16, 16)
    with pytest.raises(InvalidConfig, match="W_K buffer too small"):
        ops.qkv_project_int8(d, x, w, w[:8], w, 1.0, 1.0, 1.0, *o, 64, 16, 16)
