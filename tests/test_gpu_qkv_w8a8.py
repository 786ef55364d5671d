"""GPU parity of the W8A8 fused QKV projection (kaio_b200_qkv_project_w8a8) against the CPU oracle.

The op has no counterpart in the reference (its INT8 QKV op is W8A16), so the oracle is built
from two reference pieces: the symmetric quantiser of examples/int8_matmul/src/main.rs:41-61
applied per row of x, and the exact-s32 ``cpu_reference`` of
kaio-ops/tests/matmul_int8_e2e.rs:20-34.  Every step is integer or a single correctly rounded
f32/f16 operation, so the bar is bit-equality of the f16 outputs.  Shapes are the reference's
QKV test shapes with K a multiple of 32 (kaio-ops/tests/qkv_project_int8_e2e.rs:196-236) plus
shapes that reach the CTA-pair tensor-core kernel, ragged edges included.
"""
import numpy as np
import pytest
import torch

from kaio_b200 import InvalidConfig, ops
from helpers import dev, device, host

pytestmark = pytest.mark.gpu

CASES = [
    (64, 16, 128, 0xCAFEBABE), (64, 64, 64, 0xFEEDFACE), (128, 64, 64, 0xBEEFF00D), (64, 32, 512, 0xDEADF00D),
    (256, 128, 256, 0xABCDEF01),
    # CTA-pair kernel: whole tiles, ragged M and N, several rounds of tiles
    (200, 256, 1024, 0x1234), (1024, 512, 2048, 0x77), (300, 272, 1056, 0x99), (2048, 1024, 512, 0x5),
]


def run(oracle, m, n, k, x, ws, scales):
    o = [torch.full((m * n,), float("nan"), device="cuda", dtype=torch.float16) for _ in range(3)]
    ops.qkv_project_w8a8(device(), dev(x), *[dev(w) for w in ws], *[dev(s) for s in scales], *o, m, n, k)
    variant = ops.last_variant()
    assert ops.device_status(device())[0] == 0
    for t, w, s in zip(o, ws, scales):
        want = oracle.qkv_w8a8(x, w, s, m, n, k)
        got = host(t, (m, n))
        assert np.array_equal(got.view(np.uint16), want.view(np.uint16)), variant
    return variant


@pytest.mark.parametrize("m,n,k,seed", CASES)
def test_matches_the_oracle_bit_for_bit(oracle, m, n, k, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal(m * k).astype(np.float16)
    x[: k] = 0  # an all-zero row: its scale is 1 by definition
    ws = [rng.integers(-127, 128, k * n, dtype=np.int8) for _ in range(3)]
    scales = [rng.uniform(0.001, 0.01, n).astype(np.float32) for _ in range(3)]
    variant = run(oracle, m, n, k, x, ws, scales)
    assert variant == ("qkv_w8a8_tcgen05_2cta" if m > 128 and n % 16 == 0 else "qkv_w8a8_generic")


def test_projections_are_not_mixed_up(oracle):
    """The 1/2/3 canary of qkv_project_int8_e2e.rs:244-281 in W8A8 form: constant weights 1, 2, 3
    must land in Q, K, V in that order."""
    m, n, k = 256, 256, 512
    x = np.ones(m * k, np.float16)
    ws = [np.full(k * n, v, np.int8) for v in (1, 2, 3)]
    scales = [np.full(n, 1.0 / k, np.float32) for _ in range(3)]
    o = [torch.zeros(m * n, device="cuda", dtype=torch.float16) for _ in range(3)]
    ops.qkv_project_w8a8(device(), dev(x), *[dev(w) for w in ws], *[dev(s) for s in scales], *o, m, n, k)
    for t, e in zip(o, (1.0, 2.0, 3.0)):
        assert np.all(np.abs(host(t).astype(np.float32) - e) < 1e-2)


def test_is_deterministic():
    m, n, k = 512, 512, 1024
    g = torch.Generator(device="cuda")
    g.manual_seed(3)
    x = torch.randn(m * k, device="cuda", generator=g).half()
    ws = [torch.randint(-127, 128, (k * n,), device="cuda", generator=g, dtype=torch.int8) for _ in range(3)]
    sc = [torch.rand(n, device="cuda", generator=g) * 0.009 + 0.001 for _ in range(3)]
    first = None
    for _ in range(20):
        o = [torch.zeros(m * n, device="cuda", dtype=torch.float16) for _ in range(3)]
        ops.qkv_project_w8a8(device(), x, *ws, *sc, *o, m, n, k)
        cat = torch.cat(o)
        if first is None:
            first = cat.clone()
        assert torch.equal(cat.view(torch.int16), first.view(torch.int16))


def test_rejects_bad_arguments():
    d = device()
    m, n, k = 64, 16, 48
    x = torch.zeros(m * k, device="cuda", dtype=torch.float16)
    w = torch.zeros(k * n, device="cuda", dtype=torch.int8)
    s = torch.ones(n, device="cuda")
    o = [torch.zeros(m * n, device="cuda", dtype=torch.float16) for _ in range(3)]
    with pytest.raises(InvalidConfig, match="K must be a multiple of 32"):
        ops.qkv_project_w8a8(d, x, w, w, w, s, s, s, *o, m, n, k)
    k = 64
    x = torch.zeros(m * k, device="cuda", dtype=torch.float16)
    w = torch.zeros(k * n, device="cuda", dtype=torch.int8)
    with pytest.raises(InvalidConfig, match="distinct allocations"):
        ops.qkv_project_w8a8(d, x, w, w, w, s, s, s, o[0], o[0], o[2], m, n, k)
    with pytest.raises(InvalidConfig, match="scale buffers too small"):
        ops.qkv_project_w8a8(d, x, w, w, w, s[:8], s, s, *o, m, n, k)
    with pytest.raises(InvalidConfig, match="W_K buffer too small"):
        ops.qkv_project_w8a8(d, x, w, w[:10], w, s, s, s, *o, m, n, k)
