"""GPU quantisers against the CPU restatement of the reference's host quantisers
(examples/int8_matmul/src/main.rs:41-61, examples/int4_matmul/src/main.rs:48-99): bit-exact."""
import numpy as np
import pytest
import torch

from kaio_b200 import InvalidConfig, ops
from helpers import dev, device, host

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,k", [(1, 32), (17, 96), (300, 4096), (64, 11008)])
def test_quantize_rows_int8(oracle, m, k):
    rng = np.random.default_rng(m + k)
    x = (rng.standard_normal((m, k)) * rng.uniform(0.1, 5.0, (m, 1))).astype(np.float32)
    if m > 1:
        x[1] = 0.0  # all-zero row: scale 1
    x[0, 0] = 0.5 * np.abs(x[0]).max() / 127 * 3  # lands on a .5 tie after scaling more often than chance
    q_want, s_want = oracle.quantize_rows_int8(x, m, k)
    q = torch.zeros(m * k, device="cuda", dtype=torch.int8)
    s = torch.zeros(m, device="cuda", dtype=torch.float32)
    ops.quantize_rows_int8(device(), dev(x), q, s, m, k)
    assert np.array_equal(host(s), s_want)
    assert np.array_equal(host(q, (m, k)), q_want)


@pytest.mark.parametrize("k,n", [(128, 8), (256, 13), (1024, 300), (4096, 1024)])
def test_quantize_pack_int4(oracle, k, n):
    rng = np.random.default_rng(k + n)
    w = (rng.standard_normal((k, n)) * 0.05).astype(np.float32)
    w[:128, 0] = 0.0  # an all-zero group: scale 1, nibbles 0
    q_want, sc_want = oracle.quantize_gptq_lite(w, k, n)
    packed_want = oracle.pack_s4(q_want, k, n)
    packed = torch.zeros((k // 8) * n, device="cuda", dtype=torch.int32)
    scales = torch.zeros((k // 128) * n, device="cuda", dtype=torch.float16)
    ops.quantize_pack_int4(device(), dev(w), packed, scales, k, n)
    assert np.array_equal(host(scales), sc_want)
    assert np.array_equal(host(packed).view(np.uint32), packed_want)


def test_quantized_pipeline_end_to_end(oracle):
    """f32 activations and weights -> GPU quantisers -> W4A16 / W8A8 GEMMs: same result as the
    oracle run on the oracle's quantised operands."""
    m, k, n = 48, 512, 256
    rng = np.random.default_rng(5)
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((k, n)) * 0.05).astype(np.float32)
    d = device()
    packed = torch.zeros((k // 8) * n, device="cuda", dtype=torch.int32)
    scales = torch.zeros((k // 128) * n, device="cuda", dtype=torch.float16)
    ops.quantize_pack_int4(d, dev(w), packed, scales, k, n)
    c = torch.zeros(m * n, device="cuda", dtype=torch.float32)
    ops.matmul_int4(d, dev(x.astype(np.float16)), packed, scales, c, m, n, k, 128)
    q_w, sc = oracle.quantize_gptq_lite(w, k, n)
    want = oracle.matmul_int4(x.astype(np.float16), oracle.pack_s4(q_w, k, n), sc, m, n, k)
    got = host(c, (m, n))
    assert np.max(np.abs(got - want) / np.maximum(np.abs(want), 1.0)) < 1e-3
    # W8A8 with per-row activation scales from the GPU quantiser
    xq = torch.zeros(m * k, device="cuda", dtype=torch.int8)
    xs = torch.zeros(m, device="cuda", dtype=torch.float32)
    ops.quantize_rows_int8(d, dev(x), xq, xs, m, k)
    wq8 = rng.integers(-127, 128, (k, n), dtype=np.int8)
    ws = rng.uniform(0.001, 0.01, n).astype(np.float32)
    c8 = torch.zeros(m * n, device="cuda", dtype=torch.float32)
    ops.matmul_int8_scaled(d, xq, dev(wq8), c8, xs, dev(ws), m, n, k)
    xq_want, xs_want = oracle.quantize_rows_int8(x, m, k)
    want8 = oracle.matmul_int8_scaled(xq_want, wq8, xs_want, ws, m, n, k)
    assert np.array_equal(host(c8, (m, n)), want8)


def test_rejects_bad_arguments():
    d = device()
    w = torch.zeros(128 * 8, device="cuda", dtype=torch.float32)
    p = torch.zeros(16 * 8, device="cuda", dtype=torch.int32)
    s = torch.zeros(8, device="cuda", dtype=torch.float16)
    with pytest.raises(InvalidConfig, match="K must be a multiple of group_size"):
        ops.quantize_pack_int4(d, w, p, s, 100, 8)
    with pytest.raises(InvalidConfig, match="packed buffer too small"):
        ops.quantize_pack_int4(d, w, p[:4], s, 128, 8)
