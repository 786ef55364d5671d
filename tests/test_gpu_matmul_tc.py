"""GPU parity of kaio_b200_matmul_tc / matmul_tc_async against the CPU oracle.

Cases restate kaio-ops/tests/matmul_tc_api.rs (patterned inputs scaled to |x| <= 1, the ragged
and off-by-one shapes, the per-cell canary); tolerance is the reference's K-scaled bound
K * 2^-10 * max|a| * max|b| (kaio-ops/tests/common/mod.rs:56-113).
"""
import numpy as np
import pytest
import torch

from kaio_b200 import InvalidConfig, ops
from helpers import dev, device, host

pytestmark = pytest.mark.gpu


def check(oracle, m, n, k, a, b, fn=None, rows=None):
    c = torch.full((m * n,), float("nan"), device="cuda", dtype=torch.float32)
    (fn or ops.matmul_tc)(device(), dev(a), dev(b), c, m, n, k)
    variant = ops.last_variant()
    assert ops.device_status(device())[0] == 0
    got = host(c, (m, n))
    tol = k * 2.0 ** -10 * float(np.abs(a.astype(np.float32)).max()) * float(np.abs(b.astype(np.float32)).max())
    if rows is None:
        want = oracle.matmul_f16(a, b, m, n, k)
        assert float(np.abs(got - want).max()) < tol, variant
    else:
        want = oracle.matmul_f16(a.reshape(m, k)[rows], b, len(rows), n, k)
        assert float(np.abs(got[rows] - want).max()) < tol, variant
    return variant


# matmul_tc_api.rs:46-125 (tiny ... large off-by-one) plus shapes for the tcgen05 path
SHAPES = [(16, 8, 16), (32, 16, 32), (128, 8, 16), (64, 64, 64), (7, 5, 16), (15, 7, 16), (17, 9, 16),
          (33, 17, 16), (100, 50, 64), (1023, 1023, 1024),
          (256, 256, 256), (300, 528, 1056), (1024, 1024, 1024), (129, 136, 48)]


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_patterned(oracle, m, n, k):
    variant = check(oracle, m, n, k, oracle.patterned_f16(m * k), oracle.patterned_f16(k * n))
    assert variant == ("f16_tcgen05" if n % 8 == 0 else "f16_generic")


def test_async_entry_point(oracle):
    m, n, k = 128, 256, 512
    check(oracle, m, n, k, oracle.patterned_f16(m * k), oracle.patterned_f16(k * n), fn=ops.matmul_tc_async)


def test_quadrant_canary(oracle):
    """matmul_tc_api.rs:127-170: A[i,:] = (i+1) * 0.01, B[:,j] = (j+1) * 0.01, so cell (i,j) is
    (i+1) (j+1) K * 1e-4 and any mis-routed tile shows up at its cell."""
    m = n = k = 64
    a = np.repeat(((np.arange(m) + 1) * 0.01).astype(np.float16)[:, None], k, 1).reshape(-1)
    b = np.repeat(((np.arange(n) + 1) * 0.01).astype(np.float16)[None, :], k, 0).reshape(-1)
    check(oracle, m, n, k, a, b)
    c = torch.zeros(m * n, device="cuda")
    ops.matmul_tc(device(), dev(a), dev(b), c, m, n, k)
    got = host(c, (m, n))
    want = (a.reshape(m, k)[:, :1].astype(np.float32) * b.reshape(k, n)[:1, :].astype(np.float32)) * k
    assert np.allclose(got, want, rtol=2e-3)


def test_large_sampled_rows(oracle):
    m, n, k = 4096, 4096, 4096
    rng = np.random.default_rng(11)
    a = rng.uniform(-1, 1, m * k).astype(np.float16)
    b = rng.uniform(-1, 1, k * n).astype(np.float16)
    check(oracle, m, n, k, a, b, rows=[0, 127, 128, 2049, 4095])


def test_rejects_bad_arguments():
    d = device()
    a = torch.zeros(16 * 16, device="cuda", dtype=torch.float16)
    c = torch.zeros(16 * 8, device="cuda")
    with pytest.raises(InvalidConfig, match="K must be a multiple of 16"):
        ops.matmul_tc(d, a, a, c, 16, 8, 24)
    with pytest.raises(InvalidConfig, match="dimensions must be non-zero"):
        ops.matmul_tc(d, a, a, c, 0, 8, 16)
    with pytest.raises(InvalidConfig, match="B buffer too small"):
        ops.matmul_tc(d, a, a[:10], c, 16, 8, 16)
    with pytest.raises(InvalidConfig, match="C buffer too small"):
        ops.matmul_tc(d, a, a, c[:10], 16, 8, 16)


def test_allgather_cols_single_rank_is_a_copy():
    """kaio_b200_allgather_cols with one rank: the shard is the whole matrix (no NCCL call);
    argument checks as for the other entry points."""
    from kaio_b200 import InvalidConfig
    m, n = 37, 256
    shard = torch.randn(m * n, device="cuda").half()
    out = torch.zeros(m * n, device="cuda", dtype=torch.float16)
    ops.allgather_cols(device(), shard, out, m, n, 1, nccl_comm=1)  # the communicator is not used
    assert ops.last_variant() == "allgather_cols_copy"
    assert torch.equal(out, shard)
    with pytest.raises(InvalidConfig, match="must split into"):
        ops.allgather_cols(device(), shard, out, m, n, 3, nccl_comm=1)
    with pytest.raises(InvalidConfig, match="out buffer too small"):
        ops.allgather_cols(device(), shard, out[:100], m, n, 1, nccl_comm=1)
