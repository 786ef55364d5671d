"""A device-side wait that runs out becomes a status code on the host, not a hang or a trap.

Every mbarrier wait in the library is bounded; when one gives up the kernel raises its abort
flag, records {code, block, site, kernel} in the device's status block and runs to its normal
end.  The library's self-test kernel takes exactly that path on purpose (one CTA, a barrier that
nothing arrives at, a budget of a few microseconds), so the host side of the protocol can be
checked without faulting the GPU.  The reference has no counterpart: its kernels contain no
device-side waits (kaio-runtime/src/error.rs:4-37 has no timeout variant).
"""
import numpy as np
import pytest
import torch

from kaio_b200 import ops
from kaio_b200.errors import DeviceTimeout
from helpers import dev, device, host

pytestmark = pytest.mark.gpu


def test_wait_that_runs_out_is_reported_and_cleared(oracle):
    d = device()
    assert ops.device_status(d)[0] == 0
    ops.selftest_bounded_wait(d, 5)
    with pytest.raises(DeviceTimeout, match=r"code 1, block 0, site 99, kernel 5"):
        ops.device_status(d)
    # reported once, then clean
    assert ops.device_status(d) == [0, 0, 0, 0]
    # the context is still usable: a GEMM right after is bit-exact
    m, n, k = 256, 256, 128
    data = oracle.lcg_i8(7, m * k + k * n)
    a, b = data[:m * k], data[m * k:]
    want = oracle.matmul_int8(a, b, 0.5, m, n, k)
    c = torch.zeros(m * n, device="cuda", dtype=torch.float32)
    ops.matmul_int8(d, dev(a), dev(b), c, 0.5, m, n, k)
    assert ops.device_status(d)[0] == 0
    assert np.array_equal(host(c, (m, n)), want)


def test_split_k_decode_is_right_after_a_reported_timeout(oracle):
    """The status query also resets the split-K arrival counters, so a split-K launch after a
    reported timeout counts its contributors from zero."""
    d = device()
    m, n, k = 8, 1024, 2048
    rng = np.random.default_rng(11)
    w = rng.integers(-8, 8, k * n, dtype=np.int8)
    a = rng.standard_normal(m * k).astype(np.float16)
    s = rng.uniform(0.005, 0.02, (k // 128) * n).astype(np.float16)
    packed = oracle.pack_s4(w, k, n)
    want = oracle.matmul_int4(a, packed, s, m, n, k)
    c = torch.zeros(m * n, device="cuda", dtype=torch.float32)
    args = (dev(a), dev(packed), dev(s), c, m, n, k, 128)
    ops.matmul_int4(d, *args)  # creates the stream's scratch
    ops.selftest_bounded_wait(d, 3)
    with pytest.raises(DeviceTimeout):
        ops.device_status(d)
    c.zero_()
    ops.matmul_int4(d, *args)
    assert ops.device_status(d)[0] == 0
    got = host(c, (m, n)).astype(np.float64)
    assert np.max(np.abs(got - want) / np.maximum(np.abs(want), 1.0)) < 1e-3


def test_budget_is_validated():
    from kaio_b200 import InvalidConfig
    with pytest.raises(InvalidConfig, match="budget must be"):
        ops.selftest_bounded_wait(device(), 0)
