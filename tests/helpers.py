"""Shared helpers of the GPU parity tests: numpy <-> device buffers and comparators."""
import numpy as np
import torch

from kaio_b200 import ops


def dev(arr: np.ndarray) -> torch.Tensor:
    """numpy array -> flat CUDA tensor with the same bits (u32 travels as int32)."""
    arr = np.ascontiguousarray(arr)
    if arr.dtype == np.uint32:
        arr = arr.view(np.int32)
    return torch.from_numpy(arr.reshape(-1)).cuda()


def host(t: torch.Tensor, shape=None) -> np.ndarray:
    a = t.detach().cpu().numpy()
    return a if shape is None else a.reshape(shape)


def device():
    return ops.KaioDevice(0)


def max_rel(got, want):
    """The reference's relative error: |g-w| / max(|w|, 1) (matmul_int4_e2e.rs:141-160)."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    return float(np.max(np.abs(got - want) / np.maximum(np.abs(want), 1.0)))


def assert_attention_close(got, want, abs_tol=5e-3, rel_tol=2e-2):
    """abs < 5e-3 OR rel < 2e-2 per element (kaio-ops/tests/common/mod.rs:249-284)."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    abs_err = np.abs(got - want)
    rel_err = np.where(np.abs(want) > 1e-6, abs_err / np.maximum(np.abs(want), 1e-30), abs_err)
    bad = ~((abs_err < abs_tol) | (rel_err < rel_tol))
    assert not bad.any(), f"{bad.sum()} elements out of tolerance; max abs {abs_err.max():.3e}"
