"""ctypes binding for the CPU oracle (``kaio_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the
CPU-baseline legs of ``bench.py``.  The shipped package never imports it.

All f16 data crosses this boundary as ``numpy.float16`` arrays (bit-identical
to ``half::f16``); packed INT4 weights as ``numpy.uint32``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "kaio_oracle.c")
_SO = os.path.join(_HERE, "libkaio_oracle.so")


def build(force: bool = False) -> str:
    """Compile ``kaio_oracle.c`` with gcc into ``libkaio_oracle.so`` (in place)."""
    if not force and os.path.exists(_SO) and os.path.getmtime(_SO) >= os.path.getmtime(_SRC):
        return _SO
    cmd = [
        "gcc", "-O2", "-fopenmp", "-fPIC", "-shared", "-std=c11",
        "-ffp-contract=off", "-fno-fast-math", "-fvisibility=hidden",
        "-o", _SO, _SRC, "-lm",
    ]
    subprocess.run(cmd, check=True)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = C.CDLL(_SO)
        _lib.kaio_oracle_f16_to_f32.restype = C.c_float
        _lib.kaio_oracle_f16_to_f32.argtypes = [C.c_uint16]
        _lib.kaio_oracle_f32_to_f16.restype = C.c_uint16
        _lib.kaio_oracle_f32_to_f16.argtypes = [C.c_float]
        _lib.kaio_oracle_num_threads.restype = C.c_int
    return _lib


def set_threads(n: int) -> int:
    """Use ``n`` OpenMP threads from now on; returns the count now in effect."""
    lib().kaio_oracle_set_threads(C.c_int(int(n)))
    return num_threads()


def _p(a: np.ndarray | None):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.c_void_p)


def _rows(m, rows):
    r0, r1 = (0, m) if rows is None else rows
    assert 0 <= r0 <= r1 <= m
    return C.c_uint32(r0), C.c_uint32(r1)


def num_threads() -> int:
    return int(lib().kaio_oracle_num_threads())


def f16_to_f32(bits: int) -> float:
    return float(lib().kaio_oracle_f16_to_f32(bits))


def f32_to_f16(x: float) -> int:
    return int(lib().kaio_oracle_f32_to_f16(C.c_float(x)))


def matmul_f16(a, b, m, n, k, rows=None):
    """f16 x f16 -> f32, f32 accumulation -- kaio-ops/tests/common/mod.rs:37-54."""
    a = np.ascontiguousarray(a, dtype=np.float16)
    b = np.ascontiguousarray(b, dtype=np.float16)
    out = np.zeros((m, n), dtype=np.float32)
    r0, r1 = _rows(m, rows)
    lib().kaio_oracle_matmul_f16(_p(a), _p(b), C.c_uint32(m), C.c_uint32(n), C.c_uint32(k), r0, r1, _p(out))
    return out


def matmul_int8(a, b, scale, m, n, k, rows=None, want_acc=False):
    """``(acc as f32) * scale`` -- kaio-ops/tests/matmul_int8_e2e.rs:20-34."""
    a = np.ascontiguousarray(a, dtype=np.int8)
    b = np.ascontiguousarray(b, dtype=np.int8)
    out = np.zeros((m, n), dtype=np.float32)
    acc = np.zeros((m, n), dtype=np.int32) if want_acc else None
    r0, r1 = _rows(m, rows)
    lib().kaio_oracle_matmul_int8(_p(a), _p(b), C.c_float(scale), C.c_uint32(m), C.c_uint32(n),
                                  C.c_uint32(k), r0, r1, _p(out), _p(acc))
    return (out, acc) if want_acc else out


def matmul_int8_scaled(a, b, a_scale, w_scale, m, n, k, rows=None):
    """Extended: ``((acc as f32) * a_scale[i]) * w_scale[j]`` (no KAIO counterpart)."""
    a = np.ascontiguousarray(a, dtype=np.int8)
    b = np.ascontiguousarray(b, dtype=np.int8)
    a_scale = np.ascontiguousarray(a_scale, dtype=np.float32)
    w_scale = np.ascontiguousarray(w_scale, dtype=np.float32)
    out = np.zeros((m, n), dtype=np.float32)
    r0, r1 = _rows(m, rows)
    lib().kaio_oracle_matmul_int8_scaled(_p(a), _p(b), _p(a_scale), _p(w_scale), C.c_uint32(m),
                                         C.c_uint32(n), C.c_uint32(k), r0, r1, _p(out))
    return out


def pack_s4(w, k, n):
    """Logical [K,N] int4 values -> u32[(K/8)*N] -- kaio-ops/tests/matmul_int4_e2e.rs:37-54."""
    w = np.ascontiguousarray(w, dtype=np.int8).reshape(k, n)
    assert k % 8 == 0
    out = np.zeros((k // 8) * n, dtype=np.uint32)
    lib().kaio_oracle_pack_s4(_p(w), C.c_uint32(k), C.c_uint32(n), _p(out))
    return out


def matmul_int4(a, packed, scales, m, n, k, group_size=128, rows=None, f16_out=False):
    """kaio-ops/tests/matmul_int4_e2e.rs:60-95; ``f16_out`` adds the final f16 narrow."""
    a = np.ascontiguousarray(a, dtype=np.float16)
    packed = np.ascontiguousarray(packed, dtype=np.uint32)
    scales = np.ascontiguousarray(scales, dtype=np.float16)
    o32 = None if f16_out else np.zeros((m, n), dtype=np.float32)
    o16 = np.zeros((m, n), dtype=np.float16) if f16_out else None
    r0, r1 = _rows(m, rows)
    lib().kaio_oracle_matmul_int4(_p(a), _p(packed), _p(scales), C.c_uint32(m), C.c_uint32(n),
                                  C.c_uint32(k), C.c_uint32(group_size), r0, r1, _p(o32), _p(o16))
    return o16 if f16_out else o32


def qkv_int8(x, w, scale, m, n, k, col_scale=None, rows=None):
    """One W8A16 projection -- kaio-ops/tests/qkv_project_int8_e2e.rs:48-72."""
    x = np.ascontiguousarray(x, dtype=np.float16)
    w = np.ascontiguousarray(w, dtype=np.int8)
    cs = None if col_scale is None else np.ascontiguousarray(col_scale, dtype=np.float32)
    out = np.zeros((m, n), dtype=np.float16)
    r0, r1 = _rows(m, rows)
    lib().kaio_oracle_qkv_int8(_p(x), _p(w), C.c_float(scale), _p(cs), C.c_uint32(m),
                               C.c_uint32(n), C.c_uint32(k), r0, r1, _p(out))
    return out


def qkv_w8a8(x, w, col_scale, m, n, k, rows=None, want_acc=False):
    """One W8A8 projection (extended; no reference counterpart): per-row symmetric quantisation of
    ``x`` (examples/int8_matmul/src/main.rs:41-61), exact s32 accumulation
    (kaio-ops/tests/matmul_int8_e2e.rs:20-34), ``f16(((acc as f32) * s_x[i]) * col_scale[j])``.
    With ``want_acc`` also returns the s32 accumulators, the quantised rows and their scales."""
    x = np.ascontiguousarray(x, dtype=np.float16)
    w = np.ascontiguousarray(w, dtype=np.int8)
    cs = np.ascontiguousarray(col_scale, dtype=np.float32)
    out = np.zeros((m, n), dtype=np.float16)
    acc = np.zeros((m, n), dtype=np.int32) if want_acc else None
    xq = np.zeros((m, k), dtype=np.int8) if want_acc else None
    sx = np.zeros(m, dtype=np.float32) if want_acc else None
    r0, r1 = _rows(m, rows)
    lib().kaio_oracle_qkv_w8a8(_p(x), _p(w), _p(cs), C.c_uint32(m), C.c_uint32(n), C.c_uint32(k), r0, r1,
                               _p(out), _p(acc), _p(xq), _p(sx))
    return (out, acc, xq, sx) if want_acc else out


def qkv_int4(x, packed, scales, m, n, k, group_size=128, rows=None):
    """One W4A16 projection -- kaio-ops/tests/qkv_project_int4_e2e.rs:70-100."""
    return matmul_int4(x, packed, scales, m, n, k, group_size, rows=rows, f16_out=True)


def attention(q, k, v, seq_q, seq_k, d_k, d_v, causal=False, strides=None, rows=None,
              f16_out=False, out=None):
    """kaio-ops/tests/common/mod.rs:163-235.

    ``strides`` = (q, k, v, out) row strides in elements (default: dense), so a
    head of a ``[rows, H*D]`` buffer can be addressed in place by passing array
    views that start at the head's first element.
    """
    qs, ks, vs, os_ = strides if strides is not None else (d_k, d_k, d_v, d_v)
    if out is None:
        out = np.zeros((seq_q, d_v), dtype=np.float16 if f16_out else np.float32)
    r0, r1 = _rows(seq_q, rows)
    o32 = None if f16_out else out
    o16 = out if f16_out else None
    C_u = C.c_uint32
    lib().kaio_oracle_attention(
        C.c_void_p(q.ctypes.data), C.c_void_p(k.ctypes.data), C.c_void_p(v.ctypes.data),
        C_u(seq_q), C_u(seq_k), C_u(d_k), C_u(d_v), C_u(qs), C_u(ks), C_u(vs), C_u(os_),
        C.c_int(1 if causal else 0), r0, r1,
        None if o32 is None else C.c_void_p(o32.ctypes.data),
        None if o16 is None else C.c_void_p(o16.ctypes.data))
    return out


def silu_gate_f32(x, gate):
    """``cpu_reference`` of examples/fused_silu_gate/src/main.rs:23-33 (f64 arithmetic, f32 result)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    gate = np.ascontiguousarray(gate, dtype=np.float32)
    out = np.zeros(x.size, dtype=np.float32)
    lib().kaio_oracle_silu_gate_f32(_p(x), _p(gate), _p(out), C.c_size_t(x.size))
    return out


def silu_gate_f16(x, gate, rows, cols, x_ld=None, gate_ld=None):
    """The f16 matrix form: the f32 result above rounded once to f16.  ``x`` and ``gate`` are flat
    f16 arrays holding [rows, cols] with row strides ``x_ld`` / ``gate_ld``; the result is
    contiguous [rows, cols]."""
    x = np.ascontiguousarray(x, dtype=np.float16)
    gate = np.ascontiguousarray(gate, dtype=np.float16)
    out = np.zeros((rows, cols), dtype=np.float16)
    lib().kaio_oracle_silu_gate_f16(_p(x), _p(gate), _p(out), C.c_uint32(rows), C.c_uint32(cols),
                                    C.c_uint32(x_ld or cols), C.c_uint32(gate_ld or cols), C.c_uint32(cols))
    return out


def quantize_rows_int8(x, m, k):
    """Per-row ``derive_scale`` + ``quantize`` -- examples/int8_matmul/src/main.rs:41-61."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    q = np.zeros((m, k), dtype=np.int8)
    scale = np.zeros(m, dtype=np.float32)
    lib().kaio_oracle_quantize_rows_int8(_p(x), C.c_uint32(m), C.c_uint32(k), _p(q), _p(scale))
    return q, scale


def quantize_gptq_lite(w, k, n, group_size=128):
    """``quantize_gptq_lite`` -- examples/int4_matmul/src/main.rs:48-85.  Returns (q [K,N], scales)."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    q = np.zeros((k, n), dtype=np.int8)
    scales = np.zeros((k // group_size) * n, dtype=np.float16)
    lib().kaio_oracle_quantize_gptq_lite(_p(w), C.c_uint32(k), C.c_uint32(n), C.c_uint32(group_size),
                                         _p(q), _p(scales))
    return q, scales


# ---------------------------------------------------------------------------
# Deterministic generators of the reference tests (64-bit LCG).  Pure numpy,
# vectorised by jumping the LCG, bit-identical to the scalar Rust closures.
# ---------------------------------------------------------------------------

_LCG_A = 6364136223846793005
_LCG_C = 1442695040888963407
_MASK = (1 << 64) - 1


def lcg_states(seed: int, count: int) -> np.ndarray:
    """States s_1..s_count of ``s = s*A + C (mod 2^64)`` starting from ``seed``."""
    out = np.empty(count, dtype=np.uint64)
    s = seed & _MASK
    # scalar loop in chunks with numpy jump-ahead: s_{i+B} = s_i*A^B + C*(A^B-1)/(A-1)
    block = 4096
    first = min(block, count)
    for i in range(first):
        s = (s * _LCG_A + _LCG_C) & _MASK
        out[i] = s
    if count > block:
        ab, cb = 1, 0
        for _ in range(block):  # compose the affine map `block` times
            cb = (cb * _LCG_A + _LCG_C) & _MASK
            ab = (ab * _LCG_A) & _MASK
        ab64, cb64 = np.uint64(ab), np.uint64(cb)
        pos = block
        with np.errstate(over="ignore"):
            while pos < count:
                take = min(block, count - pos)
                out[pos:pos + take] = out[pos - block:pos - block + take] * ab64 + cb64
                pos += take
    return out


def lcg_i8(seed: int, count: int) -> np.ndarray:
    """``(state >> 56) as i8`` -- kaio-ops/tests/matmul_int8_e2e.rs:50-56."""
    return (lcg_states(seed, count) >> np.uint64(56)).astype(np.uint8).view(np.int8)


def lcg_i8_div4(seed: int, count: int) -> np.ndarray:
    """``((state >> 56) as i8) / 4`` (truncating) -- qkv_project_int8_e2e.rs:162-172."""
    v = lcg_i8(seed, count).astype(np.int32)
    return (np.sign(v) * (np.abs(v) // 4)).astype(np.int8)


def lcg_s4(seed: int, count: int) -> np.ndarray:
    """``((state >> 60) as i8 - 8).clamp(-8,7)`` -- matmul_int4_e2e.rs:180-190."""
    v = (lcg_states(seed, count) >> np.uint64(60)).astype(np.int32) - 8
    return np.clip(v, -8, 7).astype(np.int8)


def _lcg_unit(seed: int, count: int) -> np.ndarray:
    top = (lcg_states(seed, count) >> np.uint64(32)).astype(np.uint32)
    return top.astype(np.float32) / np.float32(4294967295.0)


def lcg_f16_pm1(seed: int, count: int) -> np.ndarray:
    """f16 in [-1,1): ``top/u32::MAX*2-1`` -- matmul_int4_e2e.rs:166-178."""
    return (_lcg_unit(seed, count) * np.float32(2.0) - np.float32(1.0)).astype(np.float16)


def lcg_f16_pm_half(seed: int, count: int) -> np.ndarray:
    """f16 in [-0.5,0.5): ``top/u32::MAX-0.5`` -- qkv_project_int8_e2e.rs:146-160."""
    return (_lcg_unit(seed, count) - np.float32(0.5)).astype(np.float16)


def lcg_small_scales(seed: int, count: int) -> np.ndarray:
    """f16 in [0.0625,0.125) -- qkv_project_int4_e2e.rs:225-238."""
    return (_lcg_unit(seed, count) * np.float32(0.0625) + np.float32(0.0625)).astype(np.float16)


def patterned_f16(count: int) -> np.ndarray:
    """``(i % 17)/17 - 0.5`` -- kaio-ops/tests/common/mod.rs:27-35."""
    i = np.arange(count, dtype=np.int64) % 17
    return (i.astype(np.float32) / np.float32(17.0) - np.float32(0.5)).astype(np.float16)
