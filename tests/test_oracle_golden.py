"""Pins the CPU oracle against the known-answer vectors of the KAIO test suite.

Each case cites the reference test it restates (paths relative to the KAIO tree).
No GPU needed.
"""
import numpy as np
import pytest

GROUP = 128


def f16(x):
    return np.float16(x)


# ---------------------------------------------------------------- f16 conversions

def test_f16_roundtrip_all_bit_patterns(oracle):
    bits = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    as_np = bits.view(np.float16).astype(np.float32)
    for b in range(0, 65536, 7):  # stride keeps the ctypes loop short; full sweep below for f32->f16
        got = oracle.f16_to_f32(int(bits[b]))
        want = float(as_np[b])
        assert (np.isnan(got) and np.isnan(want)) or got == want
    finite = bits[np.isfinite(as_np)]
    for b in finite[::5]:
        assert oracle.f32_to_f16(float(np.array([b], np.uint16).view(np.float16)[0])) == int(b)


def test_f32_to_f16_matches_numpy_rne(oracle):
    rng = np.random.default_rng(7)
    xs = np.concatenate([
        rng.standard_normal(4000).astype(np.float32) * np.float32(100.0),
        rng.standard_normal(2000).astype(np.float32) * np.float32(1e-5),
        np.array([65504.0, 65519.9, 65520.0, 1e6, 2.0 ** -24, 2.0 ** -25, 2.0 ** -25 * 1.0001,
                  2.0 ** -14, 2.0 ** -14 - 2.0 ** -25, 0.0, -0.0, 1.00048828125, 1.0009765625 * 1.5],
                 dtype=np.float32),
    ])
    with np.errstate(over="ignore"):
        want = xs.astype(np.float16).view(np.uint16)
    for x, w in zip(xs, want):
        assert oracle.f32_to_f16(float(x)) == int(w), float(x)


# ---------------------------------------------------------------- generators

def test_lcg_matches_scalar_definition(oracle):
    seed = 0xA5A55A5AD00DFEED
    n = 10000
    s = seed
    want = []
    for _ in range(n):
        s = (s * 6364136223846793005 + 1442695040888963407) & ((1 << 64) - 1)
        want.append(s)
    got = oracle.lcg_states(seed, n)
    assert got.tolist() == want


# ---------------------------------------------------------------- W4A16

def test_pack_and_reference_smoke(oracle):
    """kaio-ops/tests/matmul_int4_e2e.rs:463-490 (host-runnable golden vector)."""
    m, n, k = 2, 2, 8
    w = np.array([1 if i % 2 == 0 else -1 for i in range(k * n)], dtype=np.int8)
    packed = oracle.pack_s4(w, k, n)
    assert packed[0] == 0x11111111
    assert packed[1] == 0xFFFFFFFF
    a = np.array([1.0 if i < k else 0.0 for i in range(m * k)], dtype=np.float16)
    scales = np.ones(n, dtype=np.float16)
    out = oracle.matmul_int4(a, packed, scales, m, n, k, group_size=k)
    assert out.reshape(-1).tolist() == [8.0, -8.0, 0.0, 0.0]


def test_int4_all_ones_is_128(oracle):
    """matmul_int4_e2e.rs:203-218."""
    m, n, k = 16, 8, 128
    out = oracle.matmul_int4(np.ones(m * k, np.float16), oracle.pack_s4(np.ones(k * n, np.int8), k, n),
                             np.ones(n, np.float16), m, n, k)
    assert np.all(out == 128.0)


def test_int4_sign_extend_negative_eights(oracle):
    """matmul_int4_e2e.rs:230-246: packed 0x88888888 -> -1024 everywhere."""
    m, n, k = 16, 8, 128
    packed = oracle.pack_s4(np.full(k * n, -8, np.int8), k, n)
    assert np.all(packed == 0x88888888)
    out = oracle.matmul_int4(np.ones(m * k, np.float16), packed, np.ones(n, np.float16), m, n, k)
    assert np.all(out == -1024.0)


def test_int4_mixed_positions(oracle):
    """matmul_int4_e2e.rs:253-278: column 0 alternates +7/-8 -> -64, others 0."""
    m, n, k = 16, 8, 128
    w = np.zeros((k, n), np.int8)
    w[0::2, 0] = 7
    w[1::2, 0] = -8
    out = oracle.matmul_int4(np.ones(m * k, np.float16), oracle.pack_s4(w, k, n),
                             np.ones(n, np.float16), m, n, k)
    assert np.all(out[:, 0] == -64.0) and np.all(out[:, 1:] == 0.0)


def test_int4_two_groups_is_384(oracle):
    """matmul_int4_e2e.rs:289-308: group scales 1.0 / 2.0 -> 128 + 256."""
    m, n, k = 32, 32, 256
    scales = np.concatenate([np.full(n, 1.0), np.full(n, 2.0)]).astype(np.float16)
    out = oracle.matmul_int4(np.ones(m * k, np.float16), oracle.pack_s4(np.ones(k * n, np.int8), k, n),
                             scales, m, n, k)
    assert np.all(out == 384.0)


def test_int4_matches_pure_python_restatement(oracle):
    """Element-by-element restatement of matmul_int4_e2e.rs:60-95 in numpy scalars."""
    m, n, k = 3, 5, 256
    w = oracle.lcg_s4(0xCAFEBABEDEADBEEF, k * n)
    a = oracle.lcg_f16_pm1(0x123456789ABCDEF0, m * k)
    scales = oracle.lcg_small_scales(99, (k // GROUP) * n)
    packed = oracle.pack_s4(w, k, n)
    got = oracle.matmul_int4(a, packed, scales, m, n, k)
    kw = k // 8
    for i in range(m):
        for j in range(n):
            acc = np.float32(0.0)
            for kk in range(k):
                nib = (int(packed[kk // 8 + j * kw]) >> (4 * (kk % 8))) & 0xF
                s = nib - 16 if nib >= 8 else nib
                raw = np.float16(np.float32(s))
                sc = scales[(kk // GROUP) * n + j]
                scaled = np.float16(np.float32(raw) * np.float32(sc))
                acc = np.float32(acc + np.float32(a[i * k + kk]) * np.float32(scaled))
            assert got[i, j] == acc


# ---------------------------------------------------------------- W8A8

def test_int8_boundary_values(oracle):
    """matmul_int8_e2e.rs:169-202 (i8::MIN / MAX / -1 / 0 / 1 at known positions)."""
    m, n, k = 16, 8, 32
    a = np.zeros((m, k), np.int8)
    a[0, :5] = [-128, 127, -1, 0, 1]
    a[0, 5:] = np.arange(k - 5)
    b = np.zeros((k, n), np.int8)
    b[:, 0] = 1
    b[:, 1] = np.where(np.arange(k) % 2 == 0, 1, -1)
    out, acc = oracle.matmul_int8(a, b, 1.0, m, n, k, want_acc=True)
    want = a.astype(np.int64) @ b.astype(np.int64)
    assert np.array_equal(acc, want.astype(np.int32))
    assert np.array_equal(out, want.astype(np.float32))
    assert acc[0, 0] == -128 + 127 - 1 + 0 + 1 + sum(range(27))


@pytest.mark.parametrize("m,n,k,scale,seed", [
    (16, 8, 32, 1.0, 0xA5A55A5AD00DFEED), (64, 64, 32, 0.5, 0x123456789ABCDEF0),
    (64, 64, 128, 0.125, 0xCAFEBABEDEADBEEF), (128, 128, 128, 0.01, 0x0123456789ABCDEF),
    (17, 8, 32, 1.0, 0xDEAD0001BEEF0002), (16, 13, 32, 1.0, 0xFACE0003BEEF0004),
])
def test_int8_round_trip_shapes_vs_int64(oracle, m, n, k, scale, seed):
    """The seeded shapes of matmul_int8_e2e.rs:72-146 against an exact int64 matmul."""
    data = oracle.lcg_i8(seed, m * k + k * n)
    a, b = data[:m * k].reshape(m, k), data[m * k:].reshape(k, n)
    out, acc = oracle.matmul_int8(a, b, scale, m, n, k, want_acc=True)
    want = a.astype(np.int64) @ b.astype(np.int64)
    assert np.array_equal(acc.astype(np.int64), want)
    assert np.array_equal(out, want.astype(np.float32) * np.float32(scale))


def test_int8_scaled_extension(oracle):
    m, n, k = 9, 20, 64
    rng = np.random.default_rng(3)
    a = rng.integers(-127, 128, (m, k), dtype=np.int8)
    b = rng.integers(-127, 128, (k, n), dtype=np.int8)
    sa = rng.uniform(0.001, 0.01, m).astype(np.float32)
    sw = rng.uniform(0.001, 0.01, n).astype(np.float32)
    out = oracle.matmul_int8_scaled(a, b, sa, sw, m, n, k)
    acc = (a.astype(np.int64) @ b.astype(np.int64)).astype(np.float32)
    assert np.array_equal(out, (acc * sa[:, None]) * sw[None, :])


# ---------------------------------------------------------------- fused QKV

@pytest.mark.parametrize("k", [32, 48])
def test_qkv_int8_slot_canary_exact(oracle, k):
    """qkv_project_int8_e2e.rs:308-372: W=1/2/3, X=1, scale 1 -> exactly K, 2K, 3K."""
    m, n = 64, 16
    x = np.ones(m * k, np.float16)
    for val in (1, 2, 3):
        out = oracle.qkv_int8(x, np.full(k * n, val, np.int8), 1.0, m, n, k)
        assert np.all(out.astype(np.float32) == float(val * k))


def test_qkv_int8_differentiation(oracle):
    """qkv_project_int8_e2e.rs:244-281: scales 1/K -> 1, 2, 3."""
    m, n, k = 64, 32, 128
    x = np.ones(m * k, np.float16)
    for val in (1, 2, 3):
        out = oracle.qkv_int8(x, np.full(k * n, val, np.int8), 1.0 / k, m, n, k)
        assert np.all(np.abs(out.astype(np.float32) - val) < 1e-2)


def test_qkv_int8_col_scale_extension(oracle):
    m, n, k = 8, 12, 64
    rng = np.random.default_rng(5)
    x = rng.standard_normal(m * k).astype(np.float16)
    w = rng.integers(-127, 128, k * n, dtype=np.int8)
    cs = rng.uniform(0.001, 0.01, n).astype(np.float32)
    got = oracle.qkv_int8(x, w, 0.0, m, n, k, col_scale=cs)
    for j in range(n):
        col = oracle.qkv_int8(x, w, float(cs[j]), m, n, k)[:, j]
        assert np.array_equal(got[:, j], col)


def test_qkv_int4_canaries(oracle):
    """qkv_project_int4_e2e.rs:318-393: -8 -> -1024; W=1/2/3 with scale 1/K -> 1,2,3."""
    m, n, k = 64, 16, 128
    x = np.ones(m * k, np.float16)
    out = oracle.qkv_int4(x, oracle.pack_s4(np.full(k * n, -8, np.int8), k, n),
                          np.ones(n, np.float16), m, n, k)
    assert np.all(out.astype(np.float32) == -1024.0)
    inv_k = np.full(n, 1.0 / k, np.float16)
    for val in (1, 2, 3):
        out = oracle.qkv_int4(x, oracle.pack_s4(np.full(k * n, val, np.int8), k, n), inv_k, m, n, k)
        assert np.all(np.abs(out.astype(np.float32) - val) < 1e-2)


# ---------------------------------------------------------------- attention

def test_attention_causal_row0_is_v_row0(oracle):
    """kaio-ops/tests/attention_tc_api.rs:153-201."""
    sq = sk = 16
    dk, dv = 16, 8
    q = oracle.patterned_f16(sq * dk)
    k = oracle.patterned_f16(sk * dk)
    v = np.repeat(((np.arange(sk, dtype=np.float32) + 1.0) * np.float32(0.1))[:, None], dv, 1)
    v = v.astype(np.float16)
    out = oracle.attention(q, k, v.reshape(-1), sq, sk, dk, dv, causal=True)
    assert np.all(np.abs(out[0] - 0.1) < 5e-3)
    assert np.array_equal(out[0], v[0].astype(np.float32))


@pytest.mark.parametrize("causal", [False, True])
def test_attention_matches_numpy_f32(oracle, causal):
    sq, sk, dk, dv = 32, 48, 32, 16
    q = oracle.patterned_f16(sq * dk)
    k = oracle.patterned_f16(sk * dk)
    v = oracle.patterned_f16(sk * dv)
    got = oracle.attention(q, k, v, sq, sk, dk, dv, causal=causal)
    qf = q.astype(np.float64).reshape(sq, dk)
    kf = k.astype(np.float64).reshape(sk, dk)
    vf = v.astype(np.float64).reshape(sk, dv)
    s = qf @ kf.T / np.sqrt(dk)
    if causal:
        s = np.where(np.arange(sk)[None, :] > np.arange(sq)[:, None], -np.inf, s)
    p = np.exp(s - s.max(1, keepdims=True))
    p /= p.sum(1, keepdims=True)
    assert np.allclose(got, p @ vf, rtol=1e-5, atol=1e-6)


def test_attention_strided_head_view(oracle):
    """Strided addressing picks one head out of a [S, H*D] buffer (extension)."""
    s, h, d = 32, 3, 16
    rng = np.random.default_rng(11)
    qkv = [rng.standard_normal((s, h * d)).astype(np.float16) for _ in range(3)]
    out = np.zeros((s, h * d), np.float16)
    for hd in range(h):
        views = [t.reshape(-1)[hd * d:] for t in qkv]
        oracle.attention(*views, s, s, d, d, causal=True, strides=(h * d,) * 4, f16_out=True,
                         out=out.reshape(-1)[hd * d:])
        dense = oracle.attention(*[np.ascontiguousarray(t[:, hd * d:(hd + 1) * d]).reshape(-1) for t in qkv],
                                 s, s, d, d, causal=True)
        assert np.array_equal(out[:, hd * d:(hd + 1) * d], dense.astype(np.float16))


def test_row_range_leaves_other_rows_untouched(oracle):
    m, n, k = 8, 16, 32
    data = oracle.lcg_i8(1, m * k + k * n)
    a, b = data[:m * k], data[m * k:]
    full = oracle.matmul_int8(a, b, 0.5, m, n, k)
    part = oracle.matmul_int8(a, b, 0.5, m, n, k, rows=(2, 5))
    assert np.array_equal(part[2:5], full[2:5]) and np.all(part[:2] == 0) and np.all(part[5:] == 0)


# ---------------------------------------------------------------- quantisers

def test_quantizers_match_numpy_restatement(oracle):
    """examples/int8_matmul/src/main.rs:41-61 and examples/int4_matmul/src/main.rs:48-85 restated
    with numpy (round half away from zero = sign * floor(|v| + 0.5))."""
    rng = np.random.default_rng(1)
    m, k = 5, 64
    x = rng.standard_normal((m, k)).astype(np.float32)
    x[2] = 0
    q, s = oracle.quantize_rows_int8(x, m, k)
    for i in range(m):
        mx = np.abs(x[i]).max()
        sc = np.float32(1.0) if mx == 0 else np.float32(mx) / np.float32(127.0)
        v = (x[i] / sc).astype(np.float32)
        r = np.sign(v) * np.floor(np.abs(v) + np.float32(0.5))
        assert s[i] == sc and np.array_equal(q[i], np.clip(r, -127, 127).astype(np.int8))
    kk, n = 256, 6
    w = (rng.standard_normal((kk, n)) * 0.1).astype(np.float32)
    qw, sc = oracle.quantize_gptq_lite(w, kk, n)
    for col in range(n):
        for g in range(kk // 128):
            blk = w[g * 128:(g + 1) * 128, col]
            mx = np.abs(blk).max()
            s32 = np.float32(1.0) if mx == 0 else np.float32(mx) / np.float32(7.0)
            v = (blk / s32).astype(np.float32)
            r = np.clip(np.sign(v) * np.floor(np.abs(v) + np.float32(0.5)), -8, 7).astype(np.int8)
            assert sc[g * n + col] == np.float16(s32) and np.array_equal(qw[g * 128:(g + 1) * 128, col], r)
    assert qw.max() == 7 and qw.min() >= -8


# ---------------------------------------------------------------- f16 GEMM (matmul_tc)

def test_matmul_f16_matches_ordered_numpy(oracle):
    """cpu_matmul_f16xf16_f32 (kaio-ops/tests/common/mod.rs:37-54): f32 multiply, f32 add, k
    ascending -- restated here with one numpy multiply and one add per k."""
    m, n, k = 9, 11, 48
    a, b = oracle.patterned_f16(m * k), oracle.patterned_f16(k * n)
    want = np.zeros((m, n), np.float32)
    af, bf = a.reshape(m, k).astype(np.float32), b.reshape(k, n).astype(np.float32)
    for p in range(k):
        want = want + af[:, p:p + 1] * bf[p:p + 1, :]
    assert np.array_equal(oracle.matmul_f16(a, b, m, n, k), want)


def test_matmul_f16_quadrant_canary(oracle):
    """matmul_tc_api.rs:127-170: cell (i,j) = (i+1)(j+1) K * 1e-4 up to f16 input rounding."""
    m = n = k = 64
    a = np.repeat(((np.arange(m) + 1) * 0.01).astype(np.float16)[:, None], k, 1)
    b = np.repeat(((np.arange(n) + 1) * 0.01).astype(np.float16)[None, :], k, 0)
    got = oracle.matmul_f16(a.reshape(-1), b.reshape(-1), m, n, k)
    want = np.outer(np.arange(m) + 1, np.arange(n) + 1) * k * 1e-4
    assert np.allclose(got, want, rtol=3e-3)


def test_qkv_w8a8_is_the_quantiser_followed_by_the_int8_reference(oracle):
    """The W8A8 QKV oracle (no reference counterpart) composes two restated reference functions:
    its s32 accumulators must equal matmul_int8 on the rows quantise_rows_int8 produces, and its
    outputs the two f32 multiplies + one f16 rounding of those accumulators."""
    rng = np.random.default_rng(21)
    m, n, k = 9, 24, 96
    x = rng.standard_normal((m, k)).astype(np.float16)
    x[3] = 0
    w = rng.integers(-127, 128, (k, n), dtype=np.int8)
    cs = rng.uniform(0.001, 0.01, n).astype(np.float32)
    out, acc, xq, sx = oracle.qkv_w8a8(x, w, cs, m, n, k, want_acc=True)
    q_ref, s_ref = oracle.quantize_rows_int8(x.astype(np.float32), m, k)
    assert np.array_equal(xq, q_ref) and np.array_equal(sx, s_ref) and sx[3] == 1.0
    _, acc_ref = oracle.matmul_int8(q_ref, w, 1.0, m, n, k, want_acc=True)
    assert np.array_equal(acc, acc_ref)
    want = ((acc.astype(np.float32) * sx[:, None]).astype(np.float32) * cs[None, :]).astype(np.float32)
    assert np.array_equal(out, want.astype(np.float16))
