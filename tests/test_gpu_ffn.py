"""SiLU-gate kernels and the W4A16 feed-forward chain on the GPU against the CPU oracle
(examples/fused_silu_gate/src/main.rs:23-33 for the activation; kaio-ops/tests/matmul_int4_e2e.rs
for the GEMMs)."""
import numpy as np
import pytest
import torch

from kaio_b200 import InvalidConfig, ffn, ops
from helpers import dev, device, host, max_rel
from test_ffn_cpu import ffn_oracle, make_ffn_case

pytestmark = pytest.mark.gpu

F16_ULP = 2.0 ** -10  # one unit in the last place of an f16 significand, relative


def test_silu_gate_f32_example_data(oracle):
    """The example's own inputs and its own bar: max abs error < 1e-5 against the f64 reference
    (examples/fused_silu_gate/src/main.rs:45-51,66-72)."""
    n = 1 << 20
    i = np.arange(n)
    x = ((i % 97).astype(np.float32) / np.float32(97.0)) - np.float32(0.5)
    g = ((i % 113).astype(np.float32) / np.float32(113.0)) - np.float32(0.5)
    out = torch.zeros(n, device="cuda")
    ops.silu_gate_f32(device(), dev(x), dev(g), out, n)
    assert ops.last_variant() == "silu_gate_f32"
    assert np.max(np.abs(host(out) - oracle.silu_gate_f32(x, g))) < 1e-5


@pytest.mark.parametrize("n,offset", [(1, 0), (3, 0), (4, 0), (1027, 0), (4096, 1), (1 << 22, 0), ((1 << 22) + 5, 3)])
def test_silu_gate_f32_sizes_and_alignment(oracle, n, offset):
    """Ragged sizes (scalar tail) and buffers that do not start on a 16-byte boundary."""
    rng = np.random.default_rng(n)
    x = (rng.standard_normal(n) * 4).astype(np.float32)
    g = (rng.standard_normal(n) * 2).astype(np.float32)
    pad = np.zeros(offset, dtype=np.float32)
    xd, gd = dev(np.concatenate([pad, x]))[offset:], dev(np.concatenate([pad, g]))[offset:]
    out = torch.full((offset + n + 8,), 7.0, device="cuda")
    ops.silu_gate_f32(device(), xd, gd, out[offset:], n)
    got = host(out)
    want = oracle.silu_gate_f32(x, g)
    err = np.abs(got[offset:offset + n] - want) / np.maximum(np.abs(want), 1.0)
    assert err.max() < 1e-6
    assert np.all(got[:offset] == 7.0) and np.all(got[offset + n:] == 7.0)  # nothing outside [0, n)


@pytest.mark.parametrize("rows,cols,strided", [(1, 8, False), (16, 3584, True), (40, 1000, True), (7, 13, False),
                                               (300, 4096, True), (5, 21, True)])
def test_silu_gate_f16(oracle, rows, cols, strided):
    """f16 matrices, contiguous or as the two halves of one [rows, 2*cols] buffer; odd widths take
    the scalar kernel.  The kernel computes in f32 and rounds once; the oracle narrows an f64
    result: at most one f16 unit in the last place apart, equal nearly everywhere."""
    rng = np.random.default_rng(rows * cols)
    both = (rng.standard_normal((rows, 2 * cols)) * 3).astype(np.float16)
    out = torch.zeros(rows * cols, device="cuda", dtype=torch.float16)
    if strided:
        buf = dev(both)
        ops.silu_gate_f16(device(), buf, buf[cols:], out, rows, cols, x_ld=2 * cols, gate_ld=2 * cols)
        want = oracle.silu_gate_f16(both.reshape(-1), both.reshape(-1)[cols:], rows, cols, 2 * cols, 2 * cols)
    else:
        xs, gs = np.ascontiguousarray(both[:, :cols]), np.ascontiguousarray(both[:, cols:])
        ops.silu_gate_f16(device(), dev(xs), dev(gs), out, rows, cols)
        want = oracle.silu_gate_f16(xs.reshape(-1), gs.reshape(-1), rows, cols)
    assert ops.last_variant() == "silu_gate_f16"
    got = host(out, (rows, cols)).astype(np.float64)
    want = want.astype(np.float64)
    assert np.all(np.abs(got - want) <= F16_ULP * np.maximum(np.abs(want), 2.0 ** -14))
    assert np.mean(got != want) < 0.01


def test_silu_gate_argument_errors():
    d = device()
    x = torch.zeros(64, device="cuda")
    with pytest.raises(InvalidConfig, match="dimensions must be non-zero"):
        ops.silu_gate_f32(d, x, x, x.clone(), 0)
    with pytest.raises(InvalidConfig, match="gate buffer too small"):
        ops.silu_gate_f32(d, x, x[:32], x.clone(), 64)
    h = torch.zeros(64, device="cuda", dtype=torch.float16)
    with pytest.raises(InvalidConfig, match="row strides must be at least cols"):
        ops.silu_gate_f16(d, h, h, h.clone(), 4, 16, x_ld=8)
    with pytest.raises(InvalidConfig, match="out buffer too small"):
        ops.silu_gate_f16(d, h, h, h.clone()[:60], 4, 16)


@pytest.mark.parametrize("hidden,inter,m", [(256, 384, 1), (256, 512, 16), (512, 1024, 40), (1024, 2048, 300)])
def test_ffn_chain_stagewise_and_end_to_end(oracle, hidden, inter, m):
    """Every stage against the oracle fed with the GPU's own input to that stage (the bars of the
    single ops), then the whole chain against the oracle's chain."""
    case = make_ffn_case(oracle, hidden, inter, m, seed=hidden + m)
    weights = [case[n] for n in ("w_gate", "s_gate", "w_up", "s_up", "w_down", "s_down")]
    chain = ffn.FfnInt4(ops, device(), hidden, inter, *weights, max_m=max(m, 16))
    got = host(chain.run(case["x"].cuda(), m)).copy()
    u32 = lambda t: t.numpy().view(np.uint32)

    # stage 1: the concatenated gate|up projection
    gu = host(chain.gu)[: m * 2 * inter].reshape(m, 2 * inter)
    g_want = oracle.matmul_int4(case["x"].numpy(), u32(case["w_gate"]), case["s_gate"].numpy(), m, inter, hidden, f16_out=True)
    u_want = oracle.matmul_int4(case["x"].numpy(), u32(case["w_up"]), case["s_up"].numpy(), m, inter, hidden, f16_out=True)
    assert max_rel(gu[:, :inter], np.asarray(g_want).reshape(m, inter)) < 2e-3
    assert max_rel(gu[:, inter:], np.asarray(u_want).reshape(m, inter)) < 2e-3
    # stage 2: the activation of the GPU's own projections
    act = host(chain.act)[: m * inter].reshape(m, inter)
    act_want = oracle.silu_gate_f16(gu.reshape(-1), gu.reshape(-1)[inter:], m, inter, 2 * inter, 2 * inter)
    a64, w64 = act.astype(np.float64), act_want.astype(np.float64)
    assert np.all(np.abs(a64 - w64) <= F16_ULP * np.maximum(np.abs(w64), 2.0 ** -14))
    # stage 3: the down projection of the GPU's own activation
    d_want = oracle.matmul_int4(act.reshape(-1), u32(case["w_down"]), case["s_down"].numpy(), m, hidden, inter, f16_out=False)
    assert max_rel(got, np.asarray(d_want).reshape(m, hidden)) < 1e-3
    # the whole chain: f16 roundings of the intermediates may fall differently on the two sides
    assert max_rel(got, ffn_oracle(oracle, case, hidden, inter, m)) < 1e-2


def test_ffn_chain_partial_sums_add_up(oracle):
    """Two ranks' shards run one after the other on one GPU: their partial outputs sum to the
    unsharded chain's output (what the all-reduce does across GPUs)."""
    hidden, inter, m = 512, 1024, 24
    case = make_ffn_case(oracle, hidden, inter, m, seed=5)
    weights = [case[n] for n in ("w_gate", "s_gate", "w_up", "s_up", "w_down", "s_down")]
    x = case["x"].cuda()
    full = host(ffn.FfnInt4(ops, device(), hidden, inter, *weights, max_m=m).run(x, m)).copy()
    parts = [host(ffn.FfnInt4(ops, device(), hidden, inter, *weights, world=2, rank=r, max_m=m,
                              reduce="none").run(x, m)).copy() for r in range(2)]
    assert max_rel(parts[0] + parts[1], full) < 1e-4


@pytest.mark.parametrize("m", [8, 64, 600])
@pytest.mark.parametrize("scatter", [False, True])
@pytest.mark.parametrize("world", [2, 8])
def test_peer_partials_ranks_emulated_on_one_gpu(oracle, m, scatter, world):
    """The row-parallel GEMM with its reduction in the epilogue, all ranks run one after the other
    on one GPU (nothing waits on anything): each "rank" stores its f32 partial into slot `rank` of
    all staging buffers (whole, or its column blocks scattered to their owners); the slot sum then
    gives the full-K product.  m = 8 / 64 / 600 go through the decode, fused-dequant and
    tensor-map-store kernels."""
    n, k = 512, 1024
    kl, blk = k // world, n // world
    rng = np.random.default_rng(m + scatter)
    w = rng.integers(-8, 8, (k, n), dtype=np.int8)
    a = rng.standard_normal((m, k)).astype(np.float16)
    sc = rng.uniform(0.005, 0.02, (k // 128, n)).astype(np.float16)
    want = np.asarray(oracle.matmul_int4(a.reshape(-1), oracle.pack_s4(w, k, n), sc.reshape(-1), m, n, k,
                                         f16_out=False)).reshape(m, n)
    d = device()
    cols = blk if scatter else n
    stages = [torch.full((world * m * cols,), float("nan"), device="cuda") for _ in range(world)]
    ptrs = [s.data_ptr() for s in stages]
    for rank in range(world):
        a_loc = dev(np.ascontiguousarray(a[:, rank * kl:(rank + 1) * kl]))
        w_loc = dev(oracle.pack_s4(np.ascontiguousarray(w[rank * kl:(rank + 1) * kl]), kl, n))
        s_loc = dev(np.ascontiguousarray(sc[rank * kl // 128:(rank + 1) * kl // 128]))
        ops.matmul_int4_peer_partials(d, a_loc, w_loc, s_loc, ptrs, world * m * cols, world, rank, scatter, m, n, kl)
        assert ops.last_variant().endswith("_peer_partials")
    outs = [torch.full((m * n,), float("nan"), device="cuda") for _ in range(world)]
    optrs = [o.data_ptr() for o in outs]
    for rank in range(world):
        if scatter:  # the owner sums its column block and stores it to every output
            ops.sum_partials_f32(d, stages[rank], world, m, blk, optrs, m * n, n, rank * blk)
        else:
            ops.sum_partials_f32(d, stages[rank], world, m, n, [optrs[rank]], m * n, n, 0)
    assert ops.device_status(d)[0] == 0
    got = [host(o, (m, n)) for o in outs]
    assert all(np.array_equal(got[0], g) for g in got[1:])
    assert max_rel(got[0], want) < 1e-3


def test_sum_partials_argument_errors():
    d = device()
    s = torch.zeros(2 * 4 * 16, device="cuda")
    o = torch.zeros(4 * 16, device="cuda")
    with pytest.raises(InvalidConfig, match="multiples of 4"):
        ops.sum_partials_f32(d, s, 2, 4, 14, [o.data_ptr()], o.numel(), 16, 0)
    with pytest.raises(InvalidConfig, match="staging buffer too small"):
        ops.sum_partials_f32(d, s[:100], 2, 4, 16, [o.data_ptr()], o.numel(), 16, 0)
    with pytest.raises(InvalidConfig, match="out buffers too small"):
        ops.sum_partials_f32(d, s, 2, 4, 16, [o.data_ptr()], 60, 16, 0)


def test_dequantize_then_f16_gemm_equals_matmul_int4(oracle):
    """kaio_b200_dequantize_int4 writes exactly f16(q) * f16(scale) (checked against numpy), and
    the f16 GEMM on those weights returns the bits matmul_int4 returns for m > 512 (it runs the
    same two steps internally)."""
    m, k, n = 768, 512, 640
    rng = np.random.default_rng(3)
    q = rng.integers(-8, 8, (k, n), dtype=np.int8)
    s = rng.uniform(0.005, 0.02, (k // 128, n)).astype(np.float16)
    a = rng.standard_normal(m * k).astype(np.float16)
    packed = oracle.pack_s4(q, k, n)
    d = device()
    w16 = torch.full((k * n,), float("nan"), device="cuda", dtype=torch.float16)
    ops.dequantize_int4(d, dev(packed), dev(s), w16, k, n)
    want_w = (q.astype(np.float16) * np.repeat(s, 128, axis=0)).astype(np.float16)  # one f16 rounding
    assert np.array_equal(host(w16, (k, n)).view(np.uint16), want_w.view(np.uint16))
    for f16_out in (False, True):
        dt = torch.float16 if f16_out else torch.float32
        ref = torch.zeros(m * n, device="cuda", dtype=dt)
        ops.matmul_int4(d, dev(a), dev(packed), dev(s), ref, m, n, k, 128)
        assert ops.last_variant() == "w4a16_tcgen05"
        got = torch.zeros(m * n, device="cuda", dtype=dt)
        (ops.matmul_tc_f16out if f16_out else ops.matmul_tc)(d, dev(a), w16, got, m, n, k)
        assert ops.device_status(d)[0] == 0
        assert torch.equal(got.view(torch.int16 if f16_out else torch.int32),
                           ref.view(torch.int16 if f16_out else torch.int32))
        want = oracle.matmul_int4(a, packed, s.reshape(-1), m, n, k, f16_out=f16_out)
        assert max_rel(host(got, (m, n)), want) < (2e-2 if f16_out else 1e-3)


def test_chunked_chain_equals_the_whole_chain(oracle):
    """FfnInt4.run_overlapped on one rank (weights dequantised once, rows in chunks): the same
    bits as the three whole launches, and the oracle's chain within the GEMMs' bar."""
    hidden, inter, m = 512, 1024, 1024
    case = make_ffn_case(oracle, hidden, inter, m, seed=9)
    weights = [case[n] for n in ("w_gate", "s_gate", "w_up", "s_up", "w_down", "s_down")]
    chain = ffn.FfnInt4(ops, device(), hidden, inter, *weights, world=1, rank=0, max_m=m, reduce="none")
    x = case["x"].cuda()
    whole = chain.local(x, m).clone()
    parts = chain.run_overlapped(x, m, chunks=[512, 256, 256]).clone()
    torch.cuda.synchronize()
    assert ops.device_status(device())[0] == 0
    assert torch.equal(whole.view(torch.int32), parts.view(torch.int32))
    want = ffn_oracle(oracle, case, hidden, inter, m)
    assert max_rel(parts.cpu().numpy(), want) < 1e-2
    assert ffn.FfnInt4.default_chunks(4096) == [2048, 1280, 768] and ffn.FfnInt4.default_chunks(512) == [512]


@pytest.mark.parametrize("hidden,inter,m", [(256, 512, 16), (512, 1024, 300), (512, 1024, 640), (1024, 2048, 1500)])
def test_silu_gate_in_the_gemm_epilogue_gives_the_same_bits(oracle, hidden, inter, m):
    """``matmul_int4_silu_gate`` (activation in the GEMM epilogue above m = 512, two launches through
    the caller's scratch below) against the two separate ops it replaces: the same bits in the
    activation and at the end of the chain; the chain stays within the oracle's bar."""
    case = make_ffn_case(oracle, hidden, inter, m, seed=7 * hidden + m)
    weights = [case[n] for n in ("w_gate", "s_gate", "w_up", "s_up", "w_down", "s_down")]
    chain = ffn.FfnInt4(ops, device(), hidden, inter, *weights, max_m=max(m, 16))
    x = case["x"].cuda()
    plain = chain.run(x, m).clone()
    act_plain = chain.act[: m * inter].clone()
    chain.enable_fused_silu()
    chain.act.zero_()
    fused = chain.run(x, m).clone()
    torch.cuda.synchronize()
    assert ops.device_status(device())[0] == 0
    assert torch.equal(chain.act[: m * inter].view(torch.int16), act_plain.view(torch.int16))
    assert torch.equal(fused.view(torch.int32), plain.view(torch.int32))
    assert max_rel(host(fused), ffn_oracle(oracle, case, hidden, inter, m)) < 1e-2
    # the entry point itself: above 512 rows one launch and no scratch
    act = torch.zeros(m * inter, device="cuda", dtype=torch.float16)
    ops.matmul_int4_silu_gate(device(), x, chain.w_gu_il, chain.s_gu_il, act, None if m > 512 else chain.gu,
                              m, inter, hidden)
    assert ops.last_variant() == ("w4a16_tcgen05_silu_gate" if m > 512 else "w4a16_then_silu_gate")
    assert torch.equal(act.view(torch.int16), act_plain.view(torch.int16))


def test_silu_gate_gemm_argument_errors():
    d = device()
    k, cols, m = 128, 64, 4
    x = torch.zeros(m * k, device="cuda", dtype=torch.float16)
    w = torch.zeros((k // 8) * 2 * cols, device="cuda", dtype=torch.int32)
    s = torch.zeros(2 * cols, device="cuda", dtype=torch.float16)
    act = torch.zeros(m * cols, device="cuda", dtype=torch.float16)
    with pytest.raises(InvalidConfig, match="multiple of 64"):
        ops.matmul_int4_silu_gate(d, x, w, s, act, None, m, 32, k)
    with pytest.raises(InvalidConfig, match="act buffer too small"):
        ops.matmul_int4_silu_gate(d, x, w, s, act[:8], None, m, cols, k)
    with pytest.raises(InvalidConfig, match="needs a 16-byte aligned scratch"):
        ops.matmul_int4_silu_gate(d, x, w, s, act, None, m, cols, k)
