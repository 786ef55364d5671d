"""The committed golden fixtures (tests/golden/golden_cases.*).

CPU part: the oracle still reproduces every fixture bit for bit (a change in the oracle or in
the restated generators shows up here, not as a silent shift of what the GPU is compared to).
GPU part: the C-ABI entry points against the same arrays - bit-exact for INT8, the reference's
tolerances for the f16 paths.
"""
import importlib.util
import json
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = os.path.join(HERE, "golden")

_spec = importlib.util.spec_from_file_location("make_golden", os.path.join(GOLDEN, "make_golden.py"))
make_golden = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(make_golden)

with open(os.path.join(GOLDEN, "golden_cases.json")) as f:
    CASES = json.load(f)
ARRAYS = np.load(os.path.join(GOLDEN, "golden_cases.npz"))
G = 128


def test_case_list_matches_generator():
    assert CASES == json.loads(json.dumps(make_golden.CASES))


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_oracle_reproduces_fixture(oracle, case):
    for name, arr in make_golden.outputs(case).items():
        want = ARRAYS[f"{case['name']}/{name}"]
        assert np.array_equal(np.asarray(arr), want), f"{case['name']}/{name}"


@pytest.mark.gpu
@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_gpu_matches_fixture(case):
    import torch
    from kaio_b200 import ops
    from helpers import assert_attention_close, dev, device, host, max_rel
    from oracle import oracle as orc  # input generators and packing only

    x, op, name = make_golden.inputs(case), case["op"], case["name"]
    d = device()
    if op == "matmul_int8":
        m, n, k = case["m"], case["n"], case["k"]
        c = torch.full((m * n,), float("nan"), device="cuda")
        acc = torch.full((m * n,), -7, device="cuda", dtype=torch.int32)
        ops.matmul_int8(d, dev(x["a"]), dev(x["b"]), c, case["scale"], m, n, k)
        ops.matmul_int8_acc(d, dev(x["a"]), dev(x["b"]), acc, m, n, k)
        assert np.array_equal(host(acc, (m, n)), ARRAYS[f"{name}/acc"])
        assert np.array_equal(host(c, (m, n)), ARRAYS[f"{name}/c"])
    elif op == "matmul_int4":
        m, n, k = case["m"], case["n"], case["k"]
        c = torch.full((m * n,), float("nan"), device="cuda")
        ops.matmul_int4(d, dev(x["a"]), dev(orc.pack_s4(x["w"], k, n)), dev(x["scales"]), c, m, n, k, G)
        assert max_rel(host(c, (m, n)), ARRAYS[f"{name}/c"]) < 1e-3
    elif op in ("qkv_int8", "qkv_int4"):
        m, n, k = case["m"], case["n"], case["k"]
        outs = [torch.full((m * n,), float("nan"), device="cuda", dtype=torch.float16) for _ in range(3)]
        if op == "qkv_int8":
            ops.qkv_project_int8(d, dev(x["x"]), *[dev(w) for w in x["w"]], *([x["scale"]] * 3), *outs, m, n, k)
        else:
            ops.qkv_project_int4(d, dev(x["x"]), *[dev(orc.pack_s4(w, k, n)) for w in x["w"]],
                                 *[dev(s) for s in x["scales"]], *outs, m, n, k, G)
        for i, o in enumerate(outs):
            assert max_rel(host(o, (m, n)), ARRAYS[f"{name}/out{i}"]) < 1e-3
    else:
        sq, sk, dk, dv = case["sq"], case["sk"], case["dk"], case["dv"]
        out = torch.full((sq * dv,), float("nan"), device="cuda")
        fn = ops.attention_tc_causal if case["causal"] else ops.attention_tc
        fn(d, dev(x["q"]), dev(x["k"]), dev(x["v"]), out, sq, sk, dk, dv)
        assert_attention_close(host(out, (sq, dv)), ARRAYS[f"{name}/out"])
    assert ops.device_status(d)[0] == 0
