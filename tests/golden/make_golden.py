"""Writes the golden fixtures of this folder.

The reference is a Rust crate whose quantized ops run only on a GPU through its own PTX JIT, so
its outputs cannot be produced here.  What the reference's tests hold for this path are
(a) seeded input generators with fixed seeds and shapes and (b) closed-form known answers
(kaio-ops/tests/matmul_int8_e2e.rs, matmul_int4_e2e.rs, qkv_project_int8_e2e.rs,
qkv_project_int4_e2e.rs, attention_tc_api.rs).  The fixtures freeze, for those seeds and shapes,
the outputs of the CPU oracle (itself pinned to the known answers by tests/test_oracle_golden.py):

    golden_cases.npz   one array per case and output, keyed "<case>/<name>"
    golden_cases.json  the case list: op, shape, seeds, scale, and the generator of every input

Inputs are not stored: every case regenerates them from its seeds with the oracle's restatement
of the reference generators (oracle.lcg_*), which test_oracle_golden.py checks against the scalar
definition.  Run from the repository root:  python tests/golden/make_golden.py
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
from oracle import oracle  # noqa: E402

G = 128

CASES = [
    # matmul_int8_e2e.rs:72-146
    {"name": "int8_16x8x32", "op": "matmul_int8", "m": 16, "n": 8, "k": 32, "scale": 1.0, "seed": 0xA5A55A5AD00DFEED},
    {"name": "int8_64x64x128", "op": "matmul_int8", "m": 64, "n": 64, "k": 128, "scale": 0.125, "seed": 0xCAFEBABEDEADBEEF},
    {"name": "int8_128x128x128", "op": "matmul_int8", "m": 128, "n": 128, "k": 128, "scale": 0.01, "seed": 0x0123456789ABCDEF},
    {"name": "int8_17x8x32", "op": "matmul_int8", "m": 17, "n": 8, "k": 32, "scale": 1.0, "seed": 0xDEAD0001BEEF0002},
    {"name": "int8_16x13x32", "op": "matmul_int8", "m": 16, "n": 13, "k": 32, "scale": 1.0, "seed": 0xFACE0003BEEF0004},
    # matmul_int4_e2e.rs:314-397
    {"name": "int4_64x64x128", "op": "matmul_int4", "m": 64, "n": 64, "k": 128, "w_seed": 0xCAFEBABEDEADBEEF, "a_seed": 0x123456789ABCDEF0, "scale": 0.1},
    {"name": "int4_128x128x256", "op": "matmul_int4", "m": 128, "n": 128, "k": 256, "w_seed": 0xF00DFACED00D1337, "a_seed": 0xA5A55A5AD00DFEED, "scale": 0.05},
    {"name": "int4_17x8x128", "op": "matmul_int4", "m": 17, "n": 8, "k": 128, "w_seed": 0xDEAD0001BEEF0002, "a_seed": 0xFACE0003BEEF0004, "scale": 0.1},
    {"name": "int4_16x13x128", "op": "matmul_int4", "m": 16, "n": 13, "k": 128, "w_seed": 0x55555555AAAAAAAA, "a_seed": 0x1111222233334444, "scale": 0.1},
    # qkv_project_int8_e2e.rs:196-236
    {"name": "qkv8_64x16x128", "op": "qkv_int8", "m": 64, "n": 16, "k": 128, "seed": 0xCAFEBABE},
    {"name": "qkv8_128x64x64", "op": "qkv_int8", "m": 128, "n": 64, "k": 64, "seed": 0xBEEFF00D},
    # qkv_project_int4_e2e.rs (seeded correctness shapes)
    {"name": "qkv4_64x16x128", "op": "qkv_int4", "m": 64, "n": 16, "k": 128, "seed": 0xDEADBEEF},
    {"name": "qkv4_128x64x256", "op": "qkv_int4", "m": 128, "n": 64, "k": 256, "seed": 0xBEEFF00D},
    # attention_tc_api.rs (patterned inputs)
    {"name": "attn_64x128_d64", "op": "attention", "sq": 64, "sk": 128, "dk": 64, "dv": 64, "causal": False},
    {"name": "attn_64x128_d64_causal", "op": "attention", "sq": 64, "sk": 128, "dk": 64, "dv": 64, "causal": True},
    {"name": "attn_128x384_d128_causal", "op": "attention", "sq": 128, "sk": 384, "dk": 128, "dv": 128, "causal": True},
]


def inputs(case):
    """The inputs of a case, regenerated from its seeds (shared with the tests)."""
    op = case["op"]
    if op == "matmul_int8":
        m, n, k = case["m"], case["n"], case["k"]
        data = oracle.lcg_i8(case["seed"], m * k + k * n)
        return {"a": data[:m * k], "b": data[m * k:]}
    if op == "matmul_int4":
        m, n, k = case["m"], case["n"], case["k"]
        return {"w": oracle.lcg_s4(case["w_seed"], k * n), "a": oracle.lcg_f16_pm1(case["a_seed"], m * k),
                "scales": np.full((k // G) * n, case["scale"], np.float16)}
    if op == "qkv_int8":
        m, n, k = case["m"], case["n"], case["k"]
        return {"x": oracle.lcg_f16_pm_half(case["seed"], m * k),
                "w": [oracle.lcg_i8_div4(case["seed"] + i, k * n) for i in (1, 2, 3)], "scale": 1.0 / k}
    if op == "qkv_int4":
        m, n, k = case["m"], case["n"], case["k"]
        return {"x": oracle.lcg_f16_pm_half(case["seed"], m * k),
                "w": [oracle.lcg_s4(case["seed"] + i, k * n) for i in (1, 2, 3)],
                "scales": [oracle.lcg_small_scales(case["seed"] + 10 + i, (k // G) * n) for i in (1, 2, 3)]}
    if op == "attention":
        return {"q": oracle.patterned_f16(case["sq"] * case["dk"]), "k": oracle.patterned_f16(case["sk"] * case["dk"]),
                "v": oracle.patterned_f16(case["sk"] * case["dv"])}
    raise ValueError(op)


def outputs(case):
    """The oracle's outputs of a case: {name: array}."""
    op, x = case["op"], inputs(case)
    if op == "matmul_int8":
        c, acc = oracle.matmul_int8(x["a"], x["b"], case["scale"], case["m"], case["n"], case["k"], want_acc=True)
        return {"c": c, "acc": acc}
    if op == "matmul_int4":
        packed = oracle.pack_s4(x["w"], case["k"], case["n"])
        return {"c": oracle.matmul_int4(x["a"], packed, x["scales"], case["m"], case["n"], case["k"])}
    if op == "qkv_int8":
        return {f"out{i}": oracle.qkv_int8(x["x"], w, x["scale"], case["m"], case["n"], case["k"])
                for i, w in enumerate(x["w"])}
    if op == "qkv_int4":
        return {f"out{i}": oracle.qkv_int4(x["x"], oracle.pack_s4(w, case["k"], case["n"]), s, case["m"], case["n"], case["k"])
                for i, (w, s) in enumerate(zip(x["w"], x["scales"]))}
    if op == "attention":
        return {"out": oracle.attention(x["q"], x["k"], x["v"], case["sq"], case["sk"], case["dk"], case["dv"],
                                        causal=case["causal"])}
    raise ValueError(op)


def main():
    arrays = {}
    for case in CASES:
        for name, arr in outputs(case).items():
            arrays[f"{case['name']}/{name}"] = np.asarray(arr)
    np.savez_compressed(os.path.join(HERE, "golden_cases.npz"), **arrays)
    with open(os.path.join(HERE, "golden_cases.json"), "w") as f:
        json.dump(CASES, f, indent=1)
    total = sum(a.nbytes for a in arrays.values())
    print(f"{len(CASES)} cases, {len(arrays)} arrays, {total / 1024:.0f} KiB uncompressed")


if __name__ == "__main__":
    main()
