#!/usr/bin/env python
"""Benchmark of the quantized-inference hot path on B200.

One "step" = one pass of the W8A8 prefill GEMMs at the Llama-7B shapes
(M=4096; (K,N) = (4096,11008), (11008,4096), (4096,4096)), int8 x int8 -> s32, per-row
activation scale x per-column weight scale, f32 output.  `value` is whole-job W8A8 TOPS
(2*M*N*K summed over the three GEMMs and over the ranks / device time, max over ranks).  The
7B-shape weights fit one GPU, so with --gpus N > 1 every rank is a replica working on its own
M rows (weak scaling, no collective).  The sharded path -- the Llama-70B-shape W4A16 FFN GEMMs,
weights sharded over the ranks -- is measured at every N in "ffn70b_w4a16" (column-parallel GEMM
+ all-gather of its output, NCCL and fused peer stores) and "ffn_chain_70b_w4a16" (gate|up ->
SiLU-gate -> down with the sum of the partial outputs), checked against the CPU oracle in
"multi_parity" and summarised in the compact "sharded" object right behind the contract keys.

The same JSON line also carries
  * "w4a16_decode": the W4A16 decode GEMM (M in {1,8,16}, K=4096, N=11008) in HBM GB/s,
  * "int8_peak_probe" (back-to-back tcgen05.mma kind::i8 on every SM) and "w8a8_sustained" (the
    three GEMMs back to back for two seconds),
  * "roofline" of the dominant kernel, "cpu_baseline" (the CPU oracle on the host cores, a
    bounded row sample), "e2e" (same step through the public API from pinned host buffers),
    "clocks" sampled through NVML during the timed region and "gpu_launches".

`--impl reference` times the reference's own CPU implementation of the path (the oracle is the
restatement of the CPU reference functions the KAIO tests hold; the Rust crate itself cannot be
built here) on all host cores, on a bounded row sample of the same GEMMs.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M_PREFILL = 4096
GEMMS_7B = [(4096, 11008), (11008, 4096), (4096, 4096)]  # (K, N)
DECODE_K, DECODE_N = 4096, 11008
DECODE_MS = (1, 8, 16)
L2_FLUSH_BYTES = 256 << 20


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def load_traffic():
    """Per-launch DRAM traffic from the committed ncu summaries (bytes), or {}."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f)
    return {}


class ClockSampler:
    """Samples SM clock, power and throttle reasons through NVML (read-only queries) every few
    milliseconds while the timed region runs."""
    REASONS = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20,
               "hw_thermal_slowdown": 0x40, "hw_power_brake_slowdown": 0x80}

    def __init__(self, gpu_index: int):
        self.gpu_index, self.samples, self.stop_flag, self.thread = gpu_index, [], False, None
        self.handle, self.err = None, None
        try:
            import pynvml
            self.nvml = pynvml
            pynvml.nvmlInit()
            # NVML enumerates physical GPUs; honour CUDA_VISIBLE_DEVICES when it lists indices
            vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
            phys = gpu_index
            if vis and all(v.strip().isdigit() for v in vis.split(",")):
                ids = [int(v) for v in vis.split(",")]
                if gpu_index < len(ids):
                    phys = ids[gpu_index]
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception as exc:  # NVML missing: report it instead of a number
            self.err = repr(exc)

    def _loop(self):
        n = self.nvml
        while not self.stop_flag:
            try:
                sm = n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)
                pw = n.nvmlDeviceGetPowerUsage(self.handle) / 1000.0
                rs = n.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                self.samples.append((float(sm), pw, int(rs), time.perf_counter()))
            except Exception as exc:
                self.err = repr(exc)
                return
            time.sleep(0.001)

    def start(self):
        if self.handle is None:
            return
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()

    def stop(self, window=None):
        """Summary of the samples taken inside `window` = (t0, t1) in perf_counter seconds (the
        timed region); without a window, of all samples."""
        if self.thread is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [f"NVML unavailable: {self.err}"]}
        self.stop_flag = True
        self.thread.join(timeout=2)
        samples = self.samples
        if window is not None:
            inside = [t for t in samples if window[0] <= t[3] <= window[1]]
            # a timed region shorter than the sampling period: the samples nearest to it
            samples = inside if inside else sorted(samples, key=lambda t: abs(t[3] - window[0]))[:2]
        if not samples:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": [f"no samples: {self.err}"]}
        reasons = set()
        for _, _, rs, _ in samples:
            for name, bit in self.REASONS.items():
                if rs & bit:
                    reasons.add(name)
        clocks = sorted(t[0] for t in samples)
        return {"sm_mhz": clocks[len(clocks) // 2], "sm_min_mhz": clocks[0], "sm_max_mhz": self.sm_max,
                "reasons": sorted(reasons), "samples": len(samples),
                "power_w_max": max(t[1] for t in samples),
                "source": "NVML, 1 ms period, samples taken inside the timed region only"}


# ------------------------------------------------------------------------------ reference arm

def cpu_int8_sample(rows_per_gemm: int, seed: int = 42):
    """The CPU oracle on `rows_per_gemm` rows of each 7B GEMM; returns (ops, seconds, threads)."""
    import numpy as np

    from oracle import oracle as orc
    orc.build()
    # A launcher such as torchrun exports OMP_NUM_THREADS=1 to its workers: ask for the host's
    # cores explicitly so the baseline is the same at every N.
    orc.set_threads(os.cpu_count() or 1)
    rng = np.random.default_rng(seed)
    ops_total, secs = 0, 0.0
    for (k, n) in GEMMS_7B:
        a = rng.integers(-127, 128, (rows_per_gemm, k), dtype=np.int8)
        b = rng.integers(-127, 128, (k, n), dtype=np.int8)
        sa = rng.uniform(0.001, 0.01, rows_per_gemm).astype(np.float32)
        sw = rng.uniform(0.001, 0.01, n).astype(np.float32)
        t0 = time.perf_counter()
        orc.matmul_int8_scaled(a, b, sa, sw, rows_per_gemm, n, k)
        secs += time.perf_counter() - t0
        ops_total += 2 * rows_per_gemm * n * k
    return ops_total, secs, orc.num_threads()


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows = 128
    for _ in range(max(args.warmup, 1)):
        cpu_int8_sample(16)
    ops_sum, sec_sum, threads = 0, 0.0, 1
    for _ in range(args.steps):
        o, s, threads = cpu_int8_sample(rows)
        ops_sum += o
        sec_sum += s
    value = ops_sum / sec_sum / 1e12
    sample = (f"{rows} of {M_PREFILL} rows of each of the three 7B GEMMs per step, all {sum(n for _, n in GEMMS_7B)} "
              "columns, full K; CPU restatement of kaio-ops/tests/matmul_int8_e2e.rs cpu_reference with "
              "row x column scales (the Rust crate cannot be built here: no cargo/rustc)")
    line = {
        "impl": "reference", "metric": "w8a8_prefill_tops", "value": value, "unit": "TOPS",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": sec_sum / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "s8 x s8 -> s32, f32 scales", "data": "synthetic",
        "config": {"workload": "w8a8_prefill_llama7b_m4096 (row sample)", "rows_per_step": rows},
        "cpu_baseline": {"value": value, "unit": "TOPS", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------ our arm

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="kaio_b200", choices=["kaio_b200", "reference"])
    ap.add_argument("--decode-only", action="store_true",
                    help="run only the W4A16 decode leg and print its JSON (profiling aid)")
    ap.add_argument("--qkv-attention-only", action="store_true",
                    help="run only the fused-QKV + attention leg and print its JSON (profiling aid)")
    ap.add_argument("--ffn70b-only", action="store_true",
                    help="run only the 70B FFN W4A16 leg and print its JSON (profiling aid)")
    ap.add_argument("--ffn-chain-only", action="store_true",
                    help="run only the 70B W4A16 feed-forward chain leg and print its JSON (profiling aid)")
    ap.add_argument("--w8a8-only", action="store_true",
                    help="run only the INT8 peak probe and the sustained W8A8 leg (profiling aid)")
    ap.add_argument("--skip-extras", action="store_true",
                    help="only the headline step (no decode / e2e / cpu baseline legs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
        return

    import numpy as np
    import torch
    import torch.distributed as dist

    from kaio_b200 import ops, sharding

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    dev = ops.KaioDevice(local_rank)
    peaks = load_peaks()
    m = M_PREFILL

    def finish_group():
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()

    if args.decode_only:
        print(json.dumps({"w4a16_decode": bench_decode(torch, ops, dev, peaks, load_traffic())}), flush=True)
        return
    if args.qkv_attention_only:
        print(json.dumps({"qkv_attention": bench_qkv_attention(torch, ops, dev, peaks)}), flush=True)
        return
    if args.w8a8_only:
        sampler = ClockSampler(local_rank)
        sampler.start()
        print(json.dumps({"int8_peak_probe": bench_int8_probe(torch, ops, dev, sampler),
                          "w8a8_sustained": bench_w8a8_sustained(torch, ops, dev, sampler, peaks)}), flush=True)
        sampler.stop()
        return
    if args.ffn70b_only:
        res, par = bench_ffn70b(torch, dist, ops, sharding, dev, rank, world)
        if rank == 0:
            print(json.dumps({"ffn70b_w4a16": res, "gather_parity": par}), flush=True)
        finish_group()
        return
    if args.ffn_chain_only:
        res, par = bench_ffn_chain(torch, dist, ops, dev, rank, world, peaks)
        if rank == 0:
            print(json.dumps({"ffn_chain_70b_w4a16": res, "chain_parity": par}), flush=True)
        finish_group()
        return

    # ---- synthetic inputs (seeded; config 3 value ranges), resident in HBM
    g = torch.Generator(device="cuda")
    g.manual_seed(42)
    probs = []
    # The 7B-shape weights fit every GPU, so with N > 1 each rank is a replica that runs the same
    # GEMMs on its own batch of M rows (own activations, same weights): weak scaling, no collective.
    for gi, (k, n) in enumerate(GEMMS_7B):
        g.manual_seed(42 + gi + 1000 * rank)
        a = torch.randint(-127, 128, (m * k,), dtype=torch.int8, device="cuda", generator=g)
        g.manual_seed(137 + gi)
        b = torch.randint(-127, 128, (k * n,), dtype=torch.int8, device="cuda", generator=g)
        g.manual_seed(4242 + gi + 1000 * rank)
        sa = torch.rand(m, device="cuda", generator=g) * 0.009 + 0.001
        g.manual_seed(4243 + gi)
        sw = torch.rand(n, device="cuda", generator=g) * 0.009 + 0.001
        c = torch.empty(m * n, dtype=torch.float32, device="cuda")
        probs.append(dict(k=k, n=n, a=a, b=b, sa=sa, sw=sw, c=c))
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device="cuda")
    total_ops = world * sum(2 * m * n * k for k, n in GEMMS_7B)

    def gemm(p):
        ops.matmul_int8_scaled(dev, p["a"], p["b"], p["c"], p["sa"], p["sw"], m, p["n"], p["k"])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        flush.zero_()
        for p in probs:
            gemm(p)
    barrier()
    assert ops.device_status(dev)[0] == 0

    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.05)
    evs = []
    barrier()
    t_wall0 = time.perf_counter()
    for _ in range(args.steps):
        flush.zero_()  # untimed: evicts the previous step's operands from L2
        e = [torch.cuda.Event(enable_timing=True) for _ in range(len(probs) + 1)]
        e[0].record()
        for i, p in enumerate(probs):
            gemm(p)
            e[i + 1].record()
        evs.append(e)
    barrier()
    t_wall1 = time.perf_counter()
    step_ms = [e[0].elapsed_time(e[-1]) for e in evs]
    gemm_ms = [[e[i].elapsed_time(e[i + 1]) for e in evs] for i in range(len(probs))]
    total_ms = sum(step_ms)
    if world > 1:
        t = torch.tensor([total_ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    value = total_ops / (ms_per_step * 1e-3) / 1e12

    ffn = chain = decode = qkv_attn = probe = sustained = parity = None
    if not args.skip_extras and world == 1:
        probe = bench_int8_probe(torch, ops, dev, sampler)
        sustained = bench_w8a8_sustained(torch, ops, dev, sampler, peaks, probs=probs)
    clocks = sampler.stop(window=(t_wall0, t_wall1))

    e2e = None
    if not args.skip_extras:
        e2e = bench_e2e(torch, dist, ops, dev, m, total_ops, world, steps=max(3, min(args.steps, 10)))
        for p in probs:  # free the headline buffers before the other legs
            p.clear()
        del flush
        torch.cuda.empty_cache()
        if world == 1:
            # The latency-sensitive decode leg runs before the legs that allocate and free gigabytes.
            decode = bench_decode(torch, ops, dev, peaks, load_traffic())
            qkv_attn = bench_qkv_attention(torch, ops, dev, peaks)
            torch.cuda.empty_cache()
        ffn, parity_gather = bench_ffn70b(torch, dist, ops, sharding, dev, rank, world)
        torch.cuda.empty_cache()
        chain, parity_chain = bench_ffn_chain(torch, dist, ops, dev, rank, world, peaks)
        torch.cuda.empty_cache()
        if world > 1:
            checked = parity_gather["checked"] + parity_chain["checked"]
            failed = parity_gather["failed"] + parity_chain["failed"]
            parity = {"checked": checked, "failed": failed, "ok": not failed}

    if rank != 0:
        finish_group()
        if parity is not None and not parity["ok"]:
            sys.exit(3)
        return

    # ---- roofline of the dominant kernel (w8a8_gemm_2cta_kernel): per-launch ops / duration
    per_gemm = []
    for i, (k, n) in enumerate(GEMMS_7B):
        avg = sum(gemm_ms[i]) / len(gemm_ms[i])
        per_gemm.append({"k": k, "n": n, "ms": avg, "tops": 2 * m * n * k / (avg * 1e-3) / 1e12})
    int8_peak = 2.0 * peaks["bf16_tflops"]
    kern_ops = sum(2 * m * n * k for k, n in GEMMS_7B)
    kern_ms = sum(p["ms"] for p in per_gemm)
    achieved = kern_ops / (kern_ms * 1e-3) / 1e12
    traffic = load_traffic()
    roofline = {
        "bound": "tensor", "kernel": "w8a8_gemm_2cta_kernel", "achieved": achieved, "peak": int8_peak,
        "unit": "TOPS", "frac": achieved / int8_peak,
        "peak_source": f"2 x {peaks['source']} dense bf16 burst ({peaks['bf16_tflops']} TF/s), the convention "
                       "for a part whose INT8 rate is twice its bf16 rate; the INT8 rate measured in this run "
                       "is in int8_peak_probe",
        "frac_of_nominal_4500": achieved / 4500.0,
        "frac_of_probe": (achieved / probe["tops"]) if probe else None,
        "traffic": traffic.get("w8a8_gemm_kernel_bytes_per_step"),
        "per_gemm": per_gemm,
        "timing": "CUDA events around each GEMM launch on rank 0 (burst: 256 MiB memset between steps)",
    }

    line = {
        "metric": "w8a8_prefill_tops", "value": value, "unit": "TOPS", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "s8 x s8 -> s32, f32 scales", "data": "synthetic",
        "config": {"workload": "w8a8_prefill_llama7b_m4096", "m_per_gpu": m, "gemms_kn": GEMMS_7B,
                   "epilogue": "per-row x per-column f32 scales, f32 out",
                   "parallelism": "single GPU" if world == 1 else
                   f"{world} replicas (weights replicated, M={m} rows per GPU, no collective); the sharded "
                   "70B-shape FFN is in ffn70b_w4a16 / ffn_chain_70b_w4a16 / sharded",
                   "l2": f"{L2_FLUSH_BYTES >> 20} MiB memset between timed steps (untimed)",
                   "wall_s_timed_loop": t_wall1 - t_wall0},
    }
    # the compact multi-GPU objects come right behind the contract keys: a reader that keeps only the
    # first few KB of the line still has them (the last key repeats the parity result for one that
    # keeps only the end)
    if parity is not None:
        line["multi_parity"] = parity
    if ffn is not None and chain is not None:
        line["sharded"] = sharded_summary(world, ffn, chain)
    line.update({"roofline": roofline, "clocks": clocks, "gpu_launches": len(probs) * args.steps})
    if e2e is not None:
        line["e2e"] = e2e
    if not args.skip_extras and world == 1:
        rows = m  # the whole step on the host cores: about 10 s with 16 threads
        o, s, threads = cpu_int8_sample(rows)
        line["cpu_baseline"] = {
            "value": o / s / 1e12, "unit": "TOPS", "cores": threads, "kind": "port",
            "sample": f"{rows} of {m} rows of each of the three GEMMs (all columns, full K), CPU oracle, {s:.1f} s"}
        line["int8_peak_probe"] = probe
        line["w8a8_sustained"] = sustained
        line["w4a16_decode"] = decode
        line["qkv_attention"] = qkv_attn
    if ffn is not None:
        line["ffn70b_w4a16"] = ffn
    if chain is not None:
        line["ffn_chain_70b_w4a16"] = chain
    if parity is not None:
        line["multi_parity_ok"] = parity["ok"]
    print(json.dumps(line), flush=True)
    finish_group()
    if parity is not None and not parity["ok"]:
        sys.exit(3)


def sharded_summary(world, ffn, chain):
    """The sharded 70B-shape results in one small object (times in ms, max over ranks)."""
    r3 = lambda v: None if v is None else round(v, 4)
    out = {"n_gpus": world}
    c4 = chain.get("m4096", {})
    out["chain_m4096_ms"] = {k: r3(c4.get(v)) for k, v in (
        ("three_launches", "ms_three_launches"), ("two_launches_silu_epilogue", "ms_two_launches_silu_epilogue"),
        ("fused_all_reduce_silu_epilogue", "ms_fused_all_reduce_silu_epilogue"),
        ("nccl_all_reduce", "ms_with_all_reduce"),
        ("overlapped_all_reduce", "ms_overlapped_all_reduce"), ("fused_all_reduce", "ms_fused_all_reduce"),
        ("fused_pipelined_all_reduce", "ms_fused_pipelined_all_reduce"),
        ("switch_all_reduce", "ms_switch_all_reduce"), ("reduce_scatter", "ms_with_reduce_scatter"))}
    out["chain_m4096_best_all_reduce_ms"] = r3(c4.get("ms_best_all_reduce"))
    for mm in (16, 256):
        cm = chain.get(f"m{mm}", {})
        out[f"chain_m{mm}_ms"] = {"graph_nccl": r3(cm.get("graph_ms_with_all_reduce")),
                                  "graph_fused": r3(cm.get("graph_ms_fused_all_reduce")),
                                  "graph_local": r3(cm.get("graph_ms_three_launches"))}
    for key, label in (("k8192_n28672", "upgate"), ("k28672_n8192", "down")):
        for mm in (16, 256, 4096):
            e = ffn.get(f"{key}_m{mm}", {})
            out[f"cfg5_{label}_m{mm}_ms"] = {"gemm": r3(e.get("ms_gemm")), "nccl_gather": r3(e.get("ms_gemm_plus_gather")),
                                             "fused": r3(e.get("ms_fused_peer_store"))}
    return out


def bench_int8_probe(torch, ops, dev, sampler):
    """The INT8 tensor-pipe rate this GPU delivers with nothing in the way: every SM issues
    back-to-back tcgen05.mma kind::i8 M128 N256 K32 on zeroed shared-memory operands.  Reported
    in TOPS and, with the SM clock NVML shows while it runs, in MAC per clock per SM."""
    iters = 1 << 17  # ~9 ms per launch at the full rate
    for _ in range(3):
        ops.probe_int8_mma_rate(dev, iters)
    torch.cuda.synchronize()
    n_launch = 40
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    work = 0
    for _ in range(n_launch):
        work += ops.probe_int8_mma_rate(dev, iters)
    e1.record()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    ms = e0.elapsed_time(e1)
    tops = work / (ms * 1e-3) / 1e12
    inside = [s[0] for s in sampler.samples if t0 + 0.1 * (t1 - t0) <= s[3] <= t1]
    mhz = sorted(inside)[len(inside) // 2] if inside else None
    sms = torch.cuda.get_device_properties(dev.ordinal).multi_processor_count
    return {"tops": tops, "ms": ms, "launches": n_launch, "sm_mhz_median": mhz,
            "mac_per_clk_per_sm": (work / 2 / (ms * 1e-3) / (mhz * 1e6) / sms) if mhz else None,
            "frac_of_nominal_4500": tops / 4500.0,
            "what": "one CTA per SM, back-to-back tcgen05.mma.cta_group::1.kind::i8 M128 N256 K32, no loads, "
                    "no epilogue; ~0.35 s under load, so the clock is the sustained one"}


def bench_w8a8_sustained(torch, ops, dev, sampler, peaks, probs=None, seconds=2.0):
    """The three config-3 GEMMs back to back for >= 2 s with nothing between them: the rate the
    kernel holds at the clock the power cap allows, next to the burst figure of the headline."""
    m = M_PREFILL
    own = probs is None
    if own:
        g = torch.Generator(device="cuda")
        probs = []
        for gi, (k, n) in enumerate(GEMMS_7B):
            g.manual_seed(42 + gi)
            probs.append(dict(k=k, n=n,
                              a=torch.randint(-127, 128, (m * k,), dtype=torch.int8, device="cuda", generator=g),
                              b=torch.randint(-127, 128, (k * n,), dtype=torch.int8, device="cuda", generator=g),
                              sa=torch.rand(m, device="cuda", generator=g) * 0.009 + 0.001,
                              sw=torch.rand(n, device="cuda", generator=g) * 0.009 + 0.001,
                              c=torch.empty(m * n, dtype=torch.float32, device="cuda")))
    ops_step = sum(2 * m * n * k for k, n in GEMMS_7B)

    def step():
        for p in probs:
            ops.matmul_int8_scaled(dev, p["a"], p["b"], p["c"], p["sa"], p["sw"], m, p["n"], p["k"])

    for _ in range(20):
        step()
    torch.cuda.synchronize()
    n_steps = int(seconds / 0.30e-3)  # ~0.3 ms per step at the burst rate
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for _ in range(n_steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    ms = e0.elapsed_time(e1)
    tops = n_steps * ops_step / (ms * 1e-3) / 1e12
    inside = [s for s in sampler.samples if t0 + 0.25 * (t1 - t0) <= s[3] <= t1]
    mhz = sorted(s[0] for s in inside)[len(inside) // 2] if inside else None
    sm_max = sampler.sm_max if sampler.handle is not None else None
    reasons = sorted({name for s in inside for name, bit in ClockSampler.REASONS.items() if s[2] & bit})
    return {"tops": tops, "seconds": ms * 1e-3, "steps": n_steps, "launches": 3 * n_steps,
            "sm_mhz_median": mhz, "sm_max_mhz": sm_max, "reasons": reasons,
            "power_w_max": max((s[1] for s in inside), default=None),
            "tops_at_max_clock": (tops * sm_max / mhz) if mhz and sm_max else None,
            "frac_of_2x_bf16_sustained": tops / (2.0 * peaks["bf16_tflops_sustained"]),
            "frac_of_nominal_4500": tops / 4500.0,
            "note": "no L2 flush and no gap between launches; operands of one step (61.9 MB) exceed half of L2 "
                    "and the f32 outputs (315 MB) stream to HBM"}


def bench_decode(torch, ops, dev, peaks, traffic):
    """W4A16 decode GEMM, M in {1,8,16}, K=4096, N=11008, f16 out.  Launches are replayed from a
    CUDA graph (the kernel is a few microseconds: host launch cost would otherwise dominate) and
    rotate over 12 distinct weight buffers (276 MB > L2) so the weights come from HBM."""
    k, n = DECODE_K, DECODE_N
    nb = 12
    g = torch.Generator(device="cuda")
    g.manual_seed(137)
    ws = [torch.randint(-2 ** 31, 2 ** 31 - 1, (k // 8 * n,), dtype=torch.int32, device="cuda", generator=g)
          for _ in range(nb)]
    sc = [(torch.rand(k // 128 * n, device="cuda", generator=g) * 0.015 + 0.005).half() for _ in range(nb)]
    out = {}
    stream = torch.cuda.Stream()
    sdev = ops.KaioDevice(dev.ordinal, stream)
    for mm in DECODE_MS:
        a = torch.randn(mm * k, device="cuda", generator=g).half()
        c = torch.zeros(mm * n, dtype=torch.float16, device="cuda")
        torch.cuda.synchronize()
        with torch.cuda.stream(stream):  # warm-up + the stream's scratch allocation, before capture
            for i in range(nb):
                ops.matmul_int4(sdev, a, ws[i], sc[i], c, mm, n, k, 128)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        reps = 4
        with torch.cuda.stream(stream):
            with torch.cuda.graph(graph, stream=stream):
                for _ in range(reps):
                    for i in range(nb):
                        ops.matmul_int4(sdev, a, ws[i], sc[i], c, mm, n, k, 128)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_replay = 5
        with torch.cuda.stream(stream):
            e0.record(stream)
            for _ in range(n_replay):
                graph.replay()
            e1.record(stream)
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (n_replay * reps * nb)
        nbytes = k * n // 2 + (k // 128) * n * 2 + 2 * mm * k + 2 * mm * n
        gbs = nbytes / us / 1e3
        out[f"m{mm}"] = {"us_per_launch": us, "gbs": gbs, "algorithmic_bytes": nbytes,
                         "frac_of_measured_hbm": gbs / peaks["hbm_gbs"], "frac_of_8tbs": gbs / 8000.0}
    out["variant"] = ops.last_variant()
    out["roofline"] = {"bound": "hbm", "kernel": "w4a16_decode_kernel", "achieved": out["m16"]["gbs"],
                       "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": out["m16"]["gbs"] / peaks["hbm_gbs"],
                       "traffic": traffic.get("w4a16_decode_kernel_bytes_per_launch")}
    return out


def bench_e2e(torch, dist, ops, dev, m, total_ops, world, steps):
    """The same step through the public API from pinned host memory: activations are copied
    host->device and the f32 outputs device->host inside the timed region, every step (weights and
    scales are model state and stay resident, as in the reference where they live in GpuBuffers).
    Three streams (copy in, compute, copy out) and two sets of device buffers let the upload of
    one GEMM overlap the download of the previous one; every copy and every GEMM of every step
    still runs inside the timed region."""
    g = torch.Generator(device="cuda")
    probs = []
    for gi, (k, n) in enumerate(GEMMS_7B):
        g.manual_seed(42 + gi)
        a = [torch.randint(-127, 128, (m * k,), dtype=torch.int8, device="cuda", generator=g) for _ in range(2)]
        b = torch.randint(-127, 128, (k * n,), dtype=torch.int8, device="cuda", generator=g)
        sa = torch.rand(m, device="cuda", generator=g) * 0.009 + 0.001
        sw = torch.rand(n, device="cuda", generator=g) * 0.009 + 0.001
        c = [torch.empty(m * n, dtype=torch.float32, device="cuda") for _ in range(2)]
        probs.append(dict(k=k, n=n, a=a, b=b, sa=sa, sw=sw, c=c))
    host_a = [torch.empty(p["a"][0].numel(), dtype=torch.int8).pin_memory() for p in probs]
    host_c = [torch.empty(p["c"][0].numel(), dtype=torch.float32).pin_memory() for p in probs]
    for h, p in zip(host_a, probs):
        h.copy_(p["a"][0].cpu())
    h2d = sum(h.numel() for h in host_a)
    d2h = sum(h.numel() * 4 for h in host_c)
    s_in, s_run, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    dev_run = ops.KaioDevice(dev.ordinal, s_run)
    ev = lambda: torch.cuda.Event()
    a_free = [[ev() for _ in range(2)] for _ in probs]   # GEMM that read a[set] has finished
    c_free = [[ev() for _ in range(2)] for _ in probs]   # download of c[set] has finished
    for gi in range(len(probs)):
        for st in range(2):
            a_free[gi][st].record(s_run)
            c_free[gi][st].record(s_out)

    def one(step):
        st = step & 1
        for gi, (h, hc, p) in enumerate(zip(host_a, host_c, probs)):
            with torch.cuda.stream(s_in):
                s_in.wait_event(a_free[gi][st])
                p["a"][st].copy_(h, non_blocking=True)
                up = ev()
                up.record(s_in)
            with torch.cuda.stream(s_run):
                s_run.wait_event(up)
                s_run.wait_event(c_free[gi][st])
                ops.matmul_int8_scaled(dev_run, p["a"][st], p["b"], p["c"][st], p["sa"], p["sw"], m, p["n"], p["k"])
                a_free[gi][st].record(s_run)
                done = ev()
                done.record(s_run)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                hc.copy_(p["c"][st], non_blocking=True)
                c_free[gi][st].record(s_out)

    for i in range(2):
        one(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for i in range(steps):
        one(i)
    torch.cuda.synchronize()
    dt = (time.perf_counter() - t0) / steps
    if world > 1:  # every rank runs its own replica's round trip; the job is as slow as the slowest
        t = torch.tensor([dt], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t.item())
    return {"value": total_ops / dt / 1e12, "unit": "TOPS", "ms_per_step": dt * 1e3,
            "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world,
            "note": "int8 activations H2D and f32 outputs D2H every step from/to pinned memory on every rank, "
                    "copies and GEMMs on three streams, max over ranks; bound by the PCIe download of the "
                    "f32 outputs"}


def _time_ms(torch, fn, iters, warm=2):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def bench_qkv_attention(torch, ops, dev, peaks):
    """Config 4: fused QKV projection (W8A16 with per-column scales; W4A16) at M = 8 x 2048,
    K = N = 4096, and causal multi-head attention (32 heads x 128) on the projection outputs."""
    bsz, seq, heads, hd = 8, 2048, 32, 128
    m, k, n = bsz * seq, 4096, heads * hd
    g = torch.Generator(device="cuda")
    g.manual_seed(42)
    x = torch.randn(m * k, device="cuda", generator=g).half()
    outs = [torch.empty(m * n, dtype=torch.float16, device="cuda") for _ in range(3)]
    w8 = [torch.randint(-127, 128, (k * n,), dtype=torch.int8, device="cuda", generator=g) for _ in range(3)]
    # per-column scales in the configuration's range [1e-3, 1e-2]: |acc| ~ 5e3 * 1e-2, far from f16 overflow
    cs = [torch.rand(n, device="cuda", generator=g) * 0.009 + 0.001 for _ in range(3)]
    t8 = _time_ms(torch, lambda: ops.qkv_project_int8(dev, x, *w8, *cs, *outs, m, n, k), 5)
    v8 = ops.last_variant()
    # the W8A8 form: x quantised per row on the fly (inside the timing), INT8 tensor pipe
    t88 = _time_ms(torch, lambda: ops.qkv_project_w8a8(dev, x, *w8, *cs, *outs, m, n, k), 5)
    v88 = ops.last_variant()
    del w8
    w4 = [torch.randint(-2 ** 31, 2 ** 31 - 1, (k // 8 * n,), dtype=torch.int32, device="cuda", generator=g)
          for _ in range(3)]
    sc = [(torch.rand(k // 128 * n, device="cuda", generator=g) * 0.015 + 0.005).half() for _ in range(3)]
    t4 = _time_ms(torch, lambda: ops.qkv_project_int4(dev, x, *w4, *sc, *outs, m, n, k, 128), 5)
    v4 = ops.last_variant()
    o = torch.empty(m * n, dtype=torch.float16, device="cuda")
    ta = _time_ms(torch, lambda: ops.attention_mha_f16(dev, outs[0], outs[1], outs[2], o, bsz, heads, seq, seq,
                                                       hd, n, True), 5)
    va = ops.last_variant()
    qkv_flops = 6 * m * n * k
    attn_flops = 4 * bsz * heads * seq * seq * hd // 2
    f16_peak = peaks["bf16_tflops"]
    return {
        "qkv_w8a16_colscale": {"ms": t8, "tflops": qkv_flops / t8 / 1e9, "frac_of_measured_f16": qkv_flops / t8 / 1e9 / f16_peak, "variant": v8},
        "qkv_w8a8": {"ms": t88, "tops": qkv_flops / t88 / 1e9, "frac_of_2x_measured_f16": qkv_flops / t88 / 1e9 / (2 * f16_peak),
                     "frac_of_nominal_4500": qkv_flops / t88 / 1e9 / 4500.0, "variant": v88,
                     "note": "includes the per-row quantisation pass of x (134 MB read, 67 MB written)"},
        "qkv_w4a16": {"ms": t4, "tflops": qkv_flops / t4 / 1e9, "frac_of_measured_f16": qkv_flops / t4 / 1e9 / f16_peak, "variant": v4},
        "attention_causal_mha": {"ms": ta, "tflops": attn_flops / ta / 1e9, "frac_of_measured_f16": attn_flops / ta / 1e9 / f16_peak, "variant": va},
        "flops": {"qkv": qkv_flops, "attention_causal": attn_flops},
        "note": "each timing includes the dequantisation pre-pass of the call; attention flops count the causal half",
    }




L2_ROTATE_BYTES = 256 << 20  # weights cycled through per timed loop at M <= 256: twice the L2


def _max_over_ranks(torch, dist, world, values):
    t = torch.tensor(values, dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t]


def _max_rel(np, got, want):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    return float(np.max(np.abs(got - want) / np.maximum(np.abs(want), 1.0)))


def _max_rel_rowscale(np, got, want):
    """|g - w| / max(|w|, rms of w's row).  For the output of a chain with f16 intermediates: a
    last-place difference in an intermediate moves every output of the row by an amount
    proportional to the row's scale, so the error is judged against that scale (at the 70B shapes
    the outputs have an rms near 150 and individual values anywhere down to zero)."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    rms = np.sqrt(np.mean(want * want, axis=-1, keepdims=True))
    return float(np.max(np.abs(got - want) / np.maximum(np.abs(want), np.maximum(rms, 1.0))))


def bench_ffn70b(torch, dist, ops, sharding, dev, rank, world):
    """Config 5: Llama-70B-shape W4A16 FFN GEMMs, N-sharded over the ranks, f16 output all-gathered
    to [M, N] on every rank.  Times are CUDA events, max over ranks.  Reported: the GEMM alone, the
    GEMM followed by the NCCL gather, and the fused form (one kernel whose epilogue stores each
    tile into every rank's buffer over peer memory, followed by a symmetric-memory barrier).  At
    M <= 256 the timed loops cycle through enough distinct weight shards to exceed twice the L2,
    so the weights come from HBM at every N.

    Returns (results, parity): with more than one rank the fused output is compared bit for bit
    with the NCCL-gathered one at M = 16 and 256, and two rows of it with the CPU oracle."""
    import numpy as np
    res, checked, failed = {}, [], []
    g = torch.Generator(device="cuda")
    for (k, n) in [(8192, 28672), (28672, 8192)]:
        n_loc = n // world
        shard_bytes = (k // 8) * n_loc * 4
        copies = max(1, -(-L2_ROTATE_BYTES // shard_bytes))
        sets = []
        for r in range(copies):
            g.manual_seed(137 + rank + 1000 * r)
            w = torch.randint(-2 ** 31, 2 ** 31 - 1, (k // 8 * n_loc,), dtype=torch.int32, device="cuda", generator=g)
            sc = (torch.rand(k // 128 * n_loc, device="cuda", generator=g) * 0.015 + 0.005).half()
            sets.append((w, sc))
        for mm in (16, 256, 4096):
            g.manual_seed(42)
            a = torch.randn(mm * k, device="cuda", generator=g).half()
            c = torch.empty(mm * n_loc, dtype=torch.float16, device="cuda")
            gather = sharding.ColumnGather(mm, n, torch.float16, "cuda") if world > 1 else None
            rotate = len(sets) if mm <= 256 else 1
            turn = [0]

            def next_set():
                turn[0] = (turn[0] + 1) % rotate
                return sets[turn[0]]

            def gemm():
                w, sc = next_set()
                ops.matmul_int4(dev, a, w, sc, c, mm, n_loc, k, 128)

            def both():
                gemm()
                if gather is not None:
                    gather(c)

            iters = max(20, 2 * rotate) if mm <= 256 else 5
            t_gemm = _time_ms(torch, gemm, iters)
            variant = ops.last_variant()
            t_all = _time_ms(torch, both, iters) if world > 1 else t_gemm
            t_fused = t_all
            fused_variant = None
            if world > 1:
                # one kernel per rank: the epilogue stores into every rank's buffer (peer memory)
                fused = sharding.FusedGatherGemm(ops, dev, mm, n, k, world, rank)

                def run_fused():
                    w, sc = next_set()
                    fused.run(a, w, sc)

                t_fused = _time_ms(torch, run_fused, iters)
                fused_variant = ops.last_variant()
                # checked at every M: the multicast epilogue serves only the large ones
                name = f"cfg5_k{k}_n{n}_m{mm}"
                ok = _check_gather(torch, dist, ops, np, dev, rank, world, fused, gather, a, c, sets[0],
                                   mm, n, k)
                checked.append(name)
                if not ok:
                    failed.append(name)
                del fused
            t_gemm, t_all, t_fused = _max_over_ranks(torch, dist, world, [t_gemm, t_all, t_fused])
            best = min(t_all, t_fused)
            flops = 2 * mm * n * k
            nbytes = k * n // 2 + (k // 128) * n * 2 + 2 * mm * k + 2 * mm * n
            res[f"k{k}_n{n}_m{mm}"] = {
                "ms_gemm": t_gemm, "ms_gemm_plus_gather": t_all, "ms_fused_peer_store": t_fused,
                "tflops": flops / best / 1e9, "weight_stream_gbs": nbytes / best / 1e6,
                "weight_sets_cycled": rotate, "variant": variant,
                "fused_variant": fused_variant if world > 1 else None}
            del a, c, gather
        del sets
        torch.cuda.empty_cache()
    res["note"] = ("whole-job figures over all ranks (tflops / weight_stream_gbs use the better of NCCL gather and "
                   "fused peer stores); weight_stream_gbs = algorithmic bytes of the full GEMM / time; at M <= 256 "
                   "the loops cycle through weight_sets_cycled distinct shards (> 2 x L2 in total)")
    return res, {"checked": checked, "failed": failed}


def _check_gather(torch, dist, ops, np, dev, rank, world, fused, gather, a, c, wset, mm, n, k):
    """Fused all-gather output == NCCL-gathered output bit for bit on every rank, and two of its
    rows == the CPU oracle's product over the full (re-assembled) weights on rank 0."""
    from oracle import oracle as orc
    w, sc = wset
    n_loc = n // world
    out_f = fused.run(a, w, sc).clone()
    ops.matmul_int4(dev, a, w, sc, c, mm, n_loc, k, 128)
    out_g = gather(c).clone()
    torch.cuda.synchronize()
    ok = bool(torch.equal(out_f.view(torch.int16), out_g.view(torch.int16)))
    # re-assemble the full weights on rank 0: packed columns are contiguous (flat concat in rank
    # order); group scales are [K/128, N/P] per rank (concat along columns)
    w_all = torch.empty(world * w.numel(), dtype=torch.int32, device="cuda")
    s_all = torch.empty(world * sc.numel(), dtype=torch.float16, device="cuda")
    dist.all_gather_into_tensor(w_all, w)
    dist.all_gather_into_tensor(s_all, sc)
    if rank == 0:
        orc.build()
        orc.set_threads(os.cpu_count() or 1)
        packed = w_all.cpu().numpy().view(np.uint32)
        scales = np.ascontiguousarray(
            s_all.cpu().numpy().reshape(world, k // 128, n_loc).transpose(1, 0, 2)).reshape(-1)
        rows = [0, mm - 1]
        a_rows = a.view(mm, k)[rows].cpu().numpy()
        want = orc.matmul_int4(a_rows.reshape(-1), packed, scales, len(rows), n, k, f16_out=True)
        got = out_f.view(mm, n)[rows].cpu().numpy()
        ok = ok and _max_rel(np, got, want) < 2e-2
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    return bool(flag.item())


def _graph_ms(torch, fn, reps, replays=10):
    """`fn` called `reps` times, captured into one CUDA graph; ms per call when the graph is replayed."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(reps):  # warm-up on the capture stream: scratch of that stream exists before capture
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        for _ in range(reps):
            fn()
    return _time_ms(torch, graph.replay, replays) / reps


def bench_ffn_chain(torch, dist, ops, dev, rank, world, peaks):
    """The W4A16 feed-forward chain at Llama-70B shapes (hidden 8192, intermediate 28672):
    gate|up projection (one GEMM), SiLU-gate, down projection; across ranks column-parallel then
    row-parallel, so the only exchange is the sum of the [M, 8192] f32 partial outputs.  CUDA
    events, max over ranks.

    M = 16 / 256: the chain replayed from a CUDA graph (its launches are a few microseconds each),
    cycling through enough distinct weight sets to exceed twice the L2: the three launches alone,
    with the NCCL all-reduce, with the all-reduce fused into the down projection.
    M = 4096: the three launches, then with NCCL all-reduce / reduce-scatter, with the fused
    all-reduce, and with the all-reduce overlapped chunk by chunk behind the GEMMs.

    Returns (results, parity): with more than one rank every reduction form is compared with the
    stage-wise CPU oracle on two rows, and the fused form's bits are compared across ranks."""
    import numpy as np

    from kaio_b200 import ffn as ffn_mod
    hidden, inter = 8192, 28672
    g = torch.Generator(device="cuda")
    g.manual_seed(137)

    def packed(k, n):
        return torch.randint(-2 ** 31, 2 ** 31 - 1, (k // 8 * n,), dtype=torch.int32, device="cuda", generator=g)

    def scales(k, n):
        return (torch.rand(k // 128 * n, device="cuda", generator=g) * 0.015 + 0.005).half()

    # the same seed on every rank: every rank holds the same unsharded weights and keeps its shard
    weights = [packed(hidden, inter), scales(hidden, inter), packed(hidden, inter), scales(hidden, inter),
               packed(inter, hidden), scales(inter, hidden)]
    host_weights = [t.cpu().numpy() for t in weights] if (world > 1 and rank == 0) else None
    chain = ffn_mod.FfnInt4(ops, dev, hidden, inter, *weights, world=world, rank=rank, max_m=4096, reduce="all")
    scatter_rows = torch.empty((4096 // world) * hidden, dtype=torch.float32, device="cuda") if world > 1 else None
    fused_ok = world > 1
    if world > 1:
        try:  # symmetric memory may be unavailable: then only the NCCL forms are timed
            chain._init_fused(torch.device("cuda", torch.cuda.current_device()))
        except Exception as exc:  # noqa: BLE001
            fused_ok = False
            print(f"fused all-reduce unavailable on rank {rank}: {exc!r}", file=sys.stderr, flush=True)
        flag = torch.tensor([1 if fused_ok else 0], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)  # every rank or none
        fused_ok = bool(flag.item())
    switch_ok = fused_ok
    if switch_ok:
        try:  # the in-switch all-reduce needs NVLink multicast addresses for the symmetric buffers
            chain._init_switch()
        except Exception as exc:  # noqa: BLE001
            switch_ok = False
            print(f"in-switch all-reduce unavailable on rank {rank}: {exc!r}", file=sys.stderr, flush=True)
        flag = torch.tensor([1 if switch_ok else 0], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        switch_ok = bool(flag.item())
    del weights
    torch.cuda.empty_cache()
    il = chain.i_loc
    # weight sets for the M <= 256 loops: set 0 is the chain's own shard, the others are random
    # shards of the same shapes
    set_bytes = chain.w_gu.numel() * 4 + chain.w_down.numel() * 4
    copies = max(1, -(-L2_ROTATE_BYTES // set_bytes))
    copies += copies % 2  # an even number: the one-step fused form alternates two staging buffers
    sets = [(chain.w_gu, chain.s_gu, chain.w_down, chain.s_down)]
    for r in range(1, copies):
        g.manual_seed(977 + rank + 1000 * r)
        sets.append((packed(hidden, 2 * il), scales(hidden, 2 * il), packed(il, hidden), scales(il, hidden)))
    turn = [0]

    def use_next_set(rotate):
        turn[0] = (turn[0] + 1) % rotate
        chain.w_gu, chain.s_gu, chain.w_down, chain.s_down = sets[turn[0]]

    res, checked, failed = {}, [], []
    for mm in (16, 256, 4096):
        g.manual_seed(42)
        x = (torch.randn(mm * hidden, device="cuda", generator=g)).half()
        rotate = len(sets) if mm <= 256 else 1

        def gate_up():
            ops.matmul_int4(dev, x, chain.w_gu, chain.s_gu, chain.gu, mm, 2 * il, hidden, 128)

        def act():
            ops.silu_gate_f16(dev, chain.gu, chain.gu.view(-1)[il:], chain.act, mm, il, x_ld=2 * il, gate_ld=2 * il)

        def down():
            ops.matmul_int4(dev, chain.act, chain.w_down, chain.s_down, chain.out, mm, hidden, il, 128)

        def local():
            use_next_set(rotate)
            chain.local(x, mm)

        def with_all_reduce():
            use_next_set(rotate)
            dist.all_reduce(chain.local(x, mm), op=dist.ReduceOp.SUM)

        def with_reduce_scatter():
            dist.reduce_scatter_tensor(scatter_rows[: (mm // world) * hidden], chain.local(x, mm).view(-1),
                                       op=dist.ReduceOp.SUM)

        def fused():
            use_next_set(rotate)
            chain.run_fused(x, mm)

        local()
        gate_up()
        variant_gu = ops.last_variant()
        down()
        variant_down = ops.last_variant()
        entry = {"variants": [variant_gu, "silu_gate_f16", variant_down], "weight_sets_cycled": rotate}
        flops = 2 * mm * hidden * inter * 3
        wbytes = 3 * (hidden * inter // 2 + (hidden // 128) * inter * 2)
        if mm <= 256:
            iters = 20
            t_gu, t_act, t_down = [_time_ms(torch, f, iters) for f in (gate_up, act, down)]
            tg = [_graph_ms(torch, local, rotate)]
            if world > 1:
                tg += [_graph_ms(torch, with_all_reduce, rotate), _graph_ms(torch, fused, rotate) if fused_ok else 0.0]
            else:
                tg += [tg[0], tg[0]]
            t_gu, t_act, t_down, g_local, g_ar, g_fused = _max_over_ranks(torch, dist, world,
                                                                          [t_gu, t_act, t_down] + tg)
            best = min(g_ar, g_fused) if (world > 1 and fused_ok) else g_ar
            entry.update({
                "ms_gate_up_gemm": t_gu, "ms_silu_gate": t_act, "ms_down_gemm": t_down,
                "graph_ms_three_launches": g_local, "graph_ms_with_all_reduce": g_ar,
                "graph_ms_fused_all_reduce": g_fused if fused_ok else None,
                "fused_form": "-" if not fused_ok else ("one step" if mm <= chain.m_one else "two steps"),
                "tflops": flops / best / 1e9, "weight_stream_gbs": wbytes / best / 1e6})
        else:
            iters = 5
            ts = [_time_ms(torch, f, iters) for f in (gate_up, act, down, local)]
            chunk_sets = [chain.default_chunks(mm), [mm // 2, mm // 2]]
            if world > 1:
                # the reductions, timed in two rounds in opposite order (the GPU sits at its power cap
                # at M = 4096, so whatever is timed last would otherwise look slowest); min of the two
                forms = [with_all_reduce, with_reduce_scatter if mm % world == 0 else with_all_reduce,
                         fused if fused_ok else with_all_reduce]
                forms += [(lambda ch=ch: chain.run_overlapped(x, mm, chunks=ch)) for ch in chunk_sets]
                fp_chunks = [[mm // 2, mm // 2], [mm // 4] * 4]
                forms += [(lambda ch=ch: chain.run_fused_pipelined(x, mm, chunks=ch)) if fused_ok else with_all_reduce
                          for ch in fp_chunks]
                sw_chunks = [[mm], [mm // 2, mm // 2]]
                forms += [(lambda ch=ch: chain.run_switch(x, mm, chunks=ch)) if switch_ok else with_all_reduce
                          for ch in sw_chunks]
                first = [_time_ms(torch, f, iters) for f in forms]
                second = [_time_ms(torch, f, iters) for f in reversed(forms)][::-1]
                ts += [min(a, b) for a, b in zip(first, second)]
            else:
                ts += [ts[3]] * 3 + [_time_ms(torch, lambda ch=ch: chain.run_overlapped(x, mm, chunks=ch), iters)
                                     for ch in chunk_sets] + [ts[3]] * 4
                fp_chunks = [[mm], [mm]]
                sw_chunks = [[mm], [mm]]
            t_gu, t_act, t_down, t_local, t_ar, t_rs, t_fused, t_ov0, t_ov1, t_fp0, t_fp1, t_sw0, t_sw1 = \
                _max_over_ranks(torch, dist, world, ts)
            t_sw, sw_best = (t_sw0, sw_chunks[0]) if t_sw0 <= t_sw1 else (t_sw1, sw_chunks[1])
            # gate|up and the SiLU-gate as one launch (activation in the GEMM's epilogue): the local
            # chain and, at N > 1, the fused all-reduce form on top of it
            # (timed in alternation with the three-launch form, two rounds, min of each: at M = 4096 the
            # GPU drifts along its power cap, so forms timed minutes apart do not compare)
            chain.enable_fused_silu()
            pair_a, pair_b = [], []
            for _ in range(2):
                chain.enable_fused_silu(False)
                pair_a.append(_time_ms(torch, lambda: chain.local(x, mm), iters))
                chain.enable_fused_silu(True)
                pair_b.append(_time_ms(torch, lambda: chain.local(x, mm), iters))
            fs = [min(pair_b), min(pair_a)]
            if world > 1 and fused_ok:
                fs.append(_time_ms(torch, lambda: chain.run_fused(x, mm), iters))
            chain.enable_fused_silu(False)
            fs = _max_over_ranks(torch, dist, world, fs)
            t_local_same = fs[1]
            fs = [fs[0]] + fs[2:]
            t_local_fs, t_fused_fs = fs[0], (fs[1] if len(fs) > 1 else None)
            stage_ms = None
            if world > 1 and fused_ok:
                # where the fused form's time goes: events between its launches, 5 runs, the mean per
                # stage, max over ranks (a stage that waits for the slowest rank shows as a long barrier)
                labels, sums = [], {}
                for it in range(2 + iters):
                    evs = []

                    def mark(label):
                        ev = torch.cuda.Event(enable_timing=True)
                        ev.record()
                        evs.append((label, ev))
                    mark("start")
                    chain.run_fused(x, mm, mark=mark)
                    torch.cuda.synchronize()
                    if it >= 2:
                        labels = [l for l, _ in evs[1:]]
                        for (_, a), (l, b) in zip(evs[:-1], evs[1:]):
                            sums[l] = sums.get(l, 0.0) + a.elapsed_time(b) / iters
                vals = _max_over_ranks(torch, dist, world, [sums[l] for l in labels])
                stage_ms = {l: round(v, 4) for l, v in zip(labels, vals)}
                stage_ms["store_back"] = "multicast" if chain.out_mc else "peer stores"
            switch_stage_ms = None
            if world > 1 and switch_ok:
                labels, sums = [], {}
                for it in range(2 + iters):
                    evs = []

                    def mark(label):
                        ev = torch.cuda.Event(enable_timing=True)
                        ev.record()
                        evs.append((label, ev))
                    mark("start")
                    chain.run_switch(x, mm, mark=mark)
                    torch.cuda.synchronize()
                    if it >= 2:
                        labels = [l for l, _ in evs[1:]]
                        for (_, a), (l, b) in zip(evs[:-1], evs[1:]):
                            sums[l] = sums.get(l, 0.0) + a.elapsed_time(b) / iters
                vals = _max_over_ranks(torch, dist, world, [sums[l] for l in labels])
                switch_stage_ms = {l: round(v, 4) for l, v in zip(labels, vals)}
            t_fp, fp_best = (t_fp0, fp_chunks[0]) if t_fp0 <= t_fp1 else (t_fp1, fp_chunks[1])
            t_ov, ov_chunks = (t_ov0, chunk_sets[0]) if t_ov0 <= t_ov1 else (t_ov1, chunk_sets[1])
            best = min(t_ar, t_fused, t_ov, t_fp, t_sw) if world > 1 else min(t_local, t_local_fs)
            if t_fused_fs is not None:
                best = min(best, t_fused_fs)
            act_bytes = 3 * mm * il * 2  # one rank's SiLU-gate pass: two f16 reads and one f16 write per element
            entry.update({
                "ms_gate_up_gemm": t_gu, "ms_silu_gate": t_act, "ms_down_gemm": t_down, "ms_three_launches": t_local,
                "ms_two_launches_silu_epilogue": t_local_fs, "ms_three_launches_same_window": t_local_same,
                "ms_fused_all_reduce_silu_epilogue": t_fused_fs,
                "ms_with_all_reduce": t_ar, "ms_with_reduce_scatter": t_rs,
                "ms_fused_all_reduce": t_fused if fused_ok else None, "fused_stage_ms": stage_ms,
                "ms_overlapped_all_reduce": t_ov, "overlap_chunks": ov_chunks,
                "ms_fused_pipelined_all_reduce": t_fp if (fused_ok and world > 1) else None,
                "fused_pipelined_chunks": fp_best,
                "ms_switch_all_reduce": t_sw if (switch_ok and world > 1) else None, "switch_chunks": sw_best,
                "ms_switch_all_reduce_unchunked": t_sw0 if (switch_ok and world > 1) else None,
                "switch_stage_ms": switch_stage_ms,
                "ms_best_all_reduce": best,
                "fused_form": "-" if not fused_ok else ("one step" if mm <= chain.m_one else "two steps"),
                "tflops": flops / best / 1e9, "weight_stream_gbs": wbytes / best / 1e6,
                "silu_gate_gbs": act_bytes / t_act / 1e6,
                "silu_gate_frac_of_hbm_peak": act_bytes / t_act / 1e6 / peaks["hbm_gbs"]})
        if world > 1:
            chain.w_gu, chain.s_gu, chain.w_down, chain.s_down = sets[0]
            name = f"chain_m{mm}"
            ok = _check_chain(torch, dist, ops, np, chain, x, mm, hidden, inter, rank, world, fused_ok, switch_ok,
                              host_weights)
            checked.append(name)
            if not ok:
                failed.append(name)
        res[f"m{mm}"] = entry
        del x
    res["note"] = ("whole-job figures over all ranks: tflops = 6*M*8192*28672 / the best complete-output time; "
                   "weight_stream_gbs = packed weights + scales of the three projections / that time; graph_ms_*: "
                   "the chain replayed from a CUDA graph over weight_sets_cycled distinct weight sets (> 2 x L2); "
                   "ms_fused_all_reduce: the down projection stores its partial tiles into the ranks' staging "
                   "slots (peer memory), then a barrier and the slot sum; ms_fused_pipelined_all_reduce: the same "
                   "with the whole chain in row chunks (gate|up weights dequantised once), each chunk's barrier + "
                   "sum + store-back on a second stream behind the next chunk's launches; "
                   "ms_two_launches_silu_epilogue: gate|up with the SiLU-gate in its epilogue (column-interleaved "
                   "weights), then down; ms_fused_all_reduce_silu_epilogue: the fused all-reduce form on top of it; "
                   "ms_switch_all_reduce: partials stay local, then multimem.ld_reduce + multimem.st through the "
                   "NVSwitch per column block (switch_chunks: rows per pipelined chunk); "
                   "ms_overlapped_all_reduce: weights "
                   "dequantised once, rows in overlap_chunks, each chunk's NCCL all-reduce on a second stream "
                   "behind the next chunk's GEMMs")
    return res, {"checked": checked, "failed": failed}


def _check_chain(torch, dist, ops, np, chain, x, mm, hidden, inter, rank, world, fused_ok, switch_ok, host_weights):
    """Every reduction form of the chain against the stage-wise CPU oracle on two rows (rank 0,
    unsharded weights; bar: 1e-2 of max(|want|, the row's rms)), and the fused form's bits across
    the ranks."""
    outs = {"nccl": None, "fused": None, "overlap": None, "fused_pipelined": None, "fused_silu_epilogue": None,
            "switch": None, "switch_chunked": None}
    part = chain.local(x, mm)
    dist.all_reduce(part, op=dist.ReduceOp.SUM)
    outs["nccl"] = part.clone()
    if fused_ok:
        outs["fused"] = chain.run_fused(x, mm).clone()
    if mm > 512:
        outs["overlap"] = chain.run_overlapped(x, mm).clone()
        if fused_ok and mm > chain.m_one:
            outs["fused_pipelined"] = chain.run_fused_pipelined(x, mm).clone()
    if fused_ok and mm > 512:
        chain.enable_fused_silu()
        outs["fused_silu_epilogue"] = chain.run_fused(x, mm).clone()
        chain.enable_fused_silu(False)
    if switch_ok:
        outs["switch"] = chain.run_switch(x, mm).clone()
        if mm > 512:
            outs["switch_chunked"] = chain.run_switch(x, mm, chunks=[mm // 2, mm - mm // 2]).clone()
    torch.cuda.synchronize()
    why = []
    ok = ops.device_status(chain.device)[0] == 0
    if not ok:
        why.append("device status")
    for name in ("fused", "switch"):  # one reducer per element: every rank holds the same bits
        if outs[name] is None:
            continue
        digest = outs[name].contiguous().view(torch.int32).to(torch.int64).sum().reshape(1)
        all_d = torch.empty(world, dtype=torch.int64, device="cuda")
        dist.all_gather_into_tensor(all_d, digest)
        if not bool((all_d == all_d[0]).all().item()):
            ok = False
            why.append(f"{name} bits differ across ranks")
    if rank == 0:
        from oracle import oracle as orc
        orc.build()
        orc.set_threads(os.cpu_count() or 1)
        wg, sg, wu, su, wd, sd = host_weights
        u32 = lambda t: t.view(np.uint32)
        rows = [0, mm - 1]
        xr = x.view(mm, hidden)[rows].cpu().numpy().reshape(-1)
        gate = orc.matmul_int4(xr, u32(wg), sg, len(rows), inter, hidden, f16_out=True)
        up = orc.matmul_int4(xr, u32(wu), su, len(rows), inter, hidden, f16_out=True)
        act = orc.silu_gate_f16(np.ascontiguousarray(gate).reshape(-1), np.ascontiguousarray(up).reshape(-1),
                                len(rows), inter)
        want = np.asarray(orc.matmul_int4(act.reshape(-1), u32(wd), sd, len(rows), hidden, inter,
                                          f16_out=False)).reshape(len(rows), hidden)
        for name, t in outs.items():
            if t is not None:
                rel = _max_rel_rowscale(np, t.reshape(mm, hidden)[rows].cpu().numpy(), want)
                if not rel < 1e-2:
                    ok = False
                    why.append(f"{name} vs oracle: max rel {rel:.3e}")
    if why:
        print(f"chain parity m={mm} rank {rank}: " + "; ".join(why), file=sys.stderr, flush=True)
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    return bool(flag.item())


if __name__ == "__main__":
    main()
