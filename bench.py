#!/usr/bin/env python
"""Benchmark of the quantized-inference hot path on B200.

One "step" = one pass of the W8A8 prefill GEMMs at the Llama-7B shapes
(M=4096; (K,N) = (4096,11008), (11008,4096), (4096,4096)), int8 x int8 -> s32, per-row
activation scale x per-column weight scale, f32 output.  `value` is whole-job W8A8 TOPS
(2*M*N*K summed over the three GEMMs and over the ranks / device time, max over ranks).  The
7B-shape weights fit one GPU, so with --gpus N > 1 every rank is a replica working on its own
M rows (weak scaling, no collective).  The sharded path -- the Llama-70B-shape W4A16 FFN GEMMs,
weights column-sharded N/P per rank, f16 output all-gathered over NCCL -- is measured at every N in
the "ffn70b_w4a16" object (GEMM alone and GEMM + gather).

The same JSON line also carries
  * "w4a16_decode": the W4A16 decode GEMM (M in {1,8,16}, K=4096, N=11008) in HBM GB/s,
  * "roofline" of the dominant kernel, "cpu_baseline" (the CPU oracle on the host cores, a
    bounded row sample), "e2e" (same step through the public API from pinned host buffers),
    "clocks" sampled with nvidia-smi during the timed region and "gpu_launches".

`--impl reference` times the reference's own CPU implementation of the path (the oracle is the
restatement of the CPU reference functions the KAIO tests hold; the Rust crate itself cannot be
built here) on the host cores, on a bounded row sample of the same GEMMs.
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
                self.samples.append((float(sm), pw, int(rs)))
            except Exception as exc:
                self.err = repr(exc)
                return
            time.sleep(0.002)

    def start(self):
        if self.handle is None:
            return
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()

    def stop(self):
        if self.thread is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [f"NVML unavailable: {self.err}"]}
        self.stop_flag = True
        self.thread.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": [f"no samples: {self.err}"]}
        reasons = set()
        for _, _, rs in self.samples:
            for name, bit in self.REASONS.items():
                if rs & bit:
                    reasons.add(name)
        # median clock over the samples taken under load (upper half of the power readings)
        order = sorted(self.samples, key=lambda t: t[1])
        loaded = sorted(t[0] for t in order[len(order) // 2:])
        return {"sm_mhz": loaded[len(loaded) // 2], "sm_max_mhz": self.sm_max, "reasons": sorted(reasons),
                "samples": len(self.samples), "power_w_max": max(t[1] for t in self.samples),
                "source": "NVML, 2 ms period, during the timed loop"}


# ------------------------------------------------------------------------------ reference arm

def cpu_int8_sample(rows_per_gemm: int, seed: int = 42):
    """The CPU oracle on `rows_per_gemm` rows of each 7B GEMM; returns (ops, seconds, threads)."""
    import numpy as np

    from oracle import oracle as orc
    orc.build()
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
    ap.add_argument("--graphs", action="store_true",
                    help="with --ffn-chain-only: also time the M <= 256 chains replayed from CUDA graphs "
                         "(device time without the Python launch overhead)")
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
    if args.decode_only:
        print(json.dumps({"w4a16_decode": bench_decode(torch, ops, dev, peaks, load_traffic())}), flush=True)
        return
    if args.qkv_attention_only:
        print(json.dumps({"qkv_attention": bench_qkv_attention(torch, ops, dev, peaks)}), flush=True)
        return
    if args.ffn70b_only:
        res = bench_ffn70b(torch, dist, ops, sharding, dev, rank, world)
        if rank == 0:
            print(json.dumps({"ffn70b_w4a16": res}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    if args.ffn_chain_only:
        res = bench_ffn_chain(torch, dist, ops, dev, rank, world, peaks, graphs=args.graphs)
        if rank == 0:
            print(json.dumps({"ffn_chain_70b_w4a16": res}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- synthetic inputs (seeded; config 3 value ranges), resident in HBM
    g = torch.Generator(device="cuda")
    g.manual_seed(42)
    probs = []
    # The 7B-shape weights fit every GPU, so with N > 1 each rank is a replica that runs the same
    # GEMMs on its own batch of M rows (own activations, same weights): weak scaling, no collective.
    for gi, (k, n) in enumerate(GEMMS_7B):
        n_loc = n
        g.manual_seed(42 + gi + 1000 * rank)
        a = torch.randint(-127, 128, (m * k,), dtype=torch.int8, device="cuda", generator=g)
        g.manual_seed(137 + gi)
        b = torch.randint(-127, 128, (k * n_loc,), dtype=torch.int8, device="cuda", generator=g)
        g.manual_seed(4242 + gi + 1000 * rank)
        sa = torch.rand(m, device="cuda", generator=g) * 0.009 + 0.001
        g.manual_seed(4243 + gi)
        sw = torch.rand(n_loc, device="cuda", generator=g) * 0.009 + 0.001
        c_loc = torch.empty(m * n_loc, dtype=torch.float32, device="cuda")
        probs.append(dict(k=k, n=n, n_loc=n_loc, a=a, b=b, sa=sa, sw=sw, c=c_loc))
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device="cuda")
    total_ops = world * sum(2 * m * n * k for k, n in GEMMS_7B)

    def gemm(p):
        ops.matmul_int8_scaled(dev, p["a"], p["b"], p["c"], p["sa"], p["sw"], m, p["n_loc"], p["k"])

    def step():
        for p in probs:
            gemm(p)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        flush.zero_()
        step()
    barrier()
    assert ops.device_status(dev)[0] == 0

    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.3)
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
    t_wall = time.perf_counter() - t_wall0
    clocks = sampler.stop()
    step_ms = [e[0].elapsed_time(e[-1]) for e in evs]
    gemm_ms = [[e[i].elapsed_time(e[i + 1]) for e in evs] for i in range(len(probs))]
    total_ms = sum(step_ms)
    if world > 1:
        t = torch.tensor([total_ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    value = total_ops / (ms_per_step * 1e-3) / 1e12

    ffn = chain = decode = qkv_attn = None
    if not args.skip_extras:
        for p in probs:  # free the headline buffers before the other legs
            p.clear()
        torch.cuda.empty_cache()
        if world == 1:
            # The latency-sensitive decode leg runs before the legs that allocate and free gigabytes:
            # after them the same kernel on freshly allocated buffers measures 10-40 % slower (18 us
            # alone or straight after the headline, 20-27 us after the 70B-shape legs).
            decode = bench_decode(torch, ops, dev, peaks, load_traffic())
            qkv_attn = bench_qkv_attention(torch, ops, dev, peaks)
            torch.cuda.empty_cache()
        ffn = bench_ffn70b(torch, dist, ops, sharding, dev, rank, world)
        torch.cuda.empty_cache()
        chain = bench_ffn_chain(torch, dist, ops, dev, rank, world, peaks)
        torch.cuda.empty_cache()

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel (w8a8_gemm_kernel), N=1 semantics: per-launch ops / duration
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
        "bound": "tensor", "kernel": "w8a8_gemm_kernel", "achieved": achieved, "peak": int8_peak,
        "unit": "TOPS", "frac": achieved / int8_peak,
        "peak_source": f"2 x {peaks['source']} dense bf16 burst ({peaks['bf16_tflops']} TF/s); INT8 peak itself is not in MEASURED_PEAKS.json; nominal dense INT8 is 4500 TOPS",
        "frac_of_nominal_4500": achieved / 4500.0,
        "traffic": traffic.get("w8a8_gemm_kernel_bytes_per_step"),
        "per_gemm": per_gemm,
        "timing": "CUDA events around each GEMM launch on rank 0",
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
                   "70B-shape FFN with its NCCL all-gather is in ffn70b_w4a16",
                   "l2": f"{L2_FLUSH_BYTES >> 20} MiB memset between timed steps (untimed)",
                   "wall_s_timed_loop": t_wall},
        "roofline": roofline, "clocks": clocks, "gpu_launches": len(probs) * args.steps,
    }

    if ffn is not None:
        line["ffn70b_w4a16"] = ffn
    if chain is not None:
        line["ffn_chain_70b_w4a16"] = chain
    if not args.skip_extras and world == 1:
        line["w4a16_decode"] = decode
        line["qkv_attention"] = qkv_attn
        line["e2e"] = bench_e2e(torch, ops, dev, m, total_ops, steps=max(3, min(args.steps, 10)))
        rows = m  # the whole step on the host cores: about 10 s with 16 threads
        o, s, threads = cpu_int8_sample(rows)
        line["cpu_baseline"] = {
            "value": o / s / 1e12, "unit": "TOPS", "cores": threads, "kind": "port",
            "sample": f"{rows} of {m} rows of each of the three GEMMs (all columns, full K), CPU oracle, {s:.1f} s"}
    elif world > 1:
        line["e2e"] = None
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


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


def bench_e2e(torch, ops, dev, m, total_ops, steps):
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
    t0 = time.perf_counter()
    for i in range(steps):
        one(i)
    torch.cuda.synchronize()
    dt = (time.perf_counter() - t0) / steps
    return {"value": total_ops / dt / 1e12, "unit": "TOPS", "ms_per_step": dt * 1e3,
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "note": "int8 activations H2D and f32 outputs D2H every step from/to pinned memory, copies "
                    "and GEMMs on three streams; bound by the PCIe download of the f32 outputs"}


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


def bench_ffn70b(torch, dist, ops, sharding, dev, rank, world):
    """Config 5: Llama-70B-shape W4A16 FFN GEMMs, N-sharded over the ranks, f16 output all-gathered
    to [M, N] on every rank.  Times are CUDA events, max over ranks.  Reported: the GEMM alone, the
    GEMM followed by the NCCL gather, the pipelined form (the shard is computed in column panels and
    panel i is gathered on a second stream while panel i+1 is computed), and the fused form (one
    kernel whose epilogue stores each tile into every rank's buffer over peer memory, followed by
    a symmetric-memory barrier)."""
    res = {}
    g = torch.Generator(device="cuda")
    comm_stream = torch.cuda.Stream()
    for (k, n) in [(8192, 28672), (28672, 8192)]:
        n_loc = n // world
        g.manual_seed(137 + rank)
        w = torch.randint(-2 ** 31, 2 ** 31 - 1, (k // 8 * n_loc,), dtype=torch.int32, device="cuda", generator=g)
        sc = (torch.rand(k // 128 * n_loc, device="cuda", generator=g) * 0.015 + 0.005).half()
        for mm in (16, 256, 4096):
            g.manual_seed(42)
            a = torch.randn(mm * k, device="cuda", generator=g).half()
            c = torch.empty(mm * n_loc, dtype=torch.float16, device="cuda")
            gather = sharding.ColumnGather(mm, n, torch.float16, "cuda") if world > 1 else None

            def gemm():
                ops.matmul_int4(dev, a, w, sc, c, mm, n_loc, k, 128)

            def both():
                gemm()
                if gather is not None:
                    gather(c)

            iters = 20 if mm <= 256 else 5
            t_gemm = _time_ms(torch, gemm, iters)
            t_all = _time_ms(torch, both, iters) if world > 1 else t_gemm
            t_pipe = t_fused = t_all
            if world > 1 and mm >= 256:
                pipe = sharding.PanelPipeline(ops, dev, a, w, sc, mm, n, k, world, rank, comm_stream, panels=4)
                t_pipe = _time_ms(torch, pipe.run, iters)
                del pipe
            if world > 1:
                # one kernel per rank: the epilogue stores into every rank's buffer (peer memory)
                fused = sharding.FusedGatherGemm(ops, dev, mm, n, k, world, rank)
                t_fused = _time_ms(torch, lambda: fused.run(a, w, sc), iters)
                del fused
            t = torch.tensor([t_gemm, t_all, t_pipe, t_fused], dtype=torch.float64, device="cuda")
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            t_gemm, t_all, t_pipe, t_fused = float(t[0]), float(t[1]), float(t[2]), float(t[3])
            best = min(t_all, t_pipe, t_fused)
            flops = 2 * mm * n * k
            nbytes = k * n // 2 + (k // 128) * n * 2 + 2 * mm * k + 2 * mm * n
            res[f"k{k}_n{n}_m{mm}"] = {
                "ms_gemm": t_gemm, "ms_gemm_plus_gather": t_all, "ms_pipelined": t_pipe,
                "ms_fused_peer_store": t_fused,
                "tflops": flops / best / 1e9, "weight_stream_gbs": nbytes / best / 1e6,
                "variant": ops.last_variant()}
            del a, c, gather
        del w, sc
        torch.cuda.empty_cache()
    res["note"] = ("whole-job figures over all ranks (tflops / weight_stream_gbs use the better of the sequential "
                   "and the pipelined time); weight_stream_gbs = algorithmic bytes of the full GEMM / time; the "
                   "L2 is not flushed between iterations (117 MB of weights per GEMM at 1 GPU, 126 MB L2: treat "
                   "the 1-GPU decode figures as an upper bound)")
    return res


def _graph_ms(torch, fn, reps=2, replays=20):
    """`fn` called `reps` times, captured into one CUDA graph; ms per call when the graph is replayed."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(reps):
            fn()
    return _time_ms(torch, graph.replay, replays) / reps


def bench_ffn_chain(torch, dist, ops, dev, rank, world, peaks, graphs=False):
    """The W4A16 feed-forward chain at Llama-70B shapes (hidden 8192, intermediate 28672):
    gate|up projection (one GEMM), SiLU-gate, down projection; across ranks column-parallel then
    row-parallel, so the only exchange is the sum of the [M, 8192] f32 partial outputs.  CUDA
    events, max over ranks.  Reported per M: the three launches alone (and each on its own), and
    the chain with its NCCL all-reduce / reduce-scatter."""
    from kaio_b200 import ffn as ffn_mod
    hidden, inter = 8192, 28672
    g = torch.Generator(device="cuda")
    g.manual_seed(137)

    def packed(k, n):
        return torch.randint(-2 ** 31, 2 ** 31 - 1, (k // 8 * n,), dtype=torch.int32, device="cuda", generator=g)

    def scales(k, n):
        return (torch.rand(k // 128 * n, device="cuda", generator=g) * 0.015 + 0.005).half()

    weights = [packed(hidden, inter), scales(hidden, inter), packed(hidden, inter), scales(hidden, inter),
               packed(inter, hidden), scales(inter, hidden)]
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
    del weights
    torch.cuda.empty_cache()
    il = chain.i_loc
    res = {}
    for mm in (16, 256, 4096):
        g.manual_seed(42)
        x = (torch.randn(mm * hidden, device="cuda", generator=g)).half()
        iters = 20 if mm <= 256 else 5

        def gate_up():
            ops.matmul_int4(dev, x, chain.w_gu, chain.s_gu, chain.gu, mm, 2 * il, hidden, 128)

        def act():
            ops.silu_gate_f16(dev, chain.gu, chain.gu.view(-1)[il:], chain.act, mm, il, x_ld=2 * il, gate_ld=2 * il)

        def down():
            ops.matmul_int4(dev, chain.act, chain.w_down, chain.s_down, chain.out, mm, hidden, il, 128)

        def local():
            chain.local(x, mm)

        def with_all_reduce():
            dist.all_reduce(chain.local(x, mm), op=dist.ReduceOp.SUM)

        def with_reduce_scatter():
            dist.reduce_scatter_tensor(scatter_rows[: (mm // world) * hidden], chain.local(x, mm).view(-1),
                                       op=dist.ReduceOp.SUM)

        local()
        variant_gu = None
        gate_up()
        variant_gu = ops.last_variant()
        down()
        variant_down = ops.last_variant()
        ts = [_time_ms(torch, f, iters) for f in (gate_up, act, down, local)]
        if world > 1:
            # the three reductions, timed in two rounds in opposite order (the GPU sits at its power
            # cap at M = 4096, so whatever is timed last would otherwise look slowest); min of the two
            forms = [with_all_reduce, with_reduce_scatter if mm % world == 0 else with_all_reduce,
                     (lambda: chain.run_fused(x, mm)) if fused_ok else with_all_reduce]
            first = [_time_ms(torch, f, iters) for f in forms]
            second = [_time_ms(torch, f, iters) for f in reversed(forms)][::-1]
            ts += [min(a, b) for a, b in zip(first, second)]
        else:
            ts += [ts[3]] * 3
        if graphs and mm <= 256:
            # two calls per graph: the one-step fused form alternates between two staging buffers
            tg = [_graph_ms(torch, local)]
            tg += [_graph_ms(torch, with_all_reduce),
                   _graph_ms(torch, lambda: chain.run_fused(x, mm)) if fused_ok else 0.0] if world > 1 else [tg[0], tg[0]]
        else:
            tg = [0.0, 0.0, 0.0]
        t = torch.tensor(ts + tg, dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        t_gu, t_act, t_down, t_local, t_ar, t_rs, t_fused, tg_local, tg_ar, tg_fused = [float(v) for v in t]
        t_best = min(t_ar, t_fused)
        flops = 2 * mm * hidden * inter * 3
        wbytes = 3 * (hidden * inter // 2 + (hidden // 128) * inter * 2)
        act_bytes = 3 * mm * il * 2  # the SiLU-gate pass of one rank: two f16 reads and one f16 write per element
        res[f"m{mm}"] = {
            "ms_gate_up_gemm": t_gu, "ms_silu_gate": t_act, "ms_down_gemm": t_down, "ms_three_launches": t_local,
            "ms_with_all_reduce": t_ar, "ms_with_reduce_scatter": t_rs, "ms_fused_all_reduce": t_fused,
            "fused_form": "-" if not fused_ok else ("one step" if mm <= chain.m_one else "two steps"),
            "tflops": flops / t_best / 1e9, "weight_stream_gbs": wbytes / t_best / 1e6,
            "silu_gate_gbs": act_bytes / t_act / 1e6, "silu_gate_frac_of_hbm_peak": act_bytes / t_act / 1e6 / peaks["hbm_gbs"],
            "variants": [variant_gu, "silu_gate_f16", variant_down]}
        if graphs and mm <= 256:
            res[f"m{mm}"]["cuda_graph_replay_ms"] = {"three_launches": tg_local, "with_all_reduce": tg_ar,
                                                    "fused_all_reduce": tg_fused}
        del x
    res["note"] = ("whole-job figures over all ranks: tflops = 6*M*8192*28672 / the better of the NCCL and the fused "
                   "all-reduce time; weight_stream_gbs = packed weights + scales of the three projections / that "
                   "time; ms_fused_all_reduce: the down projection stores its partial tiles into the ranks' "
                   "staging slots (peer memory), then a barrier and the slot sum; "
                   "silu_gate_gbs is one rank's pass (6 bytes per element of its [M, 28672/P] shard); the L2 "
                   "is not flushed between iterations")
    return res


if __name__ == "__main__":
    main()
