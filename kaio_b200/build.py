"""Builds ``libkaio_b200.so`` (sm_100a) in place with nvcc.

Run as ``python -m kaio_b200.build`` or through ``__graft_entry__.build()``.  nvcc
cross-compiles without a GPU.  Each ``csrc/*.cu`` is compiled to an object in parallel and
linked into ``kaio_b200/lib/libkaio_b200.so``; the CUDA runtime is linked statically and the
driver API is reached through the runtime's entry-point lookup, so the library loads on a
machine without ``libcuda.so`` (where every op then reports a CUDA error).
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
OBJ_DIR = os.path.join(HERE, "build")
LIB = os.path.join(LIB_DIR, "libkaio_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr",
    "-Xptxas", "-v", "-Xptxas", "-warn-spills",
]


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: cannot build libkaio_b200.so")


def _newest_header_mtime() -> float:
    hdrs = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h"))
    hdrs += glob.glob(os.path.join(os.path.dirname(HERE), "include", "*.h"))
    return max(os.path.getmtime(h) for h in hdrs)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(LIB_DIR, exist_ok=True)
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = _nvcc()
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    hdr_m = _newest_header_mtime()
    jobs = []
    for src in srcs:
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
        stale = force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hdr_m)
        jobs.append((src, obj, stale))

    def compile_one(job):
        src, obj, stale = job
        if not stale:
            return src, ""
        extra = os.environ.get("KAIO_B200_NVCC_EXTRA", "").split()
        r = subprocess.run([nvcc, *NVCC_FLAGS, *extra, "-c", src, "-o", obj], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        return src, r.stderr

    with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
        logs = list(ex.map(compile_one, jobs))
    usage = os.path.join(OBJ_DIR, "resource_usage.txt")
    with open(usage, "a" if not force else "w") as f:
        for src, log in logs:
            if log:
                f.write(f"==== {os.path.basename(src)}\n{log}\n")
                if verbose:
                    print(log)
    objs = [j[1] for j in jobs]
    if force or any(j[2] for j in jobs) or not os.path.exists(LIB):
        r = subprocess.run([nvcc, "-shared", "-o", LIB, *objs, "-cudart", "static", "-ldl",
                            "-gencode", "arch=compute_100a,code=sm_100a"], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
