"""Builds libpcb200.so (hand-written CUDA for sm_100a behind the C ABI of include/pcb200.h)
in-tree with nvcc.  `python -m lvd_pg_b200.build [--force] [--verbose]`."""
from __future__ import annotations

import os
import shlex
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libpcb200.so")
SOURCES = ["pcb_compile.cu", "pcb_em.cu", "pcb_dense.cu", "pcb_dense_tc.cu", "pcb_dense_mn.cu", "pcb_dense_edge.cu", "pcb_kld.cu", "pcb_sample.cu", "pcb_comm.cu", "pcb_persample.cu", "pcb_mi.cu", "pcb_selftest.cu"]
NVCC = os.environ.get("PCB_NVCC", "/usr/local/cuda/bin/nvcc")
EXTRA = shlex.split(os.environ.get("PCB_NVCC_FLAGS", ""))   # e.g. -DPCB_DIAG for the timing-experiment build
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
         "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall"]


def _deps():
    files = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    inc = os.path.join(HERE, "..", "include")
    files += [os.path.join(inc, f) for f in os.listdir(inc)]
    return files


def build(force: bool = False, verbose: bool = False) -> str:
    stale = not os.path.exists(LIB) or any(os.path.getmtime(f) > os.path.getmtime(LIB) for f in _deps())
    if not (force or stale):
        return LIB
    headers = [f for f in _deps() if f.endswith((".h", ".cuh"))]

    def compile_one(src):
        path, obj = os.path.join(CSRC, src), os.path.join(CSRC, src.replace(".cu", ".o"))
        fresh = os.path.exists(obj) and all(os.path.getmtime(f) <= os.path.getmtime(obj) for f in [path] + headers)
        if fresh and not (force or verbose):
            return obj
        cmd = [NVCC] + FLAGS + EXTRA + (["-Xptxas", "-v"] if verbose else []) + ["-c", path, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode != 0:
            sys.stderr.write("== " + src + "\n" + r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed on " + src)
        return obj

    with ThreadPoolExecutor(max_workers=min(len(SOURCES), os.cpu_count() or 1)) as pool:   # one nvcc per source
        objs = list(pool.map(compile_one, SOURCES))
    cmd = [NVCC, "-shared", "-o", LIB] + objs + ["-lcudart", "-ldl"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
