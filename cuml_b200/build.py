"""Build recipe of libb2fil.so: nvcc for sm_100a, in-tree output under cuml_b200/lib/.

`python -m cuml_b200.build [--force] [--verbose]` (also called by `__graft_entry__.build()`).
The register / shared-memory report of ptxas is written to cuml_b200/lib/ptxas.log.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIB_DIR, "libb2fil.so")
SOURCES = ["api.cu", "kernels.cu", "kernels_q_top6.cu", "kernels_q_plain6.cu", "kernels_q_plain4.cu",
           "kernels_q_cat.cu", "kernels_q_generic.cu", "kernels_q_pair.cu", "kernels_q_leafg.cu",
           "kernels_q_vec.cu",
           "kernels_sparse_c.cu",
           "pack.cpp"]
HEADERS = ["forest.hpp", "kernels.hpp", "kernels_q.hpp", "device_common.cuh", "dense_q.cuh",
           os.path.join("..", "..", "include", "b2fil.h")]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libb2fil.so cannot be built")
    return exe


def up_to_date() -> bool:
    if not os.path.exists(LIB):
        return False
    t = os.path.getmtime(LIB)
    deps = [os.path.join(SRC, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return all((not os.path.exists(d)) or os.path.getmtime(d) <= t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and up_to_date():
        return LIB
    if not all(os.path.exists(os.path.join(SRC, s)) for s in SOURCES):
        raise RuntimeError("kernel sources missing; cannot build libb2fil.so")
    os.makedirs(LIB_DIR, exist_ok=True)
    # one nvcc per translation unit, all at once (the kernel families are split over several
    # files for exactly this), then one link step
    obj_dir = os.path.join(LIB_DIR, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    base = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
            "-Xcompiler", "-fPIC,-Wall", "-Xptxas", "-v"]
    jobs = []
    for src in SOURCES:
        obj = os.path.join(obj_dir, os.path.splitext(src)[0] + ".o")
        cmd = base + ["-c", os.path.join(SRC, src), "-o", obj]
        out = open(obj + ".log", "w+")  # a file, not a pipe: nothing blocks while others run
        jobs.append((cmd, obj, subprocess.Popen(cmd, stdout=out, stderr=subprocess.STDOUT), out))
    log, failed = [], False
    for cmd, obj, proc, out in jobs:
        proc.wait()
        out.seek(0)
        log.append(" ".join(cmd) + "\n" + out.read())
        out.close()
        failed |= proc.returncode != 0
    if not failed:
        cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIB]
        cmd += [obj for _, obj, _, _ in jobs]
        proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        log.append(" ".join(cmd) + "\n" + proc.stdout)
        failed = proc.returncode != 0
    text = "\n".join(log)
    with open(os.path.join(LIB_DIR, "ptxas.log"), "w") as fh:
        fh.write(text)
    if failed:
        sys.stderr.write(text)
        raise RuntimeError("nvcc failed building libb2fil.so")
    if verbose:
        print(text)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
