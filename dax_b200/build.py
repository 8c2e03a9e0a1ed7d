"""Builds ``libdax_b200.so`` (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

The library is compiled next to its sources (``dax_b200/lib/``) so that it travels with the
source tree; nothing is installed into site-packages and nothing is JIT-compiled at import time.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
LIBNAME = "libdax_b200.so"

SOURCES = ["capi.cu", "quant.cu", "gemm.cu", "linear.cu", "rope_pack.cu", "dit_block.cu", "attn_prep.cu", "attn.cu", "attn_tmem.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
    "--fmad=true",  # contraction stays on for plain a*b+c; the bit-exact paths use __fmul_rn/__fadd_rn
]


def nvcc_path() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found: the dax_b200 CUDA library cannot be built")
    return cand


def library_path() -> str:
    return os.path.join(LIBDIR, LIBNAME)


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile every translation unit and link the shared library.  Returns its path."""
    os.makedirs(LIBDIR, exist_ok=True)
    nvcc = nvcc_path()
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(HERE, "..", "include", "dax_b200.h"))
    objs = []
    jobs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(LIBDIR, src.replace(".cu", ".o"))
        objs.append(o)
        if force or _stale(o, [s] + headers):
            jobs.append((s, o))

    def compile_one(job):
        s, o = job
        cmd = [nvcc] + NVCC_FLAGS + ["-c", s, "-o", o]
        r = subprocess.run(cmd, capture_output=True, text=True)
        return s, r

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for s, r in ex.map(compile_one, jobs):
            if verbose or r.returncode != 0:
                sys.stderr.write(r.stdout + r.stderr)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {s}")
            with open(os.path.join(LIBDIR, os.path.basename(s) + ".ptxas.log"), "w") as f:
                f.write(r.stderr)
    lib = library_path()
    if force or jobs or _stale(lib, objs):
        cmd = [nvcc, "-shared", "-cudart", "static", "-o", lib] + objs
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("linking libdax_b200.so failed")
    return lib


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose=True))
