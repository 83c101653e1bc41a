"""Builds slopfab_b200/libsfq.so (the CUDA kernels + C++ runner + C ABI) in-tree for sm_100a.

    python slopfab_b200/build.py [--force]      (run by path: importing the package needs the library)

nvcc cross-compiles without a GPU. Objects go to slopfab_b200/build/, the library next to this file.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libsfq.so")
SOURCES = ["gemm_tc.cu", "gemm_tc2.cu", "unpack.cu", "act_quant.cu", "quant_int8_pairs.cu", "pointwise.cu", "attention.cu", "runtime.cu", "linear_runner.cu", "capi.cu",
           "capi_runner.cu", "lora_runner.cu", "static_scratch.cu", "packers.cpp", "adaln_index.cpp", "weight_views.cpp", "checkpoint.cpp"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-std=c++17", "-O3", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden,-fopenmp"]


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _headers() -> list[str]:
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    inc = os.path.join(os.path.dirname(HERE), "include")
    hs += [os.path.join(inc, "sfq.h"), os.path.join(inc, "slopfab_b200", "linear.hpp")]
    return hs


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    headers = _headers()
    jobs = []
    for src in SOURCES:
        path = os.path.join(CSRC, src)
        obj = os.path.join(OBJ, os.path.splitext(src)[0] + ".o")
        if force or _stale(obj, [path] + headers):
            cmd = ["nvcc", *COMMON, *ARCH, "-c", path, "-o", obj]
            if src.endswith(".cpp"):
                cmd[1:1] = ["-x", "cu"]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)
        if verbose and (r.stdout or r.stderr):
            print(r.stdout + r.stderr)

    with ThreadPoolExecutor(max_workers=8) as pool:
        list(pool.map(run, jobs))
    objs = [os.path.join(OBJ, os.path.splitext(s)[0] + ".o") for s in SOURCES]
    if force or jobs or _stale(LIB, objs):
        run(["nvcc", "-shared", *ARCH, "-Xcompiler", "-fPIC", "-o", LIB, *objs, "-lgomp"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
