"""Builds libquantforge_rt.so (CUDA kernels + C ABI) for sm_100a with nvcc, in-tree.

    python -m quantforge_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  The shared library lands in quantforge_b200/lib/.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libquantforge_rt.so")

SOURCES = ["qf_api.cu", "qf_unpack.cu", "qf_gemv.cu", "qf_gemv_slab.cu", "qf_gemm_tcgen05.cu", "qf_comm.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(ROOT, "include", "quantforge_rt.h"),
                                                                os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    objs = []
    procs = []
    for src in SOURCES:
        obj = os.path.join(LIB_DIR, src.replace(".cu", ".o"))
        cmd = [_nvcc(), *NVCC_FLAGS, "-I", os.path.join(ROOT, "include"), "-I", CSRC, "-c",
               os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
            print(" ".join(cmd), flush=True)
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    failed = False
    for src, pr in procs:
        out, _ = pr.communicate()
        if pr.returncode != 0 or verbose:
            print(f"--- {src}\n{out}", flush=True)
        failed |= pr.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    link = [_nvcc(), "-shared", "-o", LIB_PATH, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
            "-Xcompiler", "-fPIC", "-lcudart_static", "-ldl", "-lpthread", "-lrt"]
    subprocess.run(link, check=True)
    return LIB_PATH


OPT_SRC = os.path.join(HERE, "opt", "quantforge_opt.cpp")
OPT_BIN = os.path.join(HERE, "bin", "quantforge-opt")


def build_opt(force: bool = False) -> str:
    """Builds the re-hosted quantforge-opt driver (plain C++17, no MLIR dependency)."""
    if not force and os.path.exists(OPT_BIN) and os.path.getmtime(OPT_BIN) >= os.path.getmtime(OPT_SRC):
        return OPT_BIN
    os.makedirs(os.path.dirname(OPT_BIN), exist_ok=True)
    subprocess.run(["g++", "-O2", "-std=c++17", "-Wall", "-o", OPT_BIN, OPT_SRC], check=True)
    return OPT_BIN


if __name__ == "__main__":
    print(build_opt(force="--force" in sys.argv))
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
