"""Builds libbf_b200.so (sm_100a) in-tree with nvcc.

    python -m boundflow_b200.csrc.build [--verbose]

The library is a plain C-ABI shared object (no torch, no Python in it); the
Python package loads it with ctypes.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SOURCES = ["chain.cu", "chain_alpha.cu", "crown_linear.cu", "crown_tc.cu", "crown_tc_persist.cu", "crown_tc_adj.cu", "ibp.cu", "elementwise.cu", "conv.cu", "certificate.cu"]
HEADERS = ["common.cuh", "kernels.cuh", "gemm_ffma.cuh", "chain_internal.cuh", "tc_primitives.cuh", os.path.join("..", "..", "include", "bf_b200.h")]
LIB = os.path.join(os.path.dirname(HERE), "libbf_b200.so")


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(os.path.join(HERE, f)) > t for f in SOURCES + HEADERS)


def build(verbose: bool = False, force: bool = False) -> str:
    if not force and not needs_build():
        return LIB
    cmd = [
        _nvcc(), "-shared", "-Xcompiler", "-fPIC", "-O3", "-std=c++17", "-lineinfo",
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-o", LIB,
    ] + [os.path.join(HERE, f) for f in SOURCES]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed building libbf_b200.so")
    return LIB


if __name__ == "__main__":
    print(build(verbose="--verbose" in sys.argv, force=True))
