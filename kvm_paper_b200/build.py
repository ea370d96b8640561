"""Build libkvm_b200.so (the C-ABI library with the sm_100a kernels) in-tree with nvcc.

    python -m kvm_paper_b200.build [--force] [--verbose]

The library lands next to this file so that it travels with the source tree; nothing is installed.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libkvm_b200.so")
SOURCES = ["kvm_abi.cu", "kvm_prefill.cu", "kvm_chain_tc.cu", "kvm_vpass.cu", "kvm_attn_tc.cu", "kvm_decode.cu", "kvm_prologue.cu"]
HEADERS = ["kvm_common.cuh", "kvm_update.cuh", "kvm_tc.cuh", "kvm_tma_host.cuh", "kvm_vdelta.cuh", os.path.join("..", "..", "include", "kvm_b200.h")]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or add it to PATH")


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS]
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every .cu of the package for sm_100a into one shared library; returns its path."""
    if not force and not _stale():
        return LIB
    cmd = [
        _nvcc(), "-shared", "-o", LIB,
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-O3", "-std=c++17", "-lineinfo",
        "-Xcompiler", "-fPIC", "-Xcompiler", "-O2",
        "--threads", "0",
    ]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(CSRC, s) for s in SOURCES]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stdout + res.stderr)
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
