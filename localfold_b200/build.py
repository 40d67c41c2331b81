"""Builds ``lib/liblocalfold_pairstack.so`` from ``csrc/`` with nvcc for sm_100a.

    python -m localfold_b200.build [--force]

The library is built in-tree; nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "lib", "liblocalfold_pairstack.so")
SOURCES = ("api.cu", "tc_kernels.cu", "tc_ln_gemm.cu", "tc_attention.cu", "tc_transition.cu", "static_scratch.cu", "peer_transpose.cu", "pair_spill.cu")
NVCC_FLAGS = (
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "-shared",
)


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    built = os.path.getmtime(LIB)
    inputs = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    inputs.append(os.path.join(os.path.dirname(HERE), "include", "localfold_pairstack.h"))
    return any(os.path.getmtime(p) > built for p in inputs)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return LIB
    os.makedirs(os.path.dirname(LIB), exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, *NVCC_FLAGS, "-o", LIB, *[os.path.join(CSRC, s) for s in SOURCES], "-lcudart", "-lcuda"]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    result = subprocess.run(cmd, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + result.stdout + result.stderr)
    if verbose:
        print(result.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
