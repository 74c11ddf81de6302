"""Builds ``libb200q.so`` (the C-ABI shared library) in-tree with nvcc for sm_100a.

Run as ``python -m mlfw_b200.build`` or call :func:`build`.  nvcc cross-compiles
without a GPU, so this also works on a machine that has none.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libb200q.so")
SOURCES = ["api.cu", "quant_kernels.cu", "gemm_simt.cu", "gemm_umma.cu", "block_kernels.cu", "attention_umma.cu", "noalloc.cu", "group.cu", "conv_group.cu", "host_stage.cu"]
HEADERS = ["common.cuh", "kernels.cuh", "quant_math.cuh", "exp2_table.inc", "exp_ff_table.inc", os.path.join("..", "..", "include", "b200q.h")]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: libb200q.so cannot be built")


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every CUDA source for sm_100a and link ``libb200q.so``; returns its path."""
    if not force and not _stale():
        return LIB
    cmd = [
        _nvcc(), "-shared", "-o", LIB + ".tmp",
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-O3", "-lineinfo", "-std=c++17",
        "-Xcompiler", "-fPIC,-O2,-Wall",
        "-ccbin", "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++",
        "--fmad=false",  # the reference rounds after every operation; contraction must be explicit (fma())
    ]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(CSRC, s) for s in SOURCES]
    cmd += ["-ldl"]   # group.cu looks NCCL up at run time (dlopen), so the library itself does not depend on it
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    os.replace(LIB + ".tmp", LIB)  # a failed build leaves the previous library in place
    if verbose:
        print(res.stdout + res.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force=True, verbose="-v" in sys.argv))
