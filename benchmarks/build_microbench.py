"""Builds ``benchmarks/libpalimpsa_microbench.so``: register-resident micro-benchmarks of the FP32 FMA and MUFU
reciprocal pipes, which ``bench.py`` runs to measure the compute ceilings of the GPU it is on.  A measurement
tool beside the benchmark, not part of the operator library or its C ABI.

    python benchmarks/build_microbench.py
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "microbench.cu")
LIB = os.path.join(HERE, "libpalimpsa_microbench.so")


def build(force: bool = False) -> str:
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    cmd = [nvcc if os.path.exists(nvcc) else "nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3",
           "-std=c++17", "-Xcompiler", "-fPIC", "-shared", SRC, "-o", LIB]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on microbench.cu:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print("built", build(force="--force" in sys.argv))
