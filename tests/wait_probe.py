"""Builds ``tests/libpalimpsa_wait_probe.so`` from ``tests/wait_probe.cu`` (test-only; see the source)."""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "wait_probe.cu")
LIB = os.path.join(HERE, "libpalimpsa_wait_probe.so")


def build(force: bool = False) -> str:
    deps = [SRC, os.path.join(os.path.dirname(HERE), "palimpsa_b200", "csrc", "tc_common.cuh")]
    if not force and os.path.exists(LIB) and all(os.path.getmtime(LIB) >= os.path.getmtime(d) for d in deps):
        return LIB
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    cmd = [nvcc if os.path.exists(nvcc) else "nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3",
           "-std=c++17", "-Xcompiler", "-fPIC", "-shared", SRC, "-o", LIB]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on wait_probe.cu:\n{r.stdout}\n{r.stderr}")
    return LIB
