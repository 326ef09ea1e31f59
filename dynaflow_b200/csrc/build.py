"""Builds the C-ABI shared library in-tree with nvcc for sm_100a.

    python -m dynaflow_b200.csrc.build [--force] [--dev-knobs]

``--dev-knobs`` compiles with ``-DDF_DEV_KNOBS``: the GEMM launches then read their tuning
integers (tile grouping, pipeline depth, CTA pairs, and switches that skip the operand copies or
the output stores for timing diagnostics, which make the results invalid) from ``DF_GEMM_*``
environment variables. The default build has none of them.

The result is ``dynaflow_b200/lib/libdynaflow_b200.so``; it links against the
CUDA runtime only (the one driver entry point it needs is resolved at run time).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

CSRC = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(CSRC)
LIB_DIR = os.path.join(PKG, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libdynaflow_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
    "--cudart", "shared",
]


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _newest_input() -> float:
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh", ".h"))]
    deps.append(os.path.join(os.path.dirname(PKG), "include", "dynaflow_b200.h"))
    return max(os.path.getmtime(p) for p in deps if os.path.exists(p))


def find_nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; the dynaflow_b200 kernels cannot be built")
    return nvcc


def build(force: bool = False, verbose: bool = False, dev_knobs: bool = False) -> str:
    """Compiles the library if it is missing or older than its sources; returns its path."""
    if not force and os.path.exists(LIB_PATH) and os.path.getmtime(LIB_PATH) >= _newest_input():
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    cmd = [find_nvcc(), *NVCC_FLAGS]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    if dev_knobs:
        cmd += ["-DDF_DEV_KNOBS"]
    cmd += ["-o", LIB_PATH, *sources()]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    if verbose:
        print(proc.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv or "--dev-knobs" in sys.argv, verbose="-v" in sys.argv,
                dev_knobs="--dev-knobs" in sys.argv))
