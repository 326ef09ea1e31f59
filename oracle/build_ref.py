"""Compiles the one piece of the reference that is native code for this path, from the sources
where they lie in the reference tree, into ``oracle/_ref/`` (git-ignored; nothing is copied):

    examples/ae/up-silu-overlap.cu  ->  oracle/_ref/up_silu

the reference's own sm_100a kernel for the gate/up GEMM with a co-resident SiLU (tcgen05 through
CuTe atoms on zeroed shared-memory operands: a tensor-throughput probe without loads or an
epilogue). It is the bar the fused gate/up kernel of this library is compared with on the same
GPU (``profiles/``), nothing links against it.

    python oracle/build_ref.py [/path/to/reference]

Needs nvcc and a CUTLASS/CuTe header tree (the one vendored with the flashinfer package).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")


def cutlass_include() -> str | None:
    try:
        import flashinfer
    except ImportError:
        return None
    inc = os.path.join(os.path.dirname(flashinfer.__file__), "data", "cutlass", "include")
    return inc if os.path.isdir(os.path.join(inc, "cute")) else None


def build(reference: str) -> str | None:
    """Returns the path of the built binary, or None (with the reason printed) if it cannot be built."""
    src = os.path.join(reference, "examples", "ae", "up-silu-overlap.cu")
    if not os.path.exists(src):
        print(f"[build_ref] {src} not found: nothing built")
        return None
    inc = cutlass_include()
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if inc is None or not os.path.exists(nvcc):
        print("[build_ref] no CuTe headers or no nvcc: nothing built")
        return None
    os.makedirs(OUT_DIR, exist_ok=True)
    out = os.path.join(OUT_DIR, "up_silu")
    if os.path.exists(out) and os.path.getmtime(out) >= os.path.getmtime(src):
        return out
    cmd = [nvcc, "-gencode=arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", f"-I{inc}", src, "-o", out, "-lcuda"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        print("[build_ref] nvcc failed:\n" + proc.stdout + proc.stderr)
        return None
    return out


if __name__ == "__main__":
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("DYNAFLOW_REFERENCE", "/root/reference")
    print(build(ref))
