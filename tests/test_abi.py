"""The C-ABI library: it builds for sm_100a, loads, exports every symbol the public
header declares, and validates arguments on the host (no compute without a GPU)."""
import ctypes
import os
import re

from conftest import ROOT


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "dynaflow_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(df_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(native_lib):
    from dynaflow_b200 import _native

    declared = _declared_symbols()
    assert len(declared) >= 10
    for name in declared:
        assert hasattr(native_lib, name), f"{name} is declared in the header but not exported"
        assert name in _native.SIGNATURES, f"{name} has no ctypes prototype"
    assert sorted(_native.SIGNATURES) == declared
    assert native_lib.df_version() == 1


def test_host_side_argument_validation(native_lib):
    from dynaflow_b200 import _native

    assert native_lib.df_set_timeout_ms(0) == -1 and "positive" in _native.last_error()
    assert native_lib.df_set_timeout_ms(2000) == 0
    assert native_lib.df_gemm_bf16(None, None, None, 128, 128, 128, 128, 128, 128, 0, None, None) == -1
    assert "NULL" in _native.last_error()
    buf = (ctypes.c_char * 4096)()
    p = ctypes.addressof(buf)
    p += (-p) % 256
    # shape errors are reported before anything touches the device
    assert native_lib.df_gemm_bf16(p, p, p, 0, 128, 128, 128, 128, 128, 0, p, None) == -1
    assert native_lib.df_gemm_bf16(p, p, p, 16, 12, 128, 128, 128, 128, 0, p, None) == -3      # N % 8
    assert native_lib.df_gemm_bf16(p, p, p, 16, 16, 128, 64, 128, 128, 0, p, None) == -1       # lda < K
    assert native_lib.df_gemm_bf16(p + 2, p, p, 16, 16, 128, 128, 128, 128, 0, p, None) == -1  # alignment
    assert native_lib.df_mlp_gated_bf16(p, p, p, p, p, None, 16, 128, 128, 0, p, None) == -1
    assert native_lib.df_mlp_workspace_bytes(0, 64, 64) == 0
    assert native_lib.df_mlp_workspace_bytes(16, 4096, 14336) >= 16 * 14336 * 2
    assert native_lib.df_status_read(None, None, None) == -1


def test_ops_refuse_cpu_tensors():
    import pytest
    import torch

    from dynaflow_b200 import ops

    x = torch.zeros(4, 8, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        ops.gemm_bf16(x, x)
