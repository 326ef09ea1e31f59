"""The allocation-free MLP entry point (``df_mlp_gated_bf16_static``).

Some callers cannot hand the library scratch memory and must not allocate it
either: a policy's ``func=`` substitute only holds the subgraph's tensors, and a
serving engine that sized its KV cache from the free HBM has none left (and a
cudaMalloc in mid-forward would synchronise the device and undo the stream
overlap). For them the library keeps the intermediate in a static 64 MiB device
array. This file checks, through the C ABI, that two calls in a row give what the
workspace-taking entry point gives, and that oversize shapes are refused.

Collected last on purpose (file name), so that a run that stops at the first
failure has already run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 2e-2  # max|a-b| / max|b|, the bf16 tolerance of the other GPU tests


def _rand(shape, scale, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).bfloat16().cuda()


def _rel(a, b):
    return ((a.float() - b.float()).abs().max() / b.float().abs().max()).item()


def test_static_scratch_entry_point_matches_workspace_entry_point(native_lib):
    from dynaflow_b200 import _native, ops

    lib = native_lib
    H, I = 256, 1024
    w_gate, w_up, w_down = _rand((I, H), 0.05, 1), _rand((I, H), 0.05, 2), _rand((H, I), 0.05, 3)
    status = ops.status_block()
    stream = torch.cuda.current_stream().cuda_stream
    # two calls in a row with different row counts: the second reuses the array the first one filled
    for call, (M, seed) in enumerate([(300, 10), (129, 11)]):
        x = _rand((M, H), 1.0, seed)
        want = torch.empty(M, H, dtype=torch.bfloat16, device="cuda")
        ws = torch.empty(lib.df_mlp_workspace_bytes(M, H, I), dtype=torch.uint8, device="cuda")
        rc = lib.df_mlp_gated_bf16(x.data_ptr(), w_gate.data_ptr(), w_up.data_ptr(), w_down.data_ptr(), want.data_ptr(),
                                   ws.data_ptr(), M, H, I, 0, status.data_ptr(), stream)
        assert rc == 0, _native.last_error()
        got = torch.full((M, H), float("nan"), dtype=torch.bfloat16, device="cuda")
        rc = lib.df_mlp_gated_bf16_static(x.data_ptr(), w_gate.data_ptr(), w_up.data_ptr(), w_down.data_ptr(),
                                          got.data_ptr(), M, H, I, 0, status.data_ptr(), stream)
        assert rc == 0, _native.last_error()
        torch.cuda.synchronize()
        ops.check_status()
        assert torch.isfinite(got.float()).all(), f"call {call}: output not fully written"
        assert _rel(got, want) <= TOL, f"call {call}"
        # and against the CPU oracle, not only against the library's other entry point
        from oracle import ops_oracle

        oracle = ops_oracle.gated_mlp(x.cpu(), w_gate.cpu(), w_up.cpu(), w_down.cpu())
        assert _rel(got.cpu(), oracle) <= TOL, f"call {call} vs oracle"
    # the tensor-level wrapper goes through the same entry point
    x = _rand((64, H), 1.0, 12)
    out = torch.empty(64, H, dtype=torch.bfloat16, device="cuda")
    ops.gated_mlp_static(x, w_gate, w_up, w_down, out)
    assert _rel(out, ops.gated_mlp(x, w_gate, w_up, w_down)) <= TOL
    ops.check_status()


def test_static_scratch_entry_point_refuses_oversize_shapes(native_lib):
    from dynaflow_b200 import _native, ops

    lib = native_lib
    limit = ops.STATIC_SCRATCH_BYTES
    I = 14336
    M = limit // (2 * I) + 1          # one row past what fits
    dummy = torch.zeros(8, dtype=torch.bfloat16, device="cuda")
    p = dummy.data_ptr()
    rc = lib.df_mlp_gated_bf16_static(p, p, p, p, p, M, 4096, I, 0, ops.status_block().data_ptr(), None)
    assert rc == -3                   # DF_EUNSUPPORTED, decided on the host before any launch
    msg = _native.last_error()
    assert str(limit) in msg and "workspace" in msg
    assert lib.df_mlp_gated_bf16_static(p, p, p, p, p, 0, 4096, I, 0, ops.status_block().data_ptr(), None) == -1
