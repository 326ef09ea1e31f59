"""ctypes binding of ``libdynaflow_b200.so`` (declarations: ``include/dynaflow_b200.h``).

There is no fallback: if the library has not been built, importing this module
raises, and so does every op of the package.
"""
from __future__ import annotations

import ctypes
import os

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libdynaflow_b200.so")


class NativeLibraryMissing(RuntimeError):
    pass


class df_status_t(ctypes.Structure):
    _fields_ = [("code", ctypes.c_uint32), ("where", ctypes.c_uint32),
                ("block", ctypes.c_uint32), ("aux", ctypes.c_uint32)]


_vp, _i, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t

MAX_WORLD = 8
MAX_CTAS = 64


class df_comm_rank_t(ctypes.Structure):
    _fields_ = [("rank", ctypes.c_int), ("regions", ctypes.c_void_p * MAX_WORLD),
                ("residual_in", ctypes.c_void_p), ("residual_out", ctypes.c_void_p), ("out", ctypes.c_void_p)]


class df_a2a_rank_t(ctypes.Structure):
    _fields_ = [("rank", ctypes.c_int), ("regions", ctypes.c_void_p * MAX_WORLD)]


_handle = ctypes.c_ubyte * 64
_f = ctypes.c_float
_rank_p = ctypes.POINTER(df_comm_rank_t)

# name -> (restype, argtypes); must list every symbol the public header declares
SIGNATURES: dict[str, tuple] = {
    "df_version": (_i, []),
    "df_last_error": (ctypes.c_char_p, []),
    "df_set_timeout_ms": (_i, [_i]),
    "df_sm_count": (_i, []),
    "df_status_read": (_i, [_vp, ctypes.POINTER(df_status_t), _vp]),
    "df_status_clear": (_i, [_vp, _vp]),
    "df_gemm_bf16": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _vp]),
    "df_gateup_silu_bf16": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _vp]),
    "df_set_launch_option": (_i, [_i, _i]),
    "df_gemm_splitk_workspace_bytes": (_sz, []),
    "df_gemm_bf16_ws": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _sz, _vp, _vp]),
    "df_gateup_silu_bf16_ws": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _sz, _vp, _vp]),
    "df_mlp_workspace_bytes": (_sz, [_i, _i, _i]),
    "df_mlp_gated_bf16": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp]),
    "df_comm_region_bytes": (_sz, [_i, _i]),
    "df_comm_partial_offset": (_sz, [_i, _i]),
    "df_comm_sum_offset": (_sz, [_i, _i]),
    "df_comm_region_alloc": (_i, [_sz, ctypes.POINTER(_vp), ctypes.POINTER(_handle)]),
    "df_comm_region_open": (_i, [ctypes.POINTER(_handle), ctypes.POINTER(_vp)]),
    "df_comm_region_close": (_i, [_vp]),
    "df_comm_region_free": (_i, [_vp]),
    "df_allreduce_bf16": (_i, [_rank_p, _i, _i, _i, _i, _i, _vp, _vp]),
    "df_all_gather_bf16": (_i, [_rank_p, _i, _i, _i, _i, _i, _vp, _vp]),
    "df_reduce_scatter_bf16": (_i, [_rank_p, _i, _i, _i, _i, _i, _vp, _vp]),
    "df_moe_route_top2": (_i, [_vp, _i, _i, _vp, _vp, _vp]),
    "df_moe_select_rows": (_i, [_vp, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "df_moe_gather_rows": (_i, [_vp, _vp, _vp, _i, _i, _vp, _vp]),
    "df_moe_scatter_rows": (_i, [_vp, _vp, _vp, _vp, _i, _i, _vp, _vp]),
    "df_mlp_gated_bf16_rows_on_device": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _vp, _vp]),
    "df_a2a_region_bytes": (_sz, [_i, _i, _i, _i]),
    "df_a2a_packed_in_offset": (_sz, [_i, _i, _i, _i]),
    "df_a2a_packed_out_offset": (_sz, [_i, _i, _i, _i]),
    "df_a2a_rows_total_offset": (_sz, []),
    "df_a2a_plan": (_i, [_vp, _i, _i, _vp, _vp, _vp]),
    "df_a2a_dispatch_bf16": (_i, [ctypes.POINTER(df_a2a_rank_t), _i, _i, _i, _i, _vp, _vp, _vp, _vp, _i, _i, _vp, _vp]),
    "df_a2a_combine_bf16": (_i, [ctypes.POINTER(df_a2a_rank_t), _i, _i, _i, _i, _vp, _vp, _vp, _i, _vp, _i, _vp, _vp]),
    "df_a2a_emulated_bf16": (_i, [ctypes.POINTER(df_a2a_rank_t), _i, _i, _i, _i, _i, ctypes.POINTER(_vp), ctypes.POINTER(_vp),
                                  ctypes.POINTER(_vp), ctypes.POINTER(_vp), ctypes.POINTER(_vp), ctypes.POINTER(_vp), _i, _i,
                                  _vp, _vp]),
    "df_rope_bf16": (_i, [_vp, _vp, _i, _i, _i, _i, _f, _vp]),
    "df_allreduce_add_rmsnorm_bf16": (_i, [_rank_p, _i, _i, _i, _i, _vp, _f, _i, _vp, _vp]),
    "df_allreduce_add_rmsnorm_sharded_bf16": (_i, [_rank_p, _i, _i, _i, _i, _vp, _f, _i, _vp, _vp]),
    "df_comm_set_exclusive_smem": (_i, [_i]),
    "df_allreduce_multicast_bf16": (_i, [_rank_p, _vp, _i, _i, _i, _i, _i, _vp, _f, _i, _vp, _vp]),
    "df_add_rmsnorm_bf16": (_i, [_vp, _vp, _vp, _vp, _vp, _f, _i, _i, _vp]),
    "df_allreduce_emulated_bf16": (_i, [_rank_p, _i, _i, _i, _i, _vp, _f, _i, _i, _vp, _vp]),
    "df_attention_prefill_bf16": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _i, _vp, _vp]),
    "df_attention_decode_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "df_attention_decode_bf16": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _f, _vp, _sz, _i, _vp, _vp]),
    "df_kv_cache_append_bf16": (_i, [_vp, _vp, _i, _vp, _vp, _i, _vp, _i, _i, _i, _i, _vp]),
    "df_small_gemm_plan": (_i, [_i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "df_rope_append_bf16": (_i, [_vp, _i, _vp, _i, _i, _i, _i, _f, _vp, _vp, _i, _i, _vp]),
    "df_mlp_gated_bf16_static": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp]),
}

_lib = None


def lib_path() -> str:
    return _LIB_PATH


def load() -> ctypes.CDLL:
    """Loads the shared library once and attaches the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        raise NativeLibraryMissing(
            f"{_LIB_PATH} is missing: build it with `python -m dynaflow_b200.csrc.build` "
            "(dynaflow_b200 has no CPU or PyTorch fallback)")
    lib = ctypes.CDLL(_LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def last_error() -> str:
    return load().df_last_error().decode("utf-8", "replace")
