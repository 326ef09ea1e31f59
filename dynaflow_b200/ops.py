"""Tensor-level wrappers over the C ABI (``include/dynaflow_b200.h``).

PyTorch is used for device memory and streams only: every function here hands
raw device pointers and the current CUDA stream to ``libdynaflow_b200.so``.
There is no eager/PyTorch fallback; a missing library or a CPU tensor raises.

Weight layout is ``torch.nn.Linear``'s ``[out_features, in_features]``, i.e. the
layout the subgraphs of a DynaFlow-split model hold their weights in.
"""
from __future__ import annotations

import ctypes

import torch

from . import _native
from ._native import df_status_t

DEVICE_ERRORS = {1: "DF_ERR_TIMEOUT", 2: "DF_ERR_PEER"}
_WHERE = {1: "tma-producer", 2: "mma(full)", 3: "mma(tmem-empty)", 4: "epilogue", 5: "h-ready", 16: "peer-flag", 21: "small-gemm-producer", 22: "small-gemm-mma", 23: "small-gemm-epilogue", 24: "small-gemm-partial-rows", 32: "attention-producer", 33: "attention-mma", 34: "attention-softmax"}


class DeviceStatusError(RuntimeError):
    """A kernel reported a bounded wait that ran out (the context stays usable)."""


_status: dict[int, torch.Tensor] = {}


def _dev_index(t: torch.Tensor) -> int:
    if not t.is_cuda:
        raise RuntimeError("dynaflow_b200 ops take CUDA tensors only (there is no CPU path)")
    return t.device.index if t.device.index is not None else torch.cuda.current_device()


def status_block(device: int | torch.device | None = None) -> torch.Tensor:
    """The per-device 16-byte status block kernels report into."""
    if device is None:
        device = torch.cuda.current_device()
    idx = device.index if isinstance(device, torch.device) else int(device)
    st = _status.get(idx)
    if st is None:
        st = torch.zeros(4, dtype=torch.int32, device=f"cuda:{idx}")
        _status[idx] = st
    return st


def read_status(device=None) -> df_status_t:
    """Synchronises the current stream and returns the device status block."""
    st = status_block(device)
    host = df_status_t()
    rc = _native.load().df_status_read(st.data_ptr(), ctypes.byref(host), _stream_ptr(st))
    if rc != 0:
        raise RuntimeError(f"df_status_read failed ({rc}): {_native.last_error()}")
    return host


def check_status(device=None) -> None:
    """Raises ``DeviceStatusError`` if a kernel recorded an error; clears the block."""
    host = read_status(device)
    if host.code != 0:
        st = status_block(device)
        _native.load().df_status_clear(st.data_ptr(), _stream_ptr(st))
        raise DeviceStatusError(
            f"device status {DEVICE_ERRORS.get(host.code, host.code)} at {_WHERE.get(host.where, host.where)} "
            f"(block {host.block}, aux {host.aux})")


def set_timeout_ms(ms: int) -> None:
    rc = _native.load().df_set_timeout_ms(int(ms))
    if rc != 0:
        raise ValueError(_native.last_error())


LAUNCH_OPTIONS = {"stream_k": 0, "mlp_one_launch": 1, "operand_swap": 2, "split_k_small": 3, "decode_keys_on_lanes": 4, "dependent_launch": 5}


def set_launch_option(name: str, on: bool) -> None:
    """Switches one of the equally valid launch forms on or off (``df_set_launch_option``)."""
    rc = _native.load().df_set_launch_option(LAUNCH_OPTIONS[name], int(bool(on)))
    if rc != 0:
        raise ValueError(_native.last_error())


def _stream_ptr(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed ({rc}): {_native.last_error()}")


def _require_bf16_2d(name: str, t: torch.Tensor) -> None:
    if t.dtype != torch.bfloat16 or t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be a 2-D bf16 tensor with unit inner stride, got "
                         f"{t.dtype} {tuple(t.shape)} strides {t.stride()}")


_splitk_ws: dict[tuple[int, int], torch.Tensor] = {}


def splitk_workspace(device: torch.device) -> torch.Tensor:
    """Scratch for the stream-K form of the GEMMs: one per (device, stream), created on first
    use, so that launches on different streams never share partial sums."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    key = (idx, torch.cuda.current_stream(device).cuda_stream)
    ws = _splitk_ws.get(key)
    if ws is None:
        with torch.cuda.device(idx):
            ws = torch.empty(int(_native.load().df_gemm_splitk_workspace_bytes()), dtype=torch.uint8, device=device)
        _splitk_ws[key] = ws
    return ws


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, max_ctas: int = 0) -> torch.Tensor:
    """``out[M,N] = a[M,K] @ b[N,K].T`` (``b`` in ``nn.Linear`` layout)."""
    _require_bf16_2d("a", a)
    _require_bf16_2d("b", b)
    M, K = a.shape
    N, Kb = b.shape
    if K != Kb:
        raise ValueError(f"inner dimensions differ: a is {tuple(a.shape)}, b is {tuple(b.shape)}")
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    _require_bf16_2d("out", out)
    if tuple(out.shape) != (M, N):
        raise ValueError(f"out must be {(M, N)}, got {tuple(out.shape)}")
    if M == 0:
        return out
    _dev_index(a)
    st = status_block(a.device)
    ws = splitk_workspace(a.device)
    rc = _native.load().df_gemm_bf16_ws(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0),
                                        out.stride(0), max_ctas, ws.data_ptr(), ws.numel(), st.data_ptr(),
                                        _stream_ptr(a))
    _check(rc, "df_gemm_bf16_ws")
    return out


def gateup_silu(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, out: torch.Tensor | None = None,
                max_ctas: int = 0) -> torch.Tensor:
    """``silu(x @ w_gate.T) * (x @ w_up.T)`` with the SiLU*mul fused into the GEMM epilogue."""
    _require_bf16_2d("x", x)
    _require_bf16_2d("w_gate", w_gate)
    _require_bf16_2d("w_up", w_up)
    M, H = x.shape
    I = w_gate.shape[0]
    if tuple(w_gate.shape) != (I, H) or tuple(w_up.shape) != (I, H) or w_gate.stride(0) != w_up.stride(0):
        raise ValueError("w_gate and w_up must both be [I, H] with equal row strides")
    if out is None:
        out = torch.empty((M, I), dtype=torch.bfloat16, device=x.device)
    _require_bf16_2d("out", out)
    if M == 0:
        return out
    _dev_index(x)
    st = status_block(x.device)
    ws = splitk_workspace(x.device)
    rc = _native.load().df_gateup_silu_bf16_ws(x.data_ptr(), w_gate.data_ptr(), w_up.data_ptr(), out.data_ptr(), M, H, I,
                                               x.stride(0), w_gate.stride(0), out.stride(0), max_ctas, ws.data_ptr(),
                                               ws.numel(), st.data_ptr(), _stream_ptr(x))
    _check(rc, "df_gateup_silu_bf16_ws")
    return out


def mlp_workspace_bytes(M: int, H: int, I: int) -> int:
    return int(_native.load().df_mlp_workspace_bytes(M, H, I))


def gated_mlp(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor,
              out: torch.Tensor | None = None, workspace: torch.Tensor | None = None,
              max_ctas: int = 0) -> torch.Tensor:
    """``(silu(x @ w_gate.T) * (x @ w_up.T)) @ w_down.T`` for one nano-batch of rows."""
    for name, t in (("x", x), ("w_gate", w_gate), ("w_up", w_up), ("w_down", w_down)):
        _require_bf16_2d(name, t)
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
    M, H = x.shape
    I = w_gate.shape[0]
    if tuple(w_gate.shape) != (I, H) or tuple(w_up.shape) != (I, H) or tuple(w_down.shape) != (H, I):
        raise ValueError("expected w_gate, w_up: [I, H] and w_down: [H, I]")
    if out is None:
        out = torch.empty((M, H), dtype=torch.bfloat16, device=x.device)
    if not out.is_contiguous() or tuple(out.shape) != (M, H) or out.dtype != torch.bfloat16:
        raise ValueError("out must be a contiguous bf16 [M, H] tensor")
    if M == 0:
        return out
    need = mlp_workspace_bytes(M, H, I)
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
    if workspace.numel() * workspace.element_size() < need:
        raise ValueError(f"workspace too small: need {need} bytes")
    _dev_index(x)
    st = status_block(x.device)
    rc = _native.load().df_mlp_gated_bf16(x.data_ptr(), w_gate.data_ptr(), w_up.data_ptr(), w_down.data_ptr(),
                                          out.data_ptr(), workspace.data_ptr(), M, H, I, max_ctas, st.data_ptr(),
                                          _stream_ptr(x))
    _check(rc, "df_mlp_gated_bf16")
    return out


def attention_prefill(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor, *, batch: int, seq_len: int,
                      cu_seqlens: torch.Tensor | None = None, scale: float | None = None, max_ctas: int = 0) -> torch.Tensor:
    """Causal grouped-query attention of a prefill nano-batch. ``q [T, Hq*128]``, ``k, v [T, Hkv*128]``,
    ``out [T, Hq*128]``: 2-D bf16 views with unit inner stride (column ranges of a fused qkv
    activation are fine). The ``T`` rows are ``batch`` sequences back to back, each ``seq_len``
    long, or starting at ``cu_seqlens[b]`` (int32 on the device, ``batch + 1`` entries; ``seq_len``
    is then the longest length)."""
    for name, t in (("q", q), ("k", k), ("v", v), ("out", out)):
        _require_bf16_2d(name, t)
    T = q.shape[0]
    hd = 128
    if q.shape[1] % hd or k.shape[1] % hd or tuple(k.shape) != tuple(v.shape) or tuple(out.shape) != tuple(q.shape) \
            or k.shape[0] != T:
        raise ValueError("expected q/out [T, Hq*128] and k/v [T, Hkv*128]")
    if T == 0:
        return out
    if cu_seqlens is not None and (cu_seqlens.dtype != torch.int32 or not cu_seqlens.is_cuda
                                   or cu_seqlens.numel() != batch + 1):
        raise ValueError("cu_seqlens must be an int32 device tensor of batch + 1 entries")
    _dev_index(q)
    st = status_block(q.device)
    rc = _native.load().df_attention_prefill_bf16(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), T, batch, seq_len,
        cu_seqlens.data_ptr() if cu_seqlens is not None else None, q.shape[1] // hd, k.shape[1] // hd, hd,
        q.stride(0), k.stride(0), v.stride(0), out.stride(0), float(scale if scale is not None else hd ** -0.5),
        max_ctas, st.data_ptr(), _stream_ptr(q))
    _check(rc, "df_attention_prefill_bf16")
    return out


def attention_decode_workspace_bytes(batch: int, q_heads: int, kv_heads: int, max_len: int) -> int:
    return int(_native.load().df_attention_decode_workspace_bytes(batch, q_heads, kv_heads, max_len))


def attention_decode_workspace(batch: int, q_heads: int, kv_heads: int, max_len: int,
                               device: torch.device | str = "cuda") -> torch.Tensor:
    """Scratch for ``attention_decode`` (the chunks' partial results); its contents are arbitrary."""
    return torch.empty(attention_decode_workspace_bytes(batch, q_heads, kv_heads, max_len), dtype=torch.uint8, device=device)


def rope_append(qkv: torch.Tensor, seq_lens: torch.Tensor, q_heads: int, kv_heads: int, k_cache: torch.Tensor,
                v_cache: torch.Tensor, theta: float) -> None:
    """Rotary embedding of the new token's query and key heads (position ``seq_lens[b] - 1``) in place in
    ``qkv [B, (Hq + 2 Hkv) * 128]``, rotated keys and values into that position of the caches, one launch."""
    _require_bf16_2d("qkv", qkv)
    B = qkv.shape[0]
    if k_cache.dim() != 3 or not k_cache.is_contiguous() or not v_cache.is_contiguous() or k_cache.shape[0] != B \
            or k_cache.shape[2] != kv_heads * 128 or tuple(v_cache.shape) != tuple(k_cache.shape):
        raise ValueError("expected contiguous bf16 caches [B, max_len, Hkv*128]")
    rc = _native.load().df_rope_append_bf16(qkv.data_ptr(), qkv.stride(0), seq_lens.data_ptr(), B, q_heads, kv_heads, 128,
                                            float(theta), k_cache.data_ptr(), v_cache.data_ptr(), k_cache.shape[2],
                                            k_cache.shape[1], _stream_ptr(qkv))
    _check(rc, "df_rope_append_bf16")


def attention_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, seq_lens: torch.Tensor,
                     out: torch.Tensor, workspace: torch.Tensor, *, scale: float | None = None,
                     max_ctas: int = 0) -> torch.Tensor:
    """One new token per sequence against its key/value cache. ``q, out [B, Hq*128]`` (2-D bf16
    views, unit inner stride), ``k_cache, v_cache [B, max_len, Hkv*128]`` contiguous bf16,
    ``seq_lens`` int32 on the device, ``workspace`` from ``attention_decode_workspace``."""
    _require_bf16_2d("q", q)
    _require_bf16_2d("out", out)
    hd = 128
    B = q.shape[0]
    if k_cache.dtype != torch.bfloat16 or k_cache.dim() != 3 or not k_cache.is_contiguous() \
            or tuple(v_cache.shape) != tuple(k_cache.shape) or not v_cache.is_contiguous() or k_cache.shape[0] != B:
        raise ValueError("expected contiguous bf16 caches [B, max_len, Hkv*128]")
    max_len, kv_cols = k_cache.shape[1], k_cache.shape[2]
    if q.shape[1] % hd or kv_cols % hd or tuple(out.shape) != tuple(q.shape):
        raise ValueError("expected q/out [B, Hq*128] and caches [B, max_len, Hkv*128]")
    if seq_lens.dtype != torch.int32 or not seq_lens.is_cuda or seq_lens.numel() != B:
        raise ValueError("seq_lens must be an int32 device tensor of B entries")
    _dev_index(q)
    st = status_block(q.device)
    rc = _native.load().df_attention_decode_bf16(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), seq_lens.data_ptr(), B, max_len,
        q.shape[1] // hd, kv_cols // hd, hd, q.stride(0), kv_cols, out.stride(0),
        float(scale if scale is not None else hd ** -0.5), workspace.data_ptr(), workspace.numel(), max_ctas,
        st.data_ptr(), _stream_ptr(q))
    _check(rc, "df_attention_decode_bf16")
    return out


def kv_cache_append(k_new: torch.Tensor, v_new: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    seq_lens: torch.Tensor) -> None:
    """``cache[b, seq_lens[b] - 1] = new[b]`` for keys and values (``k_new, v_new [B, Hkv*128]`` views
    with equal row strides)."""
    _require_bf16_2d("k_new", k_new)
    _require_bf16_2d("v_new", v_new)
    if k_new.stride(0) != v_new.stride(0) or tuple(k_new.shape) != tuple(v_new.shape):
        raise ValueError("k_new and v_new must have equal shapes and row strides")
    B, cols = k_new.shape
    rc = _native.load().df_kv_cache_append_bf16(k_new.data_ptr(), v_new.data_ptr(), k_new.stride(0), k_cache.data_ptr(),
                                                v_cache.data_ptr(), cols, seq_lens.data_ptr(), B, k_cache.shape[1],
                                                cols // 128, 128, _stream_ptr(k_new))
    _check(rc, "df_kv_cache_append_bf16")


STATIC_SCRATCH_BYTES = 64 << 20


def gated_mlp_static(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor,
                     out: torch.Tensor, max_ctas: int = 0) -> torch.Tensor:
    """``gated_mlp`` for callers that cannot provide or allocate scratch (a policy
    substitute that only holds the subgraph's tensors, a host whose HBM is fully
    budgeted): the intermediate lives in a 64 MiB array inside the library, so
    ``rows * I * 2`` must not exceed ``STATIC_SCRATCH_BYTES`` and ``out`` must be
    passed in. This wrapper itself creates no tensor. Calls that may overlap on the
    GPU share that array and race; the first call on a device should happen
    outside stream capture (it looks up the array's address)."""
    for name, t in (("x", x), ("w_gate", w_gate), ("w_up", w_up), ("w_down", w_down), ("out", out)):
        _require_bf16_2d(name, t)
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
    M, H = x.shape
    I = w_gate.shape[0]
    if tuple(w_gate.shape) != (I, H) or tuple(w_up.shape) != (I, H) or tuple(w_down.shape) != (H, I):
        raise ValueError("expected w_gate, w_up: [I, H] and w_down: [H, I]")
    if tuple(out.shape) != (M, H):
        raise ValueError("out must be [M, H]")
    if M == 0:
        return out
    _dev_index(x)
    st = status_block(x.device)
    rc = _native.load().df_mlp_gated_bf16_static(x.data_ptr(), w_gate.data_ptr(), w_up.data_ptr(), w_down.data_ptr(),
                                                 out.data_ptr(), M, H, I, max_ctas, st.data_ptr(), _stream_ptr(x))
    _check(rc, "df_mlp_gated_bf16_static")
    return out
