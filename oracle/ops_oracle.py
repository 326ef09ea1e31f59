"""Floating-point side of the hot path, restated with plain PyTorch CPU ops.

Rounding points are those of the operator chain a host model runs inside the
reference's subgraphs: every operator takes and returns bf16 (or fp32) tensors,
accumulating in fp32 inside.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def gated_mlp(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """``down(silu(gate(x)) * up(x))`` as the chain linear -> silu_and_mul -> linear.

    The SiLU*mul stage reads the (dtype-rounded) GEMM results, computes
    ``g / (1 + exp(-g)) * u`` in fp32 and rounds once
    (``examples/ae/up-silu-overlap.cu:75-90``). Weights are ``[out, in]``."""
    g = F.linear(x, w_gate)
    u = F.linear(x, w_up)
    h = silu_mul(g, u)
    return F.linear(h, w_down)


def silu_mul(g: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    gf, uf = g.float(), u.float()
    return ((gf / (1.0 + torch.exp(-gf))) * uf).to(g.dtype)


def gated_mlp_hf(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """The same MLP written the way a Hugging Face decoder block does it
    (``act_fn(gate_proj(x)) * up_proj(x)``: SiLU and the product each round to the
    tensor dtype). This is the form the reference package executes on CPU for the
    golden vectors; in fp32 it equals ``gated_mlp`` up to rounding of the division."""
    return F.linear(F.silu(F.linear(x, w_gate)) * F.linear(x, w_up), w_down)


def allreduce_add_rmsnorm(partials: list[torch.Tensor], residual: torch.Tensor | None, weight: torch.Tensor,
                          eps: float = 1e-5) -> tuple[torch.Tensor, torch.Tensor]:
    """``y = sum_r partials[r]; r' = y + residual; out = rmsnorm(r') * weight``.

    Call-site semantics: ``examples/ae/scheduler/vllm/nanoflow.py:171-211`` (residual
    is zeros when absent; eps 1e-5) and the in-tree kernel
    ``tokenweave-kernels/csrc/tokenweave.cu:38-113``: the cross-rank sum accumulates
    in fp32 and is rounded to bf16, the residual add is a bf16 add, the new residual
    is stored in bf16, the sum of squares is fp32 over the bf16 residual, and the
    normalised value is rounded to bf16 before the multiplication by the weight
    (``temp *= s_variance; temp *= weight`` on bf16 vectors).
    Returns ``(out, new_residual)``."""
    dtype = partials[0].dtype
    acc = torch.zeros_like(partials[0], dtype=torch.float32)
    for p in partials:
        acc += p.float()
    y = acc.to(dtype)
    if residual is None:
        residual = torch.zeros_like(y)
    new_res = (y.float() + residual.float()).to(dtype)
    var = new_res.float().pow(2).sum(dim=-1, keepdim=True) / new_res.shape[-1]
    inv = torch.rsqrt(var + eps)
    normed = (new_res.float() * inv).to(dtype)
    out = (normed.float() * weight.float()).to(dtype)
    return out, new_res


def top2_route(router_logits: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Mixtral-style routing: softmax over experts in fp32, top-2, renormalise.
    Returns ``(weights [T,2] fp32, expert ids [T,2] int64)``; ties resolve to the
    lower expert index (``torch.topk`` leaves the order of equal values unspecified; the
    serving stacks' routing kernels prefer the lower index, and so do this oracle and the
    CUDA kernel)."""
    probs = torch.softmax(router_logits.float(), dim=-1)
    order = torch.sort(probs, dim=-1, descending=True, stable=True)   # stable: equal values keep index order
    w, ids = order.values[..., :2], order.indices[..., :2]
    w = w / w.sum(dim=-1, keepdim=True)
    return w, ids


def moe_layer(x: torch.Tensor, router_logits: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor,
              w_down: torch.Tensor, mlp=None) -> torch.Tensor:
    """Top-2 mixture of gated-MLP experts: dispatch = index gather of the rows routed
    to an expert, combine = weighted scatter-add in fp32, rounded once at the end.
    ``w_gate, w_up: [E, I, H]``, ``w_down: [E, H, I]``. The three-way operator split
    dispatch / expert / combine is ``examples/ae/patch/vllm.patch:308-379, 423-527``.
    ``mlp`` selects the expert's operator chain (default: ``gated_mlp``, the fused-epilogue
    rounding; ``gated_mlp_hf`` reproduces the reference-executed fixture bit for bit)."""
    mlp = mlp or gated_mlp
    weights, ids = top2_route(router_logits)
    out = torch.zeros(x.shape, dtype=torch.float32)
    for e in range(w_gate.shape[0]):
        rows, slot = torch.nonzero(ids == e, as_tuple=True)
        if rows.numel() == 0:
            continue
        y = mlp(x[rows], w_gate[e], w_up[e], w_down[e])
        out.index_add_(0, rows, y.float() * weights[rows, slot].unsqueeze(-1))
    return out.to(x.dtype)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, seq_lens: list[int],
                     scale: float | None = None) -> torch.Tensor:
    """Causal grouped-query self-attention over sequences packed back to back along dim 0.
    ``q [T, Hq, D]``, ``k, v [T, Hkv, D]`` -> ``[T, Hq, D]``. The attention subgraph of a
    decoder layer is opaque to the reference (``examples/ae/scheduler/vllm/nanoflow.py:91-94``:
    whatever kernel the host model calls); the statement here is the one
    ``torch.nn.functional.scaled_dot_product_attention(is_causal=True)`` documents: scores and
    softmax in fp32, probabilities rounded to the tensor dtype before the product with ``v``,
    fp32 accumulation, one final rounding."""
    T, hq, d = q.shape
    hkv = k.shape[1]
    scale = scale if scale is not None else d ** -0.5
    out = torch.empty_like(q)
    start = 0
    for n in seq_lens:
        qs = q[start:start + n].float().transpose(0, 1)                       # [Hq, n, D]
        ks = k[start:start + n].float().transpose(0, 1).repeat_interleave(hq // hkv, dim=0)
        vs = v[start:start + n].float().transpose(0, 1).repeat_interleave(hq // hkv, dim=0)
        s = (qs @ ks.transpose(1, 2)) * scale
        s = s.masked_fill(torch.ones(n, n, dtype=torch.bool).triu(1), float("-inf"))
        p = torch.softmax(s, dim=-1).to(q.dtype).float()
        out[start:start + n] = (p @ vs).transpose(0, 1).to(q.dtype)
        start += n
    assert start == T
    return out


def decode_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, seq_lens: list[int],
                     scale: float | None = None) -> torch.Tensor:
    """One query token per sequence against its key/value cache. ``q [B, Hq, D]``,
    ``k_cache, v_cache [B, max_len, Hkv, D]`` of which the first ``seq_lens[b]`` positions are
    valid -> ``[B, Hq, D]``. Same statement as ``causal_attention`` for the last position of a
    sequence (the new token attends to every valid key, itself included)."""
    B, hq, d = q.shape
    hkv = k_cache.shape[2]
    scale = scale if scale is not None else d ** -0.5
    out = torch.empty_like(q)
    for b, n in enumerate(seq_lens):
        ks = k_cache[b, :n].float().transpose(0, 1).repeat_interleave(hq // hkv, dim=0)     # [Hq, n, D]
        vs = v_cache[b, :n].float().transpose(0, 1).repeat_interleave(hq // hkv, dim=0)
        s = torch.einsum("hd,hnd->hn", q[b].float(), ks) * scale
        p = torch.softmax(s, dim=-1).to(q.dtype).float()
        out[b] = torch.einsum("hn,hnd->hd", p, vs).to(q.dtype)
    return out
