"""Llama-style decoder written with plain PyTorch modules: the host model of the
CPU parity configuration (2 layers, hidden 1024, intermediate 2816, 16 heads of 64,
RMSNorm eps 1e-5, RoPE theta 10000, vocab 32000; weights N(0, 0.02) from a seed).

It plays the role the Hugging Face model plays in the reference's own harness
(``examples/ae/scripts/bench_hf_transformers.py:61-105``): it is traced by
``torch.compile(fullgraph=True)`` with dim 0 of the ids marked dynamic, and the
resulting FX graph is what the scheduling layer partitions and executes.
"""
from __future__ import annotations

import dataclasses

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclasses.dataclass
class LlamaShape:
    hidden: int = 1024
    intermediate: int = 2816
    heads: int = 16
    kv_heads: int = 16
    head_dim: int = 64
    layers: int = 2
    vocab: int = 32000
    eps: float = 1e-5
    rope_theta: float = 10000.0


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        xf = x.float()
        xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)
        return (xf * self.weight.float()).to(x.dtype)


def rope_tables(seq: int, head_dim: int, theta: float, device=None) -> tuple[torch.Tensor, torch.Tensor]:
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    ang = torch.outer(torch.arange(seq, dtype=torch.float32, device=device), inv)
    ang = torch.cat([ang, ang], dim=-1)
    return ang.cos(), ang.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: [B, heads, S, D]; rotate-half convention."""
    half = x.shape[-1] // 2
    rot = torch.cat([-x[..., half:], x[..., :half]], dim=-1)
    return (x.float() * cos + rot.float() * sin).to(x.dtype)


class Attention(nn.Module):
    def __init__(self, s: LlamaShape) -> None:
        super().__init__()
        self.s = s
        self.q_proj = nn.Linear(s.hidden, s.heads * s.head_dim, bias=False)
        self.k_proj = nn.Linear(s.hidden, s.kv_heads * s.head_dim, bias=False)
        self.v_proj = nn.Linear(s.hidden, s.kv_heads * s.head_dim, bias=False)
        self.o_proj = nn.Linear(s.heads * s.head_dim, s.hidden, bias=False)

    def forward(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        s = self.s
        b, t, _ = x.shape
        q = self.q_proj(x).view(b, t, s.heads, s.head_dim).transpose(1, 2)
        k = self.k_proj(x).view(b, t, s.kv_heads, s.head_dim).transpose(1, 2)
        v = self.v_proj(x).view(b, t, s.kv_heads, s.head_dim).transpose(1, 2)
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        if s.kv_heads != s.heads:
            rep = s.heads // s.kv_heads
            k = k.repeat_interleave(rep, dim=1)
            v = v.repeat_interleave(rep, dim=1)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        return self.o_proj(o.transpose(1, 2).reshape(b, t, s.heads * s.head_dim))


class GatedMLP(nn.Module):
    def __init__(self, hidden: int, intermediate: int) -> None:
        super().__init__()
        self.gate_proj = nn.Linear(hidden, intermediate, bias=False)
        self.up_proj = nn.Linear(hidden, intermediate, bias=False)
        self.down_proj = nn.Linear(intermediate, hidden, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))


class Block(nn.Module):
    def __init__(self, s: LlamaShape) -> None:
        super().__init__()
        self.input_norm = RMSNorm(s.hidden, s.eps)
        self.attn = Attention(s)
        self.post_norm = RMSNorm(s.hidden, s.eps)
        self.mlp = GatedMLP(s.hidden, s.intermediate)

    def forward(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        x = x + self.attn(self.input_norm(x), cos, sin)
        return x + self.mlp(self.post_norm(x))


class LlamaDecoder(nn.Module):
    """ids [B, S] -> logits [B, S, vocab]; dim 0 (requests) is the split axis."""

    def __init__(self, s: LlamaShape) -> None:
        super().__init__()
        self.s = s
        self.embed = nn.Embedding(s.vocab, s.hidden)
        self.blocks = nn.ModuleList(Block(s) for _ in range(s.layers))
        self.norm = RMSNorm(s.hidden, s.eps)
        self.lm_head = nn.Linear(s.hidden, s.vocab, bias=False)

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        cos, sin = rope_tables(ids.shape[1], self.s.head_dim, self.s.rope_theta, device=ids.device)
        x = self.embed(ids)
        for block in self.blocks:
            x = block(x, cos, sin)
        return self.lm_head(self.norm(x))


def build(shape: LlamaShape, seed: int = 0, dtype: torch.dtype = torch.float32) -> LlamaDecoder:
    """Model with every Linear / Embedding weight drawn N(0, 0.02) from ``seed``
    (norm weights stay 1), in evaluation mode."""
    gen = torch.Generator().manual_seed(seed)
    model = LlamaDecoder(shape)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.dim() >= 2:
                p.copy_(torch.randn(p.shape, generator=gen) * 0.02)
    return model.to(dtype).eval()


def make_ids(batch: int, seq: int, vocab: int, seed: int = 1) -> torch.Tensor:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (batch, seq), generator=gen, dtype=torch.int64)
