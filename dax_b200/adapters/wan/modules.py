"""Minimal Wan2.1-shaped modules for running and testing the attention processor without
``diffusers``.

The reference plugs its processor into ``diffusers.models.attention_processor.Attention``; these
classes expose exactly the attributes that processor touches (``to_q/to_k/to_v``, ``to_out``,
``norm_q/norm_k``, ``heads``, ``add_k_proj``…, ``set_processor``) with the same shapes, so the
processor cannot tell the difference.  With diffusers installed, ``replace_wan_attention`` patches
the real class instead."""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
from torch import nn


class RMSNorm(nn.Module):
    """RMS normalisation over the last dimension with a learned weight (eps 1e-6 in Wan)."""

    def __init__(self, dim: int, eps: float = 1e-6, elementwise_affine: bool = True):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim)) if elementwise_affine else None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + self.eps)
        if self.weight is not None:
            y = y * self.weight.float()
        return y.to(x.dtype)


class Attention(nn.Module):
    """Wan attention block: Q/K/V/O linears with bias, RMSNorm on Q and K across all heads."""

    def __init__(self, dim: int, heads: int, dim_head: int = 128, eps: float = 1e-6, cross_attention_dim: Optional[int] = None,
                 processor=None):
        super().__init__()
        assert heads * dim_head == dim
        self.heads = heads
        self.inner_dim = dim
        kv_dim = cross_attention_dim or dim
        self.to_q = nn.Linear(dim, dim, bias=True)
        self.to_k = nn.Linear(kv_dim, dim, bias=True)
        self.to_v = nn.Linear(kv_dim, dim, bias=True)
        self.to_out = nn.ModuleList([nn.Linear(dim, dim, bias=True), nn.Dropout(0.0)])
        self.norm_q = RMSNorm(dim, eps)
        self.norm_k = RMSNorm(dim, eps)
        self.add_k_proj = self.add_v_proj = self.norm_added_k = None
        self.processor = processor

    def set_processor(self, processor) -> None:
        self.processor = processor

    def forward(self, hidden_states, encoder_hidden_states=None, attention_mask=None, rotary_emb=None):
        return self.processor(self, hidden_states, encoder_hidden_states=encoder_hidden_states,
                              attention_mask=attention_mask, rotary_emb=rotary_emb)


def rope_axis_dims(head_dim: int) -> Tuple[int, int, int]:
    hw = 2 * (head_dim // 6)
    return head_dim - 2 * hw, hw, hw


def wan_rope_table(grid: Tuple[int, int, int], head_dim: int = 128, theta: float = 10000.0,
                   device=None) -> torch.Tensor:
    """Complex rotary table ``[1, 1, F*H*W, head_dim/2]`` for a token grid (frames, rows, columns):
    head_dim split 44/42/42, pair i of an axis of width d rotates by ``pos * theta^(-2i/d)``."""
    f, h, w = grid
    parts = []
    for n, d, shape in zip(grid, rope_axis_dims(head_dim), ((f, 1, 1), (1, h, 1), (1, 1, w))):
        inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float64) / d))
        ang = torch.outer(torch.arange(n, dtype=torch.float64), inv)
        parts.append(torch.polar(torch.ones_like(ang), ang).view(*shape, d // 2).expand(f, h, w, d // 2))
    table = torch.cat(parts, dim=-1).reshape(1, 1, f * h * w, head_dim // 2)
    return table.to(device) if device is not None else table


class WanSelfAttentionStack(nn.Module):
    """``layers`` self-attention blocks applied in sequence (each with its own weights): the hot path
    of one DiT denoising step with everything around the attention block left out."""

    def __init__(self, layers: int, dim: int, heads: int):
        super().__init__()
        self.blocks = nn.ModuleList([Attention(dim, heads) for _ in range(layers)])

    def forward(self, hidden_states, rotary_emb=None):
        for blk in self.blocks:
            hidden_states = blk(hidden_states, rotary_emb=rotary_emb)
        return hidden_states


class _Pipe:
    """Stand-in for a diffusers pipeline: anything with a ``.transformer`` module."""

    def __init__(self, transformer: nn.Module):
        self.transformer = transformer


def init_wan_weights_(module: nn.Module, std: float = 0.02, seed: int = 0) -> None:
    """Seeded N(0, std) weights, zero bias, unit norm weights (the synthetic-weight recipe of the
    benchmark configurations)."""
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for m in module.modules():
            if isinstance(m, nn.Linear):
                m.weight.copy_(torch.randn(m.weight.shape, generator=g) * std)
                if m.bias is not None:
                    m.bias.zero_()
