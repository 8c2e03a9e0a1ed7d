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


# ----------------------------------------------------------------------------------------------
# Wan2.1 DiT block and model (stand-ins with the published architecture and diffusers' parameter names)
# ----------------------------------------------------------------------------------------------
class _GELUProj(nn.Module):
    """First FFN linear followed by tanh-GELU (parameter name ``proj``)."""

    def __init__(self, dim: int, inner: int):
        super().__init__()
        self.proj = nn.Linear(dim, inner, bias=True)

    def forward(self, x):
        return torch.nn.functional.gelu(self.proj(x), approximate="tanh")


class FeedForward(nn.Module):
    """``net.0.proj`` (dim -> inner, tanh-GELU), ``net.1`` dropout, ``net.2`` (inner -> dim)."""

    def __init__(self, dim: int, inner: int):
        super().__init__()
        self.net = nn.ModuleList([_GELUProj(dim, inner), nn.Dropout(0.0), nn.Linear(inner, dim, bias=True)])

    def forward(self, x):
        for m in self.net:
            x = m(x)
        return x


class FP32LayerNorm(nn.LayerNorm):
    def forward(self, x):
        return torch.nn.functional.layer_norm(x.float(), self.normalized_shape,
                                              self.weight.float() if self.weight is not None else None,
                                              self.bias.float() if self.bias is not None else None, self.eps).to(x.dtype)


class WanTransformerBlock(nn.Module):
    """One Wan2.1 block: adaLN-modulated self-attention with a gated residual, cross-attention over the text
    context (affine LayerNorm in front), adaLN-modulated tanh-GELU FFN with a gated residual.  ``forward`` is
    the plain torch composition (what runs before ``optimize_pipe`` replaces it by the fused CUDA path)."""

    def __init__(self, dim: int, ffn_dim: int, heads: int, eps: float = 1e-6):
        super().__init__()
        self.norm1 = FP32LayerNorm(dim, eps, elementwise_affine=False)
        self.attn1 = Attention(dim, heads, eps=eps)
        self.attn2 = Attention(dim, heads, eps=eps)
        self.norm2 = FP32LayerNorm(dim, eps, elementwise_affine=True)
        self.ffn = FeedForward(dim, ffn_dim)
        self.norm3 = FP32LayerNorm(dim, eps, elementwise_affine=False)
        self.scale_shift_table = nn.Parameter(torch.randn(1, 6, dim) / dim ** 0.5)

    def forward(self, hidden_states, encoder_hidden_states, temb, rotary_emb):
        shift_msa, scale_msa, gate_msa, c_shift, c_scale, c_gate = (self.scale_shift_table.float() + temb.float()).chunk(6, dim=1)
        h = hidden_states
        n = (self.norm1(h.float()) * (1 + scale_msa) + shift_msa).type_as(h)
        a = self.attn1(n, rotary_emb=rotary_emb)
        h = (h.float() + a * gate_msa).type_as(h)
        n = self.norm2(h.float()).type_as(h)
        h = h + self.attn2(n, encoder_hidden_states=encoder_hidden_states)
        n = (self.norm3(h.float()) * (1 + c_scale) + c_shift).type_as(h)
        f = self.ffn(n)
        return (h.float() + f.float() * c_gate).type_as(h)


class _TimeTextEmbedding(nn.Module):
    """Timestep (sinusoidal -> MLP), its 6-way projection for adaLN, and the text-context MLP."""

    def __init__(self, dim: int, freq_dim: int, text_dim: int):
        super().__init__()
        self.freq_dim = freq_dim
        self.time_embedder = nn.Sequential(nn.Linear(freq_dim, dim), nn.SiLU(), nn.Linear(dim, dim))
        self.act_fn = nn.SiLU()
        self.time_proj = nn.Linear(dim, dim * 6)
        self.text_embedder = nn.Sequential(nn.Linear(text_dim, dim), nn.GELU(approximate="tanh"), nn.Linear(dim, dim))

    def forward(self, timestep, encoder_hidden_states, encoder_hidden_states_image=None):
        half = self.freq_dim // 2
        freqs = torch.exp(-math.log(10000.0) * torch.arange(half, dtype=torch.float32, device=timestep.device) / half)
        ang = timestep.float()[:, None] * freqs[None]
        emb = torch.cat([torch.cos(ang), torch.sin(ang)], dim=-1)
        dt = self.time_embedder[0].weight.dtype
        temb = self.time_embedder(emb.to(dt))
        timestep_proj = self.time_proj(self.act_fn(temb))
        return temb, timestep_proj, self.text_embedder(encoder_hidden_states.to(dt)), None


class _Config:
    def __init__(self, **kw):
        self.__dict__.update(kw)


class WanDiT(nn.Module):
    """Wan2.1-shaped video DiT: 3-D patch embedding, condition embedder, ``layers`` blocks, modulated output
    norm and projection, unpatchify.  ``forward(hidden_states [B,C,F,H,W], timestep [B], encoder_hidden_states
    [B,L,text_dim])`` returns the denoiser output ``[B,C,F,H,W]``; this is the plain single-GPU torch path,
    ``replace_transformer`` installs the sequence-parallel / step-cache aware one."""

    def __init__(self, layers: int = 40, dim: int = 5120, ffn_dim: int = 13824, heads: int = 40, in_channels: int = 16,
                 out_channels: int = 16, patch_size=(1, 2, 2), text_dim: int = 4096, freq_dim: int = 256, eps: float = 1e-6):
        super().__init__()
        self.config = _Config(patch_size=tuple(patch_size), num_layers=layers, num_attention_heads=heads,
                              attention_head_dim=dim // heads, in_channels=in_channels, out_channels=out_channels)
        self.patch_embedding = nn.Conv3d(in_channels, dim, kernel_size=patch_size, stride=patch_size)
        self.condition_embedder = _TimeTextEmbedding(dim, freq_dim, text_dim)
        self.blocks = nn.ModuleList([WanTransformerBlock(dim, ffn_dim, heads, eps) for _ in range(layers)])
        self.norm_out = FP32LayerNorm(dim, eps, elementwise_affine=False)
        self.proj_out = nn.Linear(dim, out_channels * math.prod(patch_size))
        self.scale_shift_table = nn.Parameter(torch.randn(1, 2, dim) / dim ** 0.5)
        self.gradient_checkpointing = False

    def rope(self, hidden_states: torch.Tensor) -> torch.Tensor:
        _, _, f, h, w = hidden_states.shape
        pt, ph, pw = self.config.patch_size
        key = ((f // pt, h // ph, w // pw), str(hidden_states.device))
        cache = self.__dict__.setdefault("_rope_cache", {})
        if key not in cache:  # the table depends on the token grid only: build and upload it once
            cache.clear()
            cache[key] = wan_rope_table(key[0], self.config.attention_head_dim, device=hidden_states.device)
        return cache[key]

    def unpatchify(self, x: torch.Tensor, batch: int, grid) -> torch.Tensor:
        pt, ph, pw = self.config.patch_size
        f, h, w = grid
        x = x.reshape(batch, f, h, w, pt, ph, pw, -1).permute(0, 7, 1, 4, 2, 5, 3, 6)
        return x.flatten(6, 7).flatten(4, 5).flatten(2, 3)

    def forward(self, hidden_states, timestep, encoder_hidden_states, encoder_hidden_states_image=None,
                return_dict: bool = False, attention_kwargs=None):
        b, _, f, h, w = hidden_states.shape
        pt, ph, pw = self.config.patch_size
        grid = (f // pt, h // ph, w // pw)
        rotary_emb = self.rope(hidden_states)
        x = self.patch_embedding(hidden_states).flatten(2).transpose(1, 2)
        temb, timestep_proj, ctx, _ = self.condition_embedder(timestep, encoder_hidden_states)
        timestep_proj = timestep_proj.unflatten(1, (6, -1))
        for blk in self.blocks:
            x = blk(x, ctx, timestep_proj, rotary_emb)
        shift, scale = (self.scale_shift_table.float() + temb.float().unsqueeze(1)).chunk(2, dim=1)
        x = (self.norm_out(x.float()) * (1 + scale) + shift).type_as(x)
        out = self.unpatchify(self.proj_out(x), b, grid)
        return (out,)
