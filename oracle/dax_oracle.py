"""CPU restatement of DAX's Ulysses self-attention hot path.  TEST INFRASTRUCTURE ONLY.

This module is the checker for the CUDA library: only the test-suite, the smoke entry and the
CPU-baseline leg of the benchmark may import it.  Nothing in the product package does, and the
product never falls back to it.

Every function restates, in eager torch on the CPU, the arithmetic of one piece of the
reference (RiseAI-Sys/DAX); the reference location is cited per function as
``path:line`` inside that project.  The DAX-owned arithmetic (quantiser, weight quantisation,
INT8 linear, the all-to-all layouts, the O-projection micro-batching) is pinned bit-for-bit by
golden vectors produced from the reference's own code (``tests/golden/make_golden.py``).

PARITY UNPINNED for the third-party pieces, whose source is not part of the reference tree:
  * RMSNorm and the 3-D rotary table come from ``diffusers==0.33.1`` (``requirements.txt:6``);
    they are restated here from their published definition (RMS over the full hidden
    dimension with eps 1e-6 and a learned weight; head_dim 128 split 44/42/42 over
    (frame, height, width), theta 10000, interleaved pairs).
  * SageAttention (``thu-ml/SageAttention``, version string "2.1.1" at
    ``dax/adapters/wan/attn_adapter.py:33``) is restated from its published algorithm
    (K mean-smoothing, INT8 Q.K^T, FP8 P.V, fp32 accumulation); the contract for attention is
    the tolerance against fp32 SDPA, which is the reference's own ``TORCH_SDPA`` branch.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

FP32_EPS = torch.finfo(torch.float32).eps  # 1.1920929e-07, the reference's scale floor


# ----------------------------------------------------------------------------------------------
# dynamic activation quantiser
# ----------------------------------------------------------------------------------------------
def quantize_rowwise(x: torch.Tensor, target_dtype: torch.dtype) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-token symmetric quantisation of the last dimension.

    Follows ``dax/quant/nn/dynamic/functional.py:124-148`` (absmax and the division by qmax are
    done in the INPUT dtype, the floor is fp32 eps, the scale is then widened to fp32) and
    ``dax/quant/nn/quantized/functional.py:11-20`` (INT8: multiply by the fp32 reciprocal, round
    half to even, clamp to [-128, 127]; FP8: true division, clamp to +-max, round-to-nearest cast).
    Returns ``(q, scale)`` with ``scale`` shaped ``[..., 1]`` fp32.
    """
    assert x.dtype in (torch.float32, torch.float16, torch.bfloat16)
    if target_dtype == torch.int8:
        qmax = 127
    else:
        qmax = torch.finfo(target_dtype).max
    amax = x.abs().amax(dim=-1, keepdim=True)
    scale = amax / float(qmax)
    scale = torch.clamp(scale, min=FP32_EPS).to(torch.float32)
    if target_dtype == torch.int8:
        q = torch.clamp(torch.round(x * (1.0 / scale)), -128, 127).to(torch.int8)
    else:
        q = (x / scale).clamp(-qmax, qmax).to(target_dtype)
    return q, scale


# ----------------------------------------------------------------------------------------------
# load-time weight quantisation
# ----------------------------------------------------------------------------------------------
def quantize_weight(w: torch.Tensor, target_dtype: torch.dtype) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-output-channel symmetric weight quantisation.

    Follows ``dax/quant/quantization/observer.py:284-312`` (row min/max of the weight cast to
    fp32), ``observer.py:98-134`` (amax = max(-min, max); scale = max(amax / qmax, fp32 eps)) and
    ``dax/quant/nn/dynamic/linear.py:276-300`` (quantise the weight IN ITS OWN dtype against the
    fp32 scale).  Returns ``(qweight [N, K], weight_scale [1, N] fp32)``.
    """
    wf = w.detach().to(torch.float32)
    mn, mx = torch.aminmax(wf, dim=1)
    qmax = 127 if target_dtype == torch.int8 else torch.finfo(target_dtype).max
    amax = torch.max(-mn, mx)
    scale = torch.max(amax / float(qmax), torch.tensor([FP32_EPS]))
    s = scale.reshape(-1, 1)
    if target_dtype == torch.int8:
        q = torch.clamp(torch.round(w * (1.0 / s)), -128, 127).to(torch.int8)
    else:
        q = (w / s).clamp(-qmax, qmax).to(target_dtype)
    return q, scale.reshape(1, -1)


# ----------------------------------------------------------------------------------------------
# dynamic linears
# ----------------------------------------------------------------------------------------------
def int_matmul(qx: torch.Tensor, qw: torch.Tensor) -> torch.Tensor:
    """Exact int32 accumulators of ``qx [M,K] @ qw[N,K]^T`` (``linear.py:218-220``).

    Computed in float64 blocks (products of int8 are < 2^14 and K < 2^20, so every partial sum is
    exactly representable), which is orders of magnitude faster than torch's CPU int32 matmul.
    """
    return (qx.to(torch.float64) @ qw.to(torch.float64).T).to(torch.int32)


def linear_int8(x: torch.Tensor, qw: torch.Tensor, w_scale: torch.Tensor, bias: Optional[torch.Tensor],
                out_dtype: torch.dtype, return_parts: bool = False):
    """INT8 branch of the dynamic linear, ``dax/quant/nn/dynamic/linear.py:180-228``:
    quantise per token, int32 GEMM, ``(acc * s_x) * s_w`` in fp32 in that order, cast to the output
    dtype, then add the bias in the output dtype."""
    prev = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    qx, sx = quantize_rowwise(x2, torch.int8)
    acc = int_matmul(qx, qw)
    out = acc * sx.reshape(-1, 1)
    out = out * w_scale.reshape(1, -1)
    out = out.view(*prev, qw.shape[0])
    if out.dtype != out_dtype:
        out = out.to(out_dtype)
    if bias is not None:
        out = out + bias
    if return_parts:
        return out, qx, sx, acc
    return out


def linear_fp8(x: torch.Tensor, qw: torch.Tensor, w_scale: torch.Tensor, bias: Optional[torch.Tensor],
               out_dtype: torch.dtype, act_dtype: torch.dtype = torch.float8_e4m3fn):
    """FP8 branch, ``dax/quant/nn/dynamic/linear.py:145-178``.  The reference hands the quantised
    operands to a row-wise scaled matmul (fp32 accumulation, bf16 result, bias added inside); that
    library call has no CPU form, so the same contraction is written out: exact products of the
    FP8 values accumulated in fp32/fp64, times both scales, plus bias, rounded once to bf16."""
    prev = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    qx, sx = quantize_rowwise(x2, act_dtype)
    acc = (qx.to(torch.float64) @ qw.to(torch.float64).T).to(torch.float32)
    out = acc * sx.reshape(-1, 1) * w_scale.reshape(1, -1)
    if bias is not None:
        out = out + bias.to(torch.float32)
    out = out.to(torch.bfloat16).view(*prev, qw.shape[0])
    if out.dtype != out_dtype:
        out = out.to(out_dtype)
    return out


# ----------------------------------------------------------------------------------------------
# RMSNorm and the 3-D rotary embedding (published definitions; parity unpinned, see header)
# ----------------------------------------------------------------------------------------------
def rmsnorm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float = 1e-6) -> torch.Tensor:
    """RMS normalisation over the full last dimension, call sites
    ``dax/adapters/wan/attn_adapter.py:82-85,108-109,121-122``: variance in fp32, scale by
    ``rsqrt(var + eps)``, multiply by the learned weight, result in the input dtype."""
    xf = x.to(torch.float32)
    var = xf.pow(2).mean(-1, keepdim=True)
    y = xf * torch.rsqrt(var + eps)
    if weight is not None:
        y = y * weight.to(torch.float32)
    return y.to(x.dtype)


def rope_axis_dims(head_dim: int) -> Tuple[int, int, int]:
    """Split of head_dim over (frame, height, width): h = w = 2*(head_dim//6), frames take the
    rest.  128 -> 44/42/42."""
    hw = 2 * (head_dim // 6)
    return head_dim - 2 * hw, hw, hw


def rope_table(grid: Tuple[int, int, int], head_dim: int = 128, theta: float = 10000.0) -> torch.Tensor:
    """Complex rotary table ``[1, 1, F*H*W, head_dim/2]`` (complex128) in the layout the
    processor multiplies with (``attn_adapter.py:164-173``): token index = (f*H + h)*W + w; the
    first 22 complex pairs rotate with the frame index, the next 21 with the row, the last 21 with
    the column; pair i of an axis with dimension d has frequency theta^(-2i/d)."""
    f, h, w = grid
    dims = rope_axis_dims(head_dim)
    parts = []
    for n, d, shape in ((f, dims[0], (f, 1, 1)), (h, dims[1], (1, h, 1)), (w, dims[2], (1, 1, w))):
        inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float64) / d))
        ang = torch.outer(torch.arange(n, dtype=torch.float64), inv)  # [n, d/2]
        fr = torch.polar(torch.ones_like(ang), ang)
        parts.append(fr.view(*shape, d // 2).expand(f, h, w, d // 2))
    return torch.cat(parts, dim=-1).reshape(1, 1, f * h * w, head_dim // 2)


def apply_rotary_emb(x: torch.Tensor, freqs: torch.Tensor) -> torch.Tensor:
    """``attn_adapter.py:164-173``: float64 complex multiply on interleaved pairs, cast back."""
    xr = torch.view_as_complex(x.to(torch.float64).unflatten(-1, (-1, 2)))
    return torch.view_as_real(xr * freqs).flatten(-2, -1).type_as(x)


# ----------------------------------------------------------------------------------------------
# attention
# ----------------------------------------------------------------------------------------------
def sdpa_fp32(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_chunk: int = 2048) -> torch.Tensor:
    """Non-causal fp32 scaled-dot-product attention over ``[B, h, S, d]``: the reference's
    ``TORCH_SDPA`` branch (``attn_adapter.py:222-229``) evaluated in fp32, chunked over queries so
    that long sequences fit in host memory."""
    qf, kf, vf = q.float(), k.float(), v.float()
    out = torch.empty_like(qf)
    for s0 in range(0, q.shape[-2], q_chunk):
        out[..., s0:s0 + q_chunk, :] = F.scaled_dot_product_attention(
            qf[..., s0:s0 + q_chunk, :], kf, vf, attn_mask=None, dropout_p=0.0, is_causal=False)
    return out


def sage_attention_model(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, k_block: int = 128,
                         qk: str = "int8", pv: str = "fp8") -> torch.Tensor:
    """Numerical model of the quantised attention the CUDA kernel implements, for error budgeting:
    K minus its per-(head, channel) mean over the sequence; Q quantised per token and K per block of
    ``k_block`` tokens to INT8 (``qk="int8"``) or rounded to fp16 (``"f16"``); exact softmax in fp32;
    P scaled to the e4m3 range and V scaled per channel, both rounded to FP8 e4m3 (``pv="fp8"``) or
    fp16 (``"f16"``); fp32 accumulation.  Shapes ``[B, h, S, d]``; returns fp32."""
    qf, kf, vf = q.float(), k.float(), v.float()
    d = q.shape[-1]
    S = k.shape[-2]
    kf = kf - kf.mean(dim=-2, keepdim=True)
    qf = qf * (1.0 / math.sqrt(d))
    if qk == "int8":
        sq = qf.abs().amax(-1, keepdim=True).clamp_min(1e-20) / 127.0
        qf = torch.round(qf / sq).clamp(-127, 127) * sq
        pad = (-S) % k_block
        kp = F.pad(kf, (0, 0, 0, pad))
        kb = kp.unflatten(-2, (-1, k_block))
        sk = kb.abs().amax(dim=(-1, -2), keepdim=True).clamp_min(1e-20) / 127.0
        kf = (torch.round(kb / sk).clamp(-127, 127) * sk).flatten(-3, -2)[..., :S, :]
    else:
        qf, kf = qf.half().float(), kf.half().float()
    s = qf @ kf.transpose(-1, -2)
    p = torch.exp(s - s.amax(-1, keepdim=True))
    l = p.sum(-1, keepdim=True)
    if pv == "fp8":
        sv = vf.abs().amax(dim=-2, keepdim=True).clamp_min(1e-20) / 448.0
        o = ((p * 448.0).to(torch.float8_e4m3fn).float() @ (vf / sv).to(torch.float8_e4m3fn).float()) * sv / 448.0
    else:
        o = p.half().float() @ vf.half().float()
    return o / l


# ----------------------------------------------------------------------------------------------
# Ulysses layouts (pure index maps: what each rank must end up holding)
# ----------------------------------------------------------------------------------------------
def collect_tokens_ref(shards: Sequence[torch.Tensor], rank: int) -> torch.Tensor:
    """What rank ``rank`` holds after the sequence->head exchange
    (``dax/parallel/comm/all_to_all.py:26-54``; ``dax/parallel/patches/wanx2_1_t2v_opt/layer.py:30-50``):
    given every rank's ``[B, s, H, d]`` shard, the full sequence of the rank's own head group,
    ``global[:, :, rank*h:(rank+1)*h, :]``."""
    P = len(shards)
    h = shards[0].shape[2] // P
    return torch.cat([x[:, :, rank * h:(rank + 1) * h, :] for x in shards], dim=1).contiguous()


def collect_heads_ref(shards: Sequence[torch.Tensor], rank: int) -> torch.Tensor:
    """Inverse exchange (``comm/all_to_all.py:56-88``; ``layer.py:13-29``): every rank holds
    ``[B, S, h, d]`` (its heads, all tokens); rank ``rank`` ends with its own token block and every
    head, ``[B, s, H, d]``."""
    P = len(shards)
    s = shards[0].shape[1] // P
    return torch.cat([x[:, rank * s:(rank + 1) * s] for x in shards], dim=2).contiguous()


def micro_batch_indices(S: int, m: int, P: int) -> List[List[int]]:
    """Token indices of each O-projection micro-batch,
    ``dax/parallel/patches/wanx2_1_t2v_opt/micro_batch_layer.py:14-29``: micro-batch i takes, from
    every destination rank j's block, the i-th slice of ``S // (P*m)`` tokens."""
    bs = S // (P * m)
    out = []
    for i in range(m):
        idx: List[int] = []
        for j in range(P):
            start = i * bs + j * m * bs
            idx.extend(range(start, start + bs))
        out.append(idx)
    return out


# ----------------------------------------------------------------------------------------------
# the whole block, single process (P ranks emulated by slicing)
# ----------------------------------------------------------------------------------------------
class LayerWeights:
    """Quantised weights of one self-attention layer (what the module swap leaves behind)."""

    def __init__(self, wq, wk, wv, wo, bq, bk, bv, bo, norm_q_w, norm_k_w, weight_dtype=torch.int8,
                 act_dtype=torch.int8):
        self.act_dtype = act_dtype
        self.weight_dtype = weight_dtype
        self.q = quantize_weight(wq, weight_dtype) + (bq,)
        self.k = quantize_weight(wk, weight_dtype) + (bk,)
        self.v = quantize_weight(wv, weight_dtype) + (bv,)
        self.o = quantize_weight(wo, weight_dtype) + (bo,)
        self.norm_q_w = norm_q_w
        self.norm_k_w = norm_k_w

    def linear(self, which: str, x: torch.Tensor) -> torch.Tensor:
        qw, sw, b = getattr(self, which)
        if self.weight_dtype == torch.int8:
            return linear_int8(x, qw, sw, b, x.dtype)
        return linear_fp8(x, qw, sw, b, x.dtype, self.act_dtype)


def self_attention_block(x: torch.Tensor, lw: LayerWeights, heads: int, freqs: Optional[torch.Tensor],
                         attention: str = "sdpa") -> torch.Tensor:
    """``DAXWanAttnProcessor2_0.__call__`` for self-attention at world size 1
    (``dax/adapters/wan/attn_adapter.py:62-304``): Q/K/V dynamic linears, RMSNorm on Q and K over the
    full hidden dimension, split into heads, rotary embedding, attention, merge heads, O linear.
    ``attention`` selects fp32 SDPA ("sdpa", the reference's CPU-runnable backend) or the
    quantised-attention model ("sage")."""
    q = lw.linear("q", x)
    k = lw.linear("k", x)
    v = lw.linear("v", x)
    q = rmsnorm(q, lw.norm_q_w)
    k = rmsnorm(k, lw.norm_k_w)
    q = q.unflatten(2, (heads, -1)).transpose(1, 2)
    k = k.unflatten(2, (heads, -1)).transpose(1, 2)
    v = v.unflatten(2, (heads, -1)).transpose(1, 2)
    if freqs is not None:
        q = apply_rotary_emb(q, freqs)
        k = apply_rotary_emb(k, freqs)
    if attention == "sdpa":
        o = sdpa_fp32(q, k, v).to(q.dtype)
    else:
        o = sage_attention_model(q, k, v).to(q.dtype)
    o = o.transpose(1, 2).flatten(2, 3).type_as(q)
    return lw.linear("o", o)


# ----------------------------------------------------------------------------------------------
# metrics
# ----------------------------------------------------------------------------------------------
def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.double().flatten(), b.double().flatten()
    return float((a - b).norm() / b.norm().clamp_min(1e-300))


def cosine(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.double().flatten(), b.double().flatten()
    return float((a @ b) / (a.norm() * b.norm()).clamp_min(1e-300))


# ----------------------------------------------------------------------------------------------
# the rest of a Wan DiT block and the DiT step around the hot path (published architecture; the block
# itself is diffusers code called from dax/adapters/wan/transformer_adapter.py:130-136: parity unpinned)
# ----------------------------------------------------------------------------------------------
def layernorm(x: torch.Tensor, weight=None, bias=None, eps: float = 1e-6) -> torch.Tensor:
    """LayerNorm over the last dimension evaluated in fp32, result fp32."""
    xf = x.float()
    return F.layer_norm(xf, xf.shape[-1:], None if weight is None else weight.float(),
                        None if bias is None else bias.float(), eps)


class QuantLinear:
    """A float linear after the module swap: per-channel quantised weight + dynamic per-token activations."""

    def __init__(self, w: torch.Tensor, b: Optional[torch.Tensor], weight_dtype=torch.int8, act_dtype=torch.int8):
        self.qw, self.sw = quantize_weight(w, weight_dtype)
        self.b, self.weight_dtype, self.act_dtype = b, weight_dtype, act_dtype

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        if self.weight_dtype == torch.int8:
            return linear_int8(x, self.qw, self.sw, self.b, x.dtype)
        return linear_fp8(x, self.qw, self.sw, self.b, x.dtype, self.act_dtype)


def attention_block(x, ctx, lins, norm_q_w, norm_k_w, heads, freqs, eps=1e-6):
    """Self- (ctx None) or cross-attention with Q/K RMSNorm, optional RoPE, fp32 SDPA, O projection
    (``dax/adapters/wan/attn_adapter.py:62-304``); ``lins`` = (q, k, v, o) callables."""
    kv = x if ctx is None else ctx
    q = rmsnorm(lins[0](x), norm_q_w, eps).unflatten(2, (heads, -1)).transpose(1, 2)
    k = rmsnorm(lins[1](kv), norm_k_w, eps).unflatten(2, (heads, -1)).transpose(1, 2)
    v = lins[2](kv).unflatten(2, (heads, -1)).transpose(1, 2)
    if freqs is not None:
        q, k = apply_rotary_emb(q, freqs), apply_rotary_emb(k, freqs)
    o = sdpa_fp32(q, k, v).to(x.dtype).transpose(1, 2).flatten(2, 3)
    return lins[3](o)


def wan_block(h, ctx, temb6, table6, attn1, attn2, norm2_w, norm2_b, ffn_up, ffn_down, heads, freqs, eps=1e-6):
    """One Wan2.1 block.  ``temb6 [B,6,D]`` + ``table6 [1,6,D]`` give shift/scale/gate of the self-attention
    and of the FFN; ``attn1`` / ``attn2`` = (q, k, v, o, norm_q_w, norm_k_w)."""
    shift_msa, scale_msa, gate_msa, c_shift, c_scale, c_gate = (table6.float() + temb6.float()).chunk(6, dim=1)
    n = (layernorm(h, eps=eps) * (1 + scale_msa) + shift_msa).type_as(h)
    a = attention_block(n, None, attn1[:4], attn1[4], attn1[5], heads, freqs, eps)
    h = (h.float() + a * gate_msa).type_as(h)
    n = layernorm(h, norm2_w, norm2_b, eps).type_as(h)
    h = h + attention_block(n, ctx, attn2[:4], attn2[4], attn2[5], heads, None, eps)
    n = (layernorm(h, eps=eps) * (1 + c_scale) + c_shift).type_as(h)
    f = ffn_down(F.gelu(ffn_up(n), approximate="tanh"))
    return (h.float() + f.float() * c_gate).type_as(h)


def dit_forward(latent: torch.Tensor, timestep: torch.Tensor, text: torch.Tensor, sd: dict, *, heads: int,
                patch_size=(1, 2, 2), freq_dim: int = 256, weight_dtype=torch.int8, act_dtype=torch.int8,
                eps: float = 1e-6) -> torch.Tensor:
    """One denoising forward of a Wan-shaped DiT at world size 1, following ``new_forward``
    (``dax/adapters/wan/transformer_adapter.py:51-179``): rotary table on the full latent (``:84``), patch
    embedding as a strided convolution flattened to ``[B, S, D]`` (``:86-87``), condition embedder (``:89-97``:
    sinusoidal timestep features -> MLP -> ``temb``; SiLU + linear -> the six modulation vectors; text MLP), the
    block stack (``:130-136``) through ``wan_block``, the modulated output norm and projection (``:142-154``),
    unpatchify (``:159-170``).  ``sd`` maps the transformer's parameter names (diffusers' naming) to tensors;
    every linear inside the blocks is quantised the way ``quantize_transformer`` leaves it (``:227-234``), the
    condition embedder and ``proj_out`` stay float.  The module definitions themselves are diffusers code
    (absent from the reference tree): parity unpinned for them, see the header."""
    dt = latent.dtype
    B, _, f, h, w = latent.shape
    pt, ph, pw = patch_size
    grid = (f // pt, h // ph, w // pw)
    freqs = rope_table(grid)

    def lin(name, x):  # float linear: fp32 accumulate, rounded to the model dtype
        b = sd.get(name + ".bias")
        return F.linear(x.float(), sd[name + ".weight"].float(), None if b is None else b.float()).to(dt)

    def qlin(name):
        return QuantLinear(sd[name + ".weight"], sd.get(name + ".bias"), weight_dtype, act_dtype)

    x = F.conv3d(latent.float(), sd["patch_embedding.weight"].float(), sd["patch_embedding.bias"].float(),
                 stride=patch_size).to(dt).flatten(2).transpose(1, 2)
    half = freq_dim // 2
    fr = torch.exp(-math.log(10000.0) * torch.arange(half, dtype=torch.float32) / half)
    ang = timestep.float()[:, None] * fr[None]
    emb = torch.cat([torch.cos(ang), torch.sin(ang)], dim=-1).to(dt)
    temb = lin("condition_embedder.time_embedder.2", F.silu(lin("condition_embedder.time_embedder.0", emb)))
    timestep_proj = lin("condition_embedder.time_proj", F.silu(temb)).unflatten(1, (6, -1))
    ctx = lin("condition_embedder.text_embedder.2",
              F.gelu(lin("condition_embedder.text_embedder.0", text.to(dt)), approximate="tanh"))

    n_layers = 1 + max(int(k.split(".")[1]) for k in sd if k.startswith("blocks."))
    for i in range(n_layers):
        p = f"blocks.{i}."
        attn = lambda a: (qlin(p + a + ".to_q"), qlin(p + a + ".to_k"), qlin(p + a + ".to_v"), qlin(p + a + ".to_out.0"),
                          sd[p + a + ".norm_q.weight"], sd[p + a + ".norm_k.weight"])
        x = wan_block(x, ctx, timestep_proj, sd[p + "scale_shift_table"], attn("attn1"), attn("attn2"),
                      sd.get(p + "norm2.weight"), sd.get(p + "norm2.bias"), qlin(p + "ffn.net.0.proj"),
                      qlin(p + "ffn.net.2"), heads, freqs, eps)

    shift, scale = (sd["scale_shift_table"].float() + temb.float().unsqueeze(1)).chunk(2, dim=1)
    x = (layernorm(x, eps=eps) * (1 + scale) + shift).to(dt)
    x = lin("proj_out", x)
    x = x.reshape(B, grid[0], grid[1], grid[2], pt, ph, pw, -1).permute(0, 7, 1, 4, 2, 5, 3, 6)
    return x.flatten(6, 7).flatten(4, 5).flatten(2, 3)
