"""Transformer-level adapters for a Wan DiT: the quantising module swap, and the forward that adds the
sequence-parallel split / gather and the TeaCache step skipping around the block stack (counterparts of
``quantize_transformer`` and ``replace_transformer`` in ``dax/adapters/wan/transformer_adapter.py:44-234``)."""
from __future__ import annotations

import types
from types import SimpleNamespace

import torch

from ... import ops
from ...cache import teacache
from ...parallel import dist as para_dist
from ...parallel.patches import wanx2_1_t2v as sp_patches
from ...quant.quantization import (
    get_dynamic_fp8_per_token_act_per_channel_weight_qconfig,
    get_dynamic_int8_per_token_act_per_channel_weight_qconfig,
    quantize_dynamic,
)


def quantize_transformer(transformer, dtype: str = "int8"):
    """Swap every ``nn.Linear`` of the transformer for the dynamic quantised Linear, except the
    condition embedder and the output projection (``transformer_adapter.py:227-234``).
    ``dtype``: "int8" (the reference's choice), "fp8_e4m3" or "fp8_e5m2" (activation format; FP8
    weights are e4m3)."""
    if dtype == "int8":
        cfg = get_dynamic_int8_per_token_act_per_channel_weight_qconfig()
    elif dtype in ("fp8", "fp8_e4m3"):
        cfg = get_dynamic_fp8_per_token_act_per_channel_weight_qconfig(activation_dtype=torch.float8_e4m3fn)
    elif dtype == "fp8_e5m2":
        cfg = get_dynamic_fp8_per_token_act_per_channel_weight_qconfig(activation_dtype=torch.float8_e5m2)
    else:
        raise ValueError(f"unknown linear dtype {dtype!r}")
    quantize_dynamic(transformer, {"": cfg, "condition_embedder": None, "proj_out": None})
    return transformer


def dit_forward(self, hidden_states, timestep, encoder_hidden_states, encoder_hidden_states_image=None,
                return_dict: bool = True, attention_kwargs=None):
    """One denoising forward of a Wan DiT (``new_forward``, ``transformer_adapter.py:51-179``): rotary table on
    the full latent, patch embedding, condition embedder, sequence split over the ranks, TeaCache decision,
    the block stack (or the cached residual), modulated output norm, output projection, gather, unpatchify."""
    batch, _, frames, height, width = hidden_states.shape
    p_t, p_h, p_w = self.config.patch_size
    grid = (frames // p_t, height // p_h, width // p_w)
    rotary_emb = self.rope(hidden_states)
    x = self.patch_embedding(hidden_states).flatten(2).transpose(1, 2)
    temb, timestep_proj, ctx, ctx_img = self.condition_embedder(timestep, encoder_hidden_states, encoder_hidden_states_image)
    timestep_proj = timestep_proj.unflatten(1, (6, -1))
    if ctx_img is not None:
        ctx = torch.concat([ctx_img, ctx], dim=1)
    sp = para_dist.parallel_state.is_enable_sequence_parallel()
    if sp:
        x = sp_patches.split(x, 1)

    if teacache.should_skip_forward_for_cached_states(self, timestep_proj=timestep_proj, temb=temb):
        x = teacache.retrieve_cached_states(self, x)
    else:
        caching = getattr(self, "enable_teacache", False)
        original = x.clone() if caching else None
        for block in self.blocks:
            x = block(x, ctx, timestep_proj, rotary_emb)
        if caching:
            teacache.maybe_cache_states(self, x, original)

    shift, scale = (self.scale_shift_table.float() + temb.float().unsqueeze(1)).chunk(2, dim=1)  # [B, 1, D] each
    if x.is_cuda and x.dtype in (torch.bfloat16, torch.float16):
        rows = [ops.layernorm_modulate_quant(x[b].contiguous(), eps=self.norm_out.eps, shift=shift[b, 0].contiguous(),
                                             scale=scale[b, 0].contiguous())[0] for b in range(batch)]
        x = rows[0].unsqueeze(0) if batch == 1 else torch.stack(rows, 0)
    else:
        x = (self.norm_out(x.float()) * (1 + scale) + shift).type_as(x)
    x = self.proj_out(x)
    if sp:
        x = sp_patches.gather(x, 1)
    x = x.reshape(batch, grid[0], grid[1], grid[2], p_t, p_h, p_w, -1).permute(0, 7, 1, 4, 2, 5, 3, 6)
    output = x.flatten(6, 7).flatten(4, 5).flatten(2, 3)
    return SimpleNamespace(sample=output) if return_dict else (output,)


def replace_transformer(transformer, cache_strategy=None, **cache_params):
    """Bind ``dit_forward`` on the transformer and install the step-cache settings on its class the way the
    reference does (``transformer_adapter.py:44-224``).  A transformer without ``patch_embedding`` (a bare
    stack of attention blocks) only gets the cache flags."""
    if getattr(transformer, "_is_parallelized", False):
        return transformer
    if hasattr(transformer, "patch_embedding") and hasattr(transformer, "condition_embedder"):
        transformer.forward = types.MethodType(dit_forward, transformer)
    if cache_strategy == "teacache":
        teacache.configure(transformer, teacache_thresh=cache_params.get("teacache_thresh", 0.1),
                           num_inference_steps=cache_params.get("num_inference_steps", 50))
    else:  # None or a strategy this build does not know: no step cache, as in the reference
        transformer.__class__.enable_teacache = False
    transformer._is_parallelized = True
    return transformer
