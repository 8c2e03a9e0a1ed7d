"""Transformer-level adapters: the quantising module swap for a Wan DiT and the hook that records
cache settings on the transformer (counterparts of ``quantize_transformer`` and
``replace_transformer`` in ``dax/adapters/wan/transformer_adapter.py:44-46,227-234``)."""
from __future__ import annotations

import torch

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


def replace_transformer(transformer, cache_strategy=None, **cache_params):
    """Record the step-cache settings on the transformer class the way the reference does
    (class attributes, ``transformer_adapter.py:183-222``) and mark it parallelised."""
    cls = transformer.__class__
    if cache_strategy == "teacache":
        cls.enable_teacache = True
        for k, v in cache_params.items():
            setattr(cls, k, v)
    elif cache_strategy is None:
        cls.enable_teacache = False
    else:
        raise ValueError(f"unknown cache_strategy {cache_strategy!r}")
    transformer._is_parallelized = True
    return transformer
