"""Quantisation scheme names and their block shapes (mirrors ``dax/quant/qscheme.py:5-26``).

The strings are kept identical to the reference's so that qconfigs and state dicts move between
the two packages unchanged."""
from typing import Tuple, Union

import torch

per_tensor_symmetric = "dax.quant.per_tensor_symmetric"
per_token_symmetric = "dax.quant.per_token_symmetric"
per_channel_symmetric = "dax.quant.per_channel_symmetric"

FP8_QSCHEME = [per_tensor_symmetric, per_token_symmetric, per_channel_symmetric]
INT8_QSCHEME = [per_tensor_symmetric, per_token_symmetric, per_channel_symmetric]


def get_block_size(input_shape: Tuple[int, ...], qscheme: Union[str, torch.qscheme]) -> Tuple[int, ...]:
    """Shape of the block of elements that shares one scale."""
    shape = tuple(input_shape)
    if qscheme == per_tensor_symmetric:
        return shape
    if qscheme == per_token_symmetric:
        return (1,) * (len(shape) - 1) + (shape[-1],)
    if qscheme == per_channel_symmetric:
        return shape[:-1] + (1,)
    raise ValueError(f"Unsupported QScheme: {qscheme}")
