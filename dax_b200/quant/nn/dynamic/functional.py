"""Dynamic (per-call) activation quantisation: the functional face of the CUDA quantiser.

Mirrors the entry points of ``dax/quant/nn/dynamic/functional.py:152-206``.  Per-token symmetric
quantisation of a CUDA tensor is one launch of ``dax_quant_rowwise``; the other schemes of the
reference (per-tensor, per-channel activations) are not on the Wan hot path and are rejected."""
from typing import List, Optional, Tuple

import torch

from ... import qscheme as _qs
from ....ops import quant_rowwise
from ..quantized.functional import FP8_ALLOWED_DTYPES


def _per_token(input_float: torch.Tensor, qscheme, block_size, target_dtype) -> Tuple[torch.Tensor, torch.Tensor]:
    if block_size is None:
        block_size = _qs.get_block_size(input_float.shape, qscheme)
    if tuple(block_size) != _qs.get_block_size(input_float.shape, _qs.per_token_symmetric):
        raise NotImplementedError(
            "dax_b200 quantises activations per token only (the scheme the Wan adapter selects); "
            f"got block_size={tuple(block_size)} for input of shape {tuple(input_float.shape)}")
    q, scale = quant_rowwise(input_float, target_dtype)
    return q.view(input_float.shape), scale.view(*input_float.shape[:-1], 1)


def dynamic_quantize_to_int8(input_float: torch.Tensor, qscheme: str = _qs.per_token_symmetric,
                             block_size: Optional[List[int]] = None,
                             target_dtype: Optional[torch.dtype] = torch.int8,
                             scale_dtype: Optional[torch.dtype] = torch.float32):
    if target_dtype != torch.int8:
        raise NotImplementedError(f"Unsupported dtype {target_dtype} for dynamic_quantize_to_int8")
    return _per_token(input_float, qscheme, block_size, target_dtype)


def dynamic_quantize_to_fp8(input_float: torch.Tensor, qscheme: str = _qs.per_token_symmetric,
                            block_size: Optional[List[int]] = None,
                            target_dtype: Optional[torch.dtype] = torch.float8_e4m3fn,
                            scale_dtype: Optional[torch.dtype] = torch.float32):
    if target_dtype not in FP8_ALLOWED_DTYPES:
        raise NotImplementedError(f"Unsupported dtype {target_dtype} for dynamic_quantize_to_fp8")
    return _per_token(input_float, qscheme, block_size, target_dtype)
