"""Static quantisation primitives used at LOAD time for weights (and by the per-tensor schemes).

Same arithmetic as ``dax/quant/nn/quantized/functional.py:11-20``.  These run as ordinary torch
ops wherever the weight lives; the per-token activation path of the hot loop does not come through
here, it is the CUDA quantiser (``dax_b200.ops.quant_rowwise``)."""
import torch
from torch import Tensor

FP8_ALLOWED_DTYPES = (torch.float8_e4m3fn, torch.float8_e5m2)


def quantize_to_fp8(x: Tensor, scale: Tensor, dtype: torch.dtype) -> Tensor:
    limit = torch.finfo(dtype).max
    return (x / scale).clamp(-limit, limit).to(dtype)


def quantize_to_int8(x: Tensor, scale: Tensor, dtype: torch.dtype = torch.int8) -> Tensor:
    info = torch.iinfo(dtype)
    return torch.clamp(torch.round(x * (1.0 / scale)), info.min, info.max).to(dtype)
