"""Dynamic INT8 / FP8 quantisation of linears (counterpart of ``dax.quant``)."""
from . import nn, quantization
from .qscheme import per_channel_symmetric, per_tensor_symmetric, per_token_symmetric
