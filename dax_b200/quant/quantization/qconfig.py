"""QConfig factories (mirrors ``dax/quant/quantization/qconfig.py``): a QConfig pairs an activation
observer constructor with a weight observer constructor.  The two per-token x per-channel factories
are the ones the CUDA linear executes; the per-tensor factories are accepted by the module swap but
their forward is rejected by ``dax_b200.quant.nn.dynamic.Linear``."""
from collections import namedtuple

import torch

from ..qscheme import per_channel_symmetric, per_tensor_symmetric, per_token_symmetric
from .observer import DynamicObserverPlaceholder, MinMaxObserver, PerChannelMinMaxObserver

QConfig = namedtuple("QConfig", ["activation", "weight"])


def get_dynamic_int8_per_token_act_per_channel_weight_qconfig(activation_dtype=torch.int8, weight_dtype=torch.int8):
    """INT8 per-token activations x INT8 per-output-channel weights (``qconfig.py:157-178``)."""
    return QConfig(
        activation=DynamicObserverPlaceholder.with_args(dtype=activation_dtype, qscheme=per_token_symmetric,
                                                        is_dynamic=True),
        weight=PerChannelMinMaxObserver.with_args(dtype=weight_dtype, qscheme=per_channel_symmetric))


def get_dynamic_fp8_per_token_act_per_channel_weight_qconfig(activation_dtype=torch.float8_e5m2,
                                                             weight_dtype=torch.float8_e4m3fn):
    """FP8 per-token activations x FP8 per-output-channel weights (``qconfig.py:85-106``).  The
    default activation dtype is e5m2 as in the reference; pass ``torch.float8_e4m3fn`` for e4m3."""
    return QConfig(
        activation=DynamicObserverPlaceholder.with_args(dtype=activation_dtype, qscheme=per_token_symmetric,
                                                        is_dynamic=True),
        weight=PerChannelMinMaxObserver.with_args(dtype=weight_dtype, qscheme=per_channel_symmetric))


def get_default_dynamic_int8_qconfig(activation_dtype=torch.int8, weight_dtype=torch.int8):
    return QConfig(
        activation=DynamicObserverPlaceholder.with_args(dtype=activation_dtype, qscheme=per_tensor_symmetric,
                                                        is_dynamic=True),
        weight=MinMaxObserver.with_args(dtype=weight_dtype, qscheme=per_tensor_symmetric))


def get_default_dynamic_fp8_qconfig(activation_dtype=torch.float8_e5m2, weight_dtype=torch.float8_e4m3fn):
    return QConfig(
        activation=DynamicObserverPlaceholder.with_args(dtype=activation_dtype, qscheme=per_tensor_symmetric,
                                                        is_dynamic=True),
        weight=MinMaxObserver.with_args(dtype=weight_dtype, qscheme=per_tensor_symmetric))
