from .qconfig import (
    QConfig,
    get_default_dynamic_fp8_qconfig,
    get_default_dynamic_int8_qconfig,
    get_dynamic_fp8_per_token_act_per_channel_weight_qconfig,
    get_dynamic_int8_per_token_act_per_channel_weight_qconfig,
)
from .quantize import propagate_qconfig_, quantize_dynamic, swap_module
