"""Float module type -> quantised module type (``dax/quant/quantization/quantization_mappings.py:21-23``)."""
import copy
from typing import Any, Callable, Dict

from torch import nn

from ..nn import dynamic as nndq

DEFAULT_DYNAMIC_QUANT_MODULE_MAPPINGS: Dict[Callable, Any] = {nn.Linear: nndq.Linear}


def get_default_dynamic_quant_module_mappings() -> Dict[Callable, Any]:
    return copy.copy(DEFAULT_DYNAMIC_QUANT_MODULE_MAPPINGS)
