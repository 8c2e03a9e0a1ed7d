"""Module swap: float ``nn.Linear`` -> dynamically quantised Linear.

Same contract as ``dax.quant.quantization.quantize_dynamic`` (``dax/quant/quantization/quantize.py:394-444``):
``qconfig_dict`` maps a module-name prefix (``""`` = the root) or a module type to a QConfig or to
``None``; a module takes the entry of its own name if there is one, else its type's, else its
parent's; ``None`` leaves the module (and, by inheritance, its children) in float."""
from __future__ import annotations

import copy
from typing import Any, Dict, Optional

from torch import nn

from .quantization_mappings import get_default_dynamic_quant_module_mappings

_UNSET = object()


def propagate_qconfig_(module: nn.Module, qconfig_dict: Optional[Dict[Any, Any]] = None) -> None:
    """Attach a ``qconfig`` attribute to every module of the tree (``quantize.py:42-120``)."""
    qconfig_dict = qconfig_dict or {}

    def visit(mod: nn.Module, parent_cfg, prefix: str) -> None:
        cfg = qconfig_dict.get(type(mod), parent_cfg)
        cfg = qconfig_dict.get(prefix, cfg)
        cfg = getattr(mod, "qconfig", cfg)
        mod.qconfig = cfg
        for name, child in mod.named_children():
            visit(child, cfg, f"{prefix}.{name}" if prefix else name)

    visit(module, None, "")


def swap_module(mod: nn.Module, mapping, reserve_float_weight: bool = False) -> nn.Module:
    """Quantised counterpart of ``mod`` if it has a qconfig and a mapping entry, else ``mod``
    (``quantize.py:470-508``).  Forward hooks and pre-hooks move over; the device is kept."""
    cfg = getattr(mod, "qconfig", None)
    if cfg is None or type(mod) not in mapping:
        return mod
    devices = {p.device for p in mod.parameters()} | {b.device for b in mod.buffers()}
    assert len(devices) <= 1, f"swap_module only works with single-device modules, got {devices}"
    new_mod = mapping[type(mod)].from_float(mod, reserve_float_weight)
    for hook in mod._forward_pre_hooks.values():
        new_mod.register_forward_pre_hook(hook)
    for hook in mod._forward_hooks.values():
        new_mod.register_forward_hook(hook)
    if devices:
        new_mod.to(next(iter(devices)))
    return new_mod


def _convert(module: nn.Module, mapping) -> nn.Module:
    for name, child in list(module.named_children()):
        _convert(child, mapping)
        module._modules[name] = swap_module(child, mapping)
    return module


def _remove_qconfig(module: nn.Module) -> None:
    for m in module.modules():
        if hasattr(m, "qconfig"):
            del m.qconfig


def quantize_dynamic(model: nn.Module, qconfig_dict=None, mapping=None, inplace: bool = True,
                     remove_qconfig: bool = True) -> nn.Module:
    """Replace every mapped module that ends up with a non-``None`` qconfig by its dynamically
    quantised version (weights are quantised here, once; the float weights are released)."""
    if mapping is None:
        mapping = get_default_dynamic_quant_module_mappings()
    if not inplace:
        model = copy.deepcopy(model)
    propagate_qconfig_(model, qconfig_dict)
    _convert(model, mapping)
    if remove_qconfig:
        _remove_qconfig(model)
    return model
