"""Observers used by the dynamic-quantisation module swap.

Only what the dynamic path needs is here: a per-channel and a per-tensor min/max observer for the
WEIGHTS (run once at load time) and the no-op placeholder that carries the activation dtype and
scheme.  Scale computation follows ``dax/quant/quantization/observer.py:98-134``:
``amax = max(-min, max)``, ``scale = max(amax / qmax, fp32 eps)``.  The reference's static
calibration tooling (running activation observers, histogram profiling, cross-rank min/max
all-reduce) is offline tooling outside the hot path and is not provided."""
from __future__ import annotations

import functools

import torch
from torch import nn

from ..qscheme import per_channel_symmetric, per_tensor_symmetric, per_token_symmetric

ALLOWED_DTYPES = (torch.float8_e4m3fn, torch.float8_e5m2, torch.int8)
FP32_EPS = torch.finfo(torch.float32).eps


class _WithArgs:
    """``Observer.with_args(**kw)`` -> a constructor with those keyword arguments bound."""

    def __init__(self, cls, **kwargs):
        self.p = functools.partial(cls, **kwargs)

    def __call__(self, *args, **kwargs):
        return self.p(*args, **kwargs)

    def with_args(self, **kwargs):
        return _WithArgs(self.p.func, **{**self.p.keywords, **kwargs})

    def __repr__(self):
        return f"{self.p.func.__name__}.with_args({self.p.keywords})"


class UniformQuantizationObserverBase(nn.Module):
    def __init__(self, dtype=torch.float8_e4m3fn, qscheme=per_tensor_symmetric, eps=FP32_EPS, is_dynamic=False,
                 factory_kwargs=None, **kwargs) -> None:
        super().__init__()
        assert qscheme in (per_tensor_symmetric, per_channel_symmetric, per_token_symmetric), (
            "observers support per_tensor_symmetric / per_channel_symmetric / per_token_symmetric only")
        assert dtype in ALLOWED_DTYPES, f"observers support {ALLOWED_DTYPES} only"
        self.dtype = dtype
        self.qscheme = qscheme
        self.is_dynamic = is_dynamic
        self.quant_max = 127 if dtype == torch.int8 else torch.finfo(dtype).max
        self.register_buffer("eps", torch.tensor([eps], **(factory_kwargs or {})))

    @classmethod
    def with_args(cls, **kwargs):
        return _WithArgs(cls, **kwargs)

    def _calculate_qparams(self, min_val: torch.Tensor, max_val: torch.Tensor):
        if min_val.numel() == 0 or max_val.numel() == 0 or bool((min_val > max_val).any()):
            return None
        amax = torch.max(-min_val, max_val)
        scale = torch.max(amax / float(self.quant_max), self.eps.to(amax.device))
        if scale.dim() == 0:
            scale = scale.reshape(1)
        return scale


class MinMaxObserver(UniformQuantizationObserverBase):
    """Per-tensor running min/max."""

    def __init__(self, **kwargs) -> None:
        kwargs.pop("sync_state", None)
        super().__init__(**kwargs)
        if self.qscheme != per_tensor_symmetric:
            raise NotImplementedError("MinMaxObserver supports per_tensor_symmetric only")
        self.register_buffer("min_val", torch.tensor(float("inf")))
        self.register_buffer("max_val", torch.tensor(float("-inf")))

    def forward(self, x_orig):
        if x_orig.numel() == 0:
            return x_orig
        x = x_orig.detach().to(torch.float32)
        mn, mx = torch.aminmax(x)
        self.min_val = torch.min(mn, self.min_val.to(mn.device))
        self.max_val = torch.max(mx, self.max_val.to(mx.device))
        return x_orig

    def calculate_qparams(self):
        return self._calculate_qparams(self.min_val, self.max_val)


class PerChannelMinMaxObserver(UniformQuantizationObserverBase):
    """Running min/max per slice of ``ch_axis`` (``observer.py:284-312``)."""

    def __init__(self, ch_axis=0, **kwargs) -> None:
        super().__init__(**kwargs)
        if self.qscheme != per_channel_symmetric:
            raise NotImplementedError("PerChannelMinMaxObserver supports per_channel_symmetric only")
        self.ch_axis = ch_axis
        self.register_buffer("min_val", torch.tensor([]))
        self.register_buffer("max_val", torch.tensor([]))

    def forward(self, x_orig):
        if x_orig.numel() == 0:
            return x_orig
        y = x_orig.detach().transpose(0, self.ch_axis).to(torch.float32).flatten(1)
        mn, mx = torch.aminmax(y, dim=1)
        if self.min_val.numel() != 0:
            mn = torch.min(mn, self.min_val.to(mn.device))
            mx = torch.max(mx, self.max_val.to(mx.device))
        self.min_val, self.max_val = mn, mx
        return x_orig

    def calculate_qparams(self):
        return self._calculate_qparams(self.min_val, self.max_val)


class DynamicObserverPlaceholder(UniformQuantizationObserverBase):
    """Carries dtype and scheme of a dynamically quantised activation; observes nothing
    (``observer.py:453-477``)."""

    def __init__(self, **kwargs) -> None:
        kwargs.setdefault("is_dynamic", True)
        super().__init__(**kwargs)

    def forward(self, x):
        return x

    def calculate_qparams(self):
        raise RuntimeError("calculate_qparams should not be called for a dynamic placeholder")
