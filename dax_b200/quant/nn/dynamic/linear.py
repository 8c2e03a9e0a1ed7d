"""Dynamically quantised Linear: the module the swap installs in place of ``nn.Linear``.

Mirrors ``dax.quant.nn.dynamic.Linear`` (``dax/quant/nn/dynamic/linear.py:27-341``): same
constructor arguments, the same persistent buffers (``qweight [N, K]``, ``weight_scale [1, N]``
fp32) and ``bias`` parameter so that state dicts are interchangeable, the same ``from_float`` /
``get_qlinear`` load-time weight quantisation.  ``forward`` is two launches of the CUDA library:
the per-token quantiser and the tcgen05 GEMM with the de-quantisation, cast and bias in its
epilogue.  There is no float fallback and no CPU path: unsupported shapes raise."""
from __future__ import annotations

import torch
from torch import Tensor, nn

from ... import qscheme as _qs
from ..quantized.functional import FP8_ALLOWED_DTYPES, quantize_to_fp8, quantize_to_int8


class Linear(nn.Module):
    _FLOAT_MODULE = nn.Linear

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, weight_dtype=None,
                 input_dtype=None, out_dtype=None, weight_qscheme=None, input_qscheme=None) -> None:
        if weight_dtype in FP8_ALLOWED_DTYPES and input_dtype in FP8_ALLOWED_DTYPES:
            per_row = input_qscheme == _qs.per_token_symmetric and weight_qscheme == _qs.per_channel_symmetric
            per_tensor = input_qscheme == _qs.per_tensor_symmetric and weight_qscheme == _qs.per_tensor_symmetric
            if not (per_row or per_tensor):
                raise ValueError("Invalid qscheme combination! "
                                 f"input_qscheme: {input_qscheme}, weight_qscheme: {weight_qscheme}")
            compute_dtype = "FP8"
        elif weight_dtype == torch.int8 and input_dtype == torch.int8:
            compute_dtype = "INT8"
        else:
            raise ValueError(f"Unsupported dtype combination! weight_dtype: {weight_dtype}, input_dtype: {input_dtype}")
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.register_buffer("qweight", torch.empty((out_features, in_features), device=device, dtype=weight_dtype),
                             persistent=True)
        if bias:
            # the reference keeps an FP8 row-wise linear's bias in bf16 (linear.py:106-118)
            bias_dtype = (torch.bfloat16 if compute_dtype == "FP8" and weight_qscheme == _qs.per_channel_symmetric
                          else out_dtype)
            self.bias = nn.Parameter(torch.empty(out_features, device=device, dtype=bias_dtype))
        else:
            self.register_parameter("bias", None)
        scale_shape = (1, out_features) if weight_qscheme == _qs.per_channel_symmetric else 1
        self.register_buffer("weight_scale", torch.ones(scale_shape, device=device, dtype=torch.float32),
                             persistent=True)
        self.out_dtype = out_dtype
        self.weight_dtype = weight_dtype
        self.input_dtype = input_dtype
        self.compute_dtype = compute_dtype
        self.weight_qscheme = weight_qscheme
        self.input_qscheme = input_qscheme

    @property
    def weight(self) -> Tensor:
        """De-quantised weight (debugging aid, as in the reference)."""
        return self.qweight.to(self.out_dtype) * self.weight_scale.T.to(self.out_dtype)

    # -- hot path ------------------------------------------------------------------------------
    def _check_supported(self) -> None:
        if self.input_qscheme != _qs.per_token_symmetric or self.weight_qscheme != _qs.per_channel_symmetric:
            raise NotImplementedError(
                "dax_b200's CUDA linear implements per-token activations x per-channel weights "
                f"(got input_qscheme={self.input_qscheme}, weight_qscheme={self.weight_qscheme})")

    def quantize_input(self, input: Tensor):
        """Per-token quantisation of ``input`` viewed as ``[-1, in_features]`` -> (q, scale)."""
        from ....ops import quant_rowwise
        return quant_rowwise(input.reshape(-1, self.in_features), self.input_dtype)

    def forward_quantized(self, qinput: Tensor, input_scale: Tensor, **gemm_kwargs) -> Tensor:
        """GEMM + de-quantisation on already quantised rows (lets callers share one quantisation
        between several projections of the same activations, and redirect the output layout)."""
        from ....ops import gemm_dequant
        return gemm_dequant(qinput, input_scale, self.qweight, self.weight_scale.reshape(-1), self.bias,
                            self.out_dtype, **gemm_kwargs)

    def forward(self, input: Tensor) -> Tensor:
        self._check_supported()
        if not input.is_cuda:
            raise RuntimeError("dax_b200.quant.nn.dynamic.Linear runs on CUDA only; there is no CPU fallback")
        from ....ops import linear_dynamic
        prev_dims = input.shape[:-1]
        x2 = input.reshape(-1, self.in_features)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        out = linear_dynamic(x2, self.qweight, self.weight_scale.reshape(-1), self.bias, self.input_dtype,
                             self.out_dtype)
        return out.view(*prev_dims, self.out_features)

    def extra_repr(self) -> str:
        s = f"in_features={self.in_features}, out_features={self.out_features}"
        if self.bias is None:
            s += ", bias=False"
        return s + f", compute_dtype={self.compute_dtype}"

    # -- load-time conversion --------------------------------------------------------------------
    @classmethod
    @torch.no_grad()
    def get_qlinear(cls, mod, activation_post_process, weight_post_process, reserve_float_weight):
        """Build the quantised module from a float ``nn.Linear`` and the two observers
        (``dax/quant/nn/dynamic/linear.py:240-307``)."""
        if activation_post_process is None or activation_post_process.dtype == torch.float:
            raise ValueError("Input must be quantized!")
        qlinear = cls(mod.in_features, mod.out_features, mod.bias is not None, mod.weight.device,
                      weight_post_process.dtype, activation_post_process.dtype, mod.weight.dtype,
                      weight_post_process.qscheme, activation_post_process.qscheme)
        weight_post_process(mod.weight)
        if weight_post_process.dtype in FP8_ALLOWED_DTYPES:
            quantize_func = quantize_to_fp8
        elif weight_post_process.dtype == torch.int8:
            quantize_func = quantize_to_int8
        else:
            raise NotImplementedError(f"Unsupported dtype {weight_post_process.dtype}")
        weight_scale = weight_post_process.calculate_qparams()
        if weight_scale is not None:
            if weight_post_process.qscheme == _qs.per_channel_symmetric:
                assert mod.weight.shape[0] == weight_scale.numel()
                weight_scale = weight_scale.reshape([mod.weight.shape[0]] + [1] * (mod.weight.ndim - 1))
            qlinear.qweight = quantize_func(mod.weight, scale=weight_scale, dtype=weight_post_process.dtype).contiguous()
            qlinear.weight_scale.copy_(weight_scale.reshape(qlinear.weight_scale.shape))
        if qlinear.bias is not None:
            qlinear.bias.copy_(mod.bias)
        if not reserve_float_weight:  # release the float weight's device memory
            del mod.weight
            del mod.bias
        return qlinear

    @classmethod
    def from_float(cls, mod, reserve_float_weight=False):
        assert type(mod) == cls._FLOAT_MODULE, (
            f"nnq.{cls.__name__}.from_float only works for {cls._FLOAT_MODULE.__name__} but got: {type(mod)}")
        assert hasattr(mod, "qconfig"), "Input float module must have qconfig defined."
        return cls.get_qlinear(mod, mod.qconfig.activation(), mod.qconfig.weight(), reserve_float_weight)
