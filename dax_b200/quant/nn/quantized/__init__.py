from .functional import FP8_ALLOWED_DTYPES, quantize_to_fp8, quantize_to_int8
