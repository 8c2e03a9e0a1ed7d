"""ctypes binding of ``libdax_b200.so`` (the C ABI declared in ``include/dax_b200.h``).

The product has no CPU path: if the library is missing the import of any operator fails loudly
with instructions to build it (``python -m dax_b200.build``).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_void_p, POINTER

from .build import library_path

DAX_OK, DAX_ERR_INVALID, DAX_ERR_ALIGN, DAX_ERR_UNSUPPORTED, DAX_ERR_CUDA, DAX_ERR_TIMEOUT = range(6)
DAX_BF16, DAX_F16, DAX_F32, DAX_I8, DAX_E4M3, DAX_E5M2 = range(6)
DAX_ATTN_QK_I8_PV_F8, DAX_ATTN_QK_BF16_PV_BF16, DAX_ATTN_QK_I8_PV_BF16 = 0, 1, 2

I64x3 = c_int64 * 3

# name -> (restype, argtypes): exactly the declarations of include/dax_b200.h
SIGNATURES = {
    "dax_version": (c_int, []),
    "dax_last_error": (c_char_p, []),
    "dax_device_status": (c_int, [POINTER(c_int)]),
    "dax_peer_copy": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p]),
    "dax_quant_rowwise": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int64, c_void_p, c_int,
                                  c_void_p, c_void_p]),
    "dax_gemm_dequant": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p,
                                 c_int, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p,
                                 c_void_p]),
    "dax_gemm_dequant_ex": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p,
                                    c_int, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p,
                                    c_int, c_void_p, c_int64, c_void_p, c_void_p]),
    "dax_gemm_dequant_scatter": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int,
                                         POINTER(c_void_p), c_int64, c_int, c_int64, c_int64, c_int64, c_int64, c_int64,
                                         c_void_p]),
    "dax_rmsnorm_rope_pack_scatter": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_int64, c_int,
                                              c_void_p, c_float, c_void_p, c_void_p, c_int64, POINTER(c_void_p), c_int64,
                                              c_int64, c_int64, c_void_p]),
    "dax_attn_forward_direct": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, I64x3, I64x3,
                                        I64x3, c_float, c_void_p, I64x3, POINTER(c_void_p), c_int64, c_int64, c_int64, c_int64,
                                        c_int64, c_int64, c_void_p]),
    "dax_attn_forward_scatter": (c_int, [POINTER(c_void_p), c_int64, c_int64, c_int, c_int64, c_int64, c_int64, c_int64,
                                         c_int64, c_int64, c_int64, c_int, c_void_p, c_size_t, c_void_p]),
    "dax_layernorm_modulate_quant": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p,
                                             c_void_p, c_float, c_void_p, c_int64, c_void_p, c_int, c_void_p, c_void_p]),
    "dax_linear_dynamic_workspace_bytes": (c_size_t, [c_int64, c_int64]),
    "dax_linear_dynamic": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                   c_int, c_void_p, c_int, c_int64, c_int64, c_void_p, c_size_t, c_void_p]),
    "dax_linear_dynamic_static": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_int, c_int, c_void_p,
                                          c_void_p, c_int, c_void_p, c_int, c_int64, c_int64, c_void_p]),
    "dax_rmsnorm_rope_pack": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_int64, c_int,
                                      c_void_p, c_float, c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int64,
                                      c_int64, c_void_p]),
    "dax_attn_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64, c_int64, c_int]),
    "dax_attn_prepare": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, I64x3,
                                 I64x3, I64x3, c_float, c_int, c_void_p, c_size_t, c_void_p]),
    "dax_attn_prepare_parts": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, I64x3,
                                       I64x3, I64x3, c_float, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "dax_attn_forward": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, I64x3, c_int64, c_int64,
                                 c_int64, c_int64, c_int, c_void_p, c_size_t, c_void_p]),
}

_LIB = None


class DaxLibraryError(RuntimeError):
    pass


def load() -> ctypes.CDLL:
    """Load the shared library (once) and attach the prototypes."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = library_path()
    if not os.path.exists(path):
        raise DaxLibraryError(
            f"{path} is missing: the CUDA library has not been built (run `python -m dax_b200.build`). "
            "dax_b200 has no CPU or eager fallback.")
    lib = ctypes.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export a declared symbol
        fn.restype = res
        fn.argtypes = args
    _LIB = lib
    return lib


_EXC = {DAX_ERR_INVALID: ValueError, DAX_ERR_ALIGN: ValueError, DAX_ERR_UNSUPPORTED: NotImplementedError,
        DAX_ERR_CUDA: RuntimeError, DAX_ERR_TIMEOUT: RuntimeError}


def check(status: int) -> None:
    """Turn a non-zero status into the Python exception type the reference raises for that class of
    problem (ValueError for bad arguments, NotImplementedError for unsupported combinations)."""
    if status != DAX_OK:
        msg = load().dax_last_error().decode("utf-8", "replace")
        raise _EXC.get(status, RuntimeError)(f"dax_b200 status {status}: {msg}")


def device_status() -> int:
    out = c_int(0)
    check(load().dax_device_status(ctypes.byref(out)))
    return out.value
