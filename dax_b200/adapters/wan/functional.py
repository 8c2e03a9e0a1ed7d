"""``optimize_pipe``: the one public call that wires sequence parallelism, quantised linears and the
attention processor into a pipeline (``dax/adapters/wan/functional.py:10-41``)."""
from __future__ import annotations

import logging

from ...parallel.initialize import initialize
from .attn_adapter import replace_wan_attention
from .block_adapter import replace_wan_blocks
from .transformer_adapter import quantize_transformer, replace_transformer

log = logging.getLogger("dax_b200")


def optimize_pipe(pipe, sequence_parallel=True, compile=True, overlap_comm=True, int8_linear=False,
                  cache_strategy=None, fp8_linear=False, attention_mode="bf16", fuse_blocks=True, **cache_params):
    """Same switches as the reference.  ``compile`` is accepted for signature compatibility and has
    no effect: every kernel is precompiled CUDA, nothing is traced.  ``attention_mode``: precision of the attention kernel's two contractions, "bf16" (default, within
    rel-L2 1e-2 of fp32 SDPA), "sage" (INT8 Q.K^T + FP8 P.V, what the reference's SAGE_ATTN backend computes) or
    "int8_bf16".  ``fp8_linear`` (not in the
    reference's signature, where FP8 is reachable only through ``quantize_dynamic``) selects e4m3
    activations x e4m3 weights; ``fuse_blocks`` binds the fused CUDA forward on every Wan block (LayerNorm /
    modulation / GELU / gated residuals ride in the quantiser and GEMM kernels)."""
    sp_size = 1
    if sequence_parallel:
        sp_size = initialize()
    replace_transformer(pipe.transformer, cache_strategy, **cache_params)
    if int8_linear and fp8_linear:
        raise ValueError("int8_linear and fp8_linear are mutually exclusive")
    if int8_linear:
        quantize_transformer(pipe.transformer, "int8")
    elif fp8_linear:
        quantize_transformer(pipe.transformer, "fp8_e4m3")
    if overlap_comm and not sequence_parallel:
        raise ValueError("Overlap communication is only valid in SP mode")
    replace_wan_attention(pipe, sp_size if sequence_parallel else 1, overlap_comm=overlap_comm,
                          attention_mode=attention_mode)
    if fuse_blocks:
        replace_wan_blocks(pipe)
    if compile:
        log.info("optimize_pipe(compile=True): ignored, dax_b200 runs precompiled CUDA kernels")
    return pipe
