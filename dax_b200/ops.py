"""Tensor-level wrappers over the C ABI: one function per kernel family.

These take CUDA ``torch.Tensor`` arguments, validate device/dtype/contiguity, allocate outputs with
torch (the library itself never allocates) and enqueue on the current CUDA stream.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import I64x3, check, load

_DT = {torch.bfloat16: _lib.DAX_BF16, torch.float16: _lib.DAX_F16, torch.float32: _lib.DAX_F32,
       torch.int8: _lib.DAX_I8, torch.float8_e4m3fn: _lib.DAX_E4M3, torch.float8_e5m2: _lib.DAX_E5M2}

# "bf16" (alias "f16", the default): bf16 contractions; the mode that meets rel-L2 <= 1e-2 against fp32 SDPA;
# "sage": INT8 Q.K^T + FP8 P.V (the arithmetic of the reference's SAGE_ATTN backend; about 3.7e-2 on Gaussian data);
# "int8_bf16": INT8 Q.K^T + bf16 P.V (V unquantised; about 1e-2)
ATTN_MODES = {"sage": _lib.DAX_ATTN_QK_I8_PV_F8, "int8_fp8": _lib.DAX_ATTN_QK_I8_PV_F8,
              "bf16": _lib.DAX_ATTN_QK_BF16_PV_BF16, "f16": _lib.DAX_ATTN_QK_BF16_PV_BF16,
              "int8_bf16": _lib.DAX_ATTN_QK_I8_PV_BF16}


class _Trace:
    """Optional launch accounting: number of library kernels launched and, when timing is on, CUDA
    events around each wrapper on the stream it launches on (used by the benchmark's roofline leg)."""

    KERNELS_PER_CALL = {"layernorm_modulate_quant": 1, "linear_dynamic": 2, "quant_rowwise": 1, "gemm_dequant": 1, "rmsnorm_rope_pack": 1, "attn_prepare": 5, "attn_forward": 1}

    def __init__(self):
        self.launches = 0
        self.timing = False
        self.events = []

    def reset(self, timing: bool = False):
        self.launches, self.timing, self.events = 0, timing, []

    def begin(self, name):
        self.launches += self.KERNELS_PER_CALL[name]
        if not self.timing:
            return None
        e0 = torch.cuda.Event(enable_timing=True)
        e0.record(torch.cuda.current_stream())
        return (name, e0)

    def end(self, tok, meta=None):
        if tok is None:
            return
        e1 = torch.cuda.Event(enable_timing=True)
        e1.record(torch.cuda.current_stream())
        self.events.append((tok[0], tok[1], e1, meta))

    def summary(self):
        """name -> (calls, total milliseconds, list of meta) after a device synchronise."""
        out = {}
        for name, e0, e1, meta in self.events:
            c, t, m = out.get(name, (0, 0.0, []))
            out[name] = (c + 1, t + e0.elapsed_time(e1), m + [meta])
        return out


TRACE = _Trace()


def _dt(dtype: torch.dtype) -> int:
    if dtype not in _DT:
        raise NotImplementedError(f"dax_b200: dtype {dtype} is not supported")
    return _DT[dtype]


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*ts) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("dax_b200 operators run on CUDA tensors only; there is no CPU path")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _ptr_array(ptrs):
    """Host array of device pointers for the ``*_scatter`` entry points."""
    import ctypes
    return (ctypes.c_void_p * len(ptrs))(*[int(p) for p in ptrs])


def peer_copy(dst_ptr: int, src: torch.Tensor, stream: Optional[torch.cuda.Stream] = None) -> None:
    """Copy the contiguous tensor ``src`` to the device address ``dst_ptr`` (possibly another GPU's buffer) with the
    copy engines, on ``stream`` (default: the current stream)."""
    _need_cuda(src)
    assert src.is_contiguous()
    st = (stream or torch.cuda.current_stream()).cuda_stream
    check(load().dax_peer_copy(int(dst_ptr), src.data_ptr(), src.numel() * src.element_size(), st))


def quant_rowwise(x: torch.Tensor, q_dtype: torch.dtype, *, col_group: Optional[int] = None,
                  group_stride: int = 0, rows: Optional[int] = None, cols: Optional[int] = None,
                  ldx: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-token quantisation of a ``[M, K]`` matrix -> ``(q [M, K], scale [M, 1] fp32)``.

    With ``col_group``/``group_stride`` (and explicit ``rows``, ``cols``, ``ldx``) ``x`` is read as
    column groups living in separate slabs, see ``dax_quant_rowwise`` in ``include/dax_b200.h``."""
    _need_cuda(x)
    if col_group is None:
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        M, K = x2.shape
        ld, cg, gs = x2.stride(0) if M > 1 else K, K, 0
        src = x2
    else:
        M, K, ld, cg, gs, src = rows, cols, ldx, col_group, group_stride, x
    q = torch.empty((M, K), dtype=q_dtype, device=x.device)
    scale = torch.empty((M, 1), dtype=torch.float32, device=x.device)
    tok = TRACE.begin("quant_rowwise")
    check(load().dax_quant_rowwise(src.data_ptr(), _dt(x.dtype), M, K, ld, cg, gs, q.data_ptr(), _dt(q_dtype),
                                   scale.data_ptr(), _stream()))
    TRACE.end(tok, (M, K, x.element_size()))
    return q, scale


def gemm_dequant(qx: torch.Tensor, sx: torch.Tensor, qw: torch.Tensor, sw: torch.Tensor,
                 bias: Optional[torch.Tensor], out_dtype: torch.dtype, *, out: Optional[torch.Tensor] = None,
                 ldo: Optional[int] = None, out_col_group: Optional[int] = None, out_group_stride: int = 0,
                 row_sumsq: Optional[torch.Tensor] = None, acc_dump: Optional[torch.Tensor] = None,
                 act: Optional[str] = None, resid: Optional[torch.Tensor] = None,
                 gate: Optional[torch.Tensor] = None, group_ptrs=None) -> Optional[torch.Tensor]:
    """``out = cast((acc(qx @ qw.T) * sx) * sw) + bias`` on the tcgen05 INT8 / FP8 pipe, optionally followed
    by ``act="gelu_tanh"`` and / or the gated residual ``out = resid + gate * out`` (gate ``[N]`` fp32).
    With ``group_ptrs`` (device addresses, one per group of ``out_col_group`` columns, possibly peer mappings of
    other GPUs' buffers) row ``t`` of group ``g`` is stored at ``group_ptrs[g] + t * ldo``; nothing is returned."""
    _need_cuda(qx, sx, qw, sw, bias, out)
    M, K = qx.shape
    N = qw.shape[0]
    assert qw.shape[1] == K and qx.is_contiguous() and qw.is_contiguous()
    assert sx.numel() == M and sw.numel() == N and sx.dtype == torch.float32 and sw.dtype == torch.float32
    if group_ptrs is not None:
        assert out is None and row_sumsq is None and acc_dump is None and act is None and resid is None
        tok = TRACE.begin("gemm_dequant")
        check(load().dax_gemm_dequant_scatter(qx.data_ptr(), _dt(qx.dtype), sx.data_ptr(), qw.data_ptr(), _dt(qw.dtype),
                                              sw.data_ptr(), _ptr(bias), _dt(bias.dtype) if bias is not None else 0,
                                              _ptr_array(group_ptrs), len(group_ptrs), _dt(out_dtype), M, N, K, ldo,
                                              out_col_group, _stream()))
        TRACE.end(tok, (M, N, K))
        return None
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=qx.device)
        ldo = N
    if out_col_group is None:
        out_col_group = N
    if act not in (None, "gelu_tanh"):
        raise NotImplementedError(f"unknown activation {act!r}")
    if resid is not None:
        _need_cuda(resid, gate)
        assert resid.dtype == out_dtype and resid.stride(-1) == 1 and resid.shape == (M, N)
        assert gate is None or (gate.dtype == torch.float32 and gate.numel() == N and gate.is_contiguous())
    tok = TRACE.begin("gemm_dequant")
    check(load().dax_gemm_dequant_ex(qx.data_ptr(), _dt(qx.dtype), sx.data_ptr(), qw.data_ptr(), _dt(qw.dtype),
                                     sw.data_ptr(), _ptr(bias), _dt(bias.dtype) if bias is not None else 0,
                                     out.data_ptr(), _dt(out_dtype), M, N, K, ldo, out_col_group, out_group_stride,
                                     _ptr(row_sumsq), _ptr(acc_dump), 1 if act else 0, _ptr(resid),
                                     resid.stride(0) if resid is not None else 0, _ptr(gate), _stream()))
    TRACE.end(tok, (M, N, K))
    return out


def linear_dynamic(x: torch.Tensor, qw: torch.Tensor, sw: torch.Tensor, bias: Optional[torch.Tensor],
                   act_dtype: torch.dtype, out_dtype: torch.dtype) -> torch.Tensor:
    """``dynamic.Linear.forward`` in one library call: quantise ``x [M, K]`` per token, multiply by the
    quantised weight ``qw [N, K]``, de-quantise, add the bias.  The workspace comes from torch."""
    _need_cuda(x, qw, sw, bias)
    M, K = x.shape
    N = qw.shape[0]
    assert x.stride(1) == 1 and qw.is_contiguous()
    n = load().dax_linear_dynamic_workspace_bytes(M, K)
    ws = torch.empty(n + 256, dtype=torch.uint8, device=x.device)
    off = (-ws.data_ptr()) % 256
    out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    tok = TRACE.begin("linear_dynamic")
    check(load().dax_linear_dynamic(x.data_ptr(), _dt(x.dtype), M, K, x.stride(0) if M > 1 else K, qw.data_ptr(),
                                    _dt(qw.dtype), _dt(act_dtype), sw.data_ptr(), _ptr(bias),
                                    _dt(bias.dtype) if bias is not None else 0, out.data_ptr(), _dt(out_dtype), N, N,
                                    ws.data_ptr() + off, n, _stream()))
    TRACE.end(tok, (M, N, K))
    return out


def layernorm_modulate_quant(x: torch.Tensor, *, eps: float = 1e-6, ln_weight: Optional[torch.Tensor] = None,
                             ln_bias: Optional[torch.Tensor] = None, shift: Optional[torch.Tensor] = None,
                             scale: Optional[torch.Tensor] = None, q_dtype: Optional[torch.dtype] = None,
                             want_y: bool = True):
    """``y = LN(x) [* w + b] [* (1 + scale) + shift]`` per token row of ``x [s, D]`` (all vectors ``[D]`` fp32),
    optionally with the per-token quantisation of ``y`` fused in.  Returns ``(y or None, q or None, qscale or None)``."""
    _need_cuda(x, ln_weight, ln_bias, shift, scale)
    s_, D = x.shape
    assert x.stride(1) == 1
    for v in (ln_weight, ln_bias, shift, scale):
        assert v is None or (v.dtype == torch.float32 and v.numel() == D and v.is_contiguous())
    y = torch.empty((s_, D), dtype=x.dtype, device=x.device) if want_y else None
    q = qs = None
    if q_dtype is not None:
        q = torch.empty((s_, D), dtype=q_dtype, device=x.device)
        qs = torch.empty((s_, 1), dtype=torch.float32, device=x.device)
    tok = TRACE.begin("layernorm_modulate_quant")
    check(load().dax_layernorm_modulate_quant(x.data_ptr(), _dt(x.dtype), s_, D, x.stride(0), _ptr(ln_weight),
                                              _ptr(ln_bias), _ptr(shift), _ptr(scale), float(eps), _ptr(y), D, _ptr(q),
                                              _dt(q_dtype) if q_dtype is not None else 0, _ptr(qs), _stream()))
    TRACE.end(tok, (s_, D))
    return y, q, qs


def rmsnorm_rope_pack(x: torch.Tensor, *, norm_weight: Optional[torch.Tensor], do_norm: bool, eps: float = 1e-6,
                      rope_cos: Optional[torch.Tensor] = None, rope_sin: Optional[torch.Tensor] = None,
                      token_offset: int = 0, row_sumsq: Optional[torch.Tensor] = None,
                      out: Optional[torch.Tensor] = None, ldo: Optional[int] = None,
                      col_group: Optional[int] = None, group_stride: int = 0, group_ptrs=None) -> Optional[torch.Tensor]:
    """RMSNorm over the full row + rotary embedding + write into a (possibly grouped) layout.  With ``group_ptrs``
    (one device address per column group, possibly in other GPUs' memory) row ``t`` of group ``g`` goes to
    ``group_ptrs[g] + t * ldo``."""
    _need_cuda(x, norm_weight, rope_cos, rope_sin, row_sumsq, out)
    s, D = x.shape
    assert x.stride(1) == 1
    if group_ptrs is not None:
        assert out is None and ldo is not None and col_group is not None
    elif out is None:
        out = torch.empty((s, D), dtype=x.dtype, device=x.device)
        ldo = D
    if col_group is None:
        col_group = D
    # the kernel reads the weight as 16-bit elements of x's dtype and the tables as fp32 [S_total, 64]
    if norm_weight is not None and (norm_weight.dtype != x.dtype or norm_weight.numel() != D or not norm_weight.is_contiguous()):
        raise ValueError(f"rmsnorm_rope_pack: norm_weight must be a contiguous [{D}] tensor of {x.dtype}, got "
                         f"{tuple(norm_weight.shape)} {norm_weight.dtype}")
    if (rope_cos is None) != (rope_sin is None):
        raise ValueError("rmsnorm_rope_pack: rope_cos and rope_sin come together")
    for tname, tab in (("rope_cos", rope_cos), ("rope_sin", rope_sin)):
        if tab is not None and (tab.dtype != torch.float32 or tab.dim() != 2 or tab.shape[1] != 64 or not tab.is_contiguous()
                                or token_offset + s > tab.shape[0]):
            raise ValueError(f"rmsnorm_rope_pack: {tname} must be a contiguous fp32 [>= {token_offset + s}, 64] table, got "
                             f"{tuple(tab.shape)} {tab.dtype}")
    if row_sumsq is not None and (row_sumsq.dtype != torch.float32 or row_sumsq.dim() != 2 or row_sumsq.shape[0] < s
                                  or not row_sumsq.is_contiguous()):
        raise ValueError(f"rmsnorm_rope_pack: row_sumsq must be a contiguous fp32 [>= {s}, n] tensor")
    n_part = row_sumsq.shape[1] if row_sumsq is not None else 0
    tok = TRACE.begin("rmsnorm_rope_pack")
    if group_ptrs is not None:
        check(load().dax_rmsnorm_rope_pack_scatter(x.data_ptr(), _dt(x.dtype), s, D, x.stride(0), _ptr(row_sumsq), n_part,
                                                   1 if do_norm else 0, _ptr(norm_weight), float(eps), _ptr(rope_cos),
                                                   _ptr(rope_sin), token_offset, _ptr_array(group_ptrs), len(group_ptrs),
                                                   ldo, col_group, _stream()))
        TRACE.end(tok, (s, D))
        return None
    check(load().dax_rmsnorm_rope_pack(x.data_ptr(), _dt(x.dtype), s, D, x.stride(0), _ptr(row_sumsq), n_part,
                                       1 if do_norm else 0, _ptr(norm_weight), float(eps), _ptr(rope_cos),
                                       _ptr(rope_sin), token_offset, out.data_ptr(), ldo, col_group, group_stride,
                                       _stream()))
    TRACE.end(tok, (s, D))
    return out


def _bhsd_strides(t: torch.Tensor) -> I64x3:
    assert t.dim() == 4 and t.shape[-1] == 128 and t.stride(-1) == 1, "expected [B, heads, S, 128], channels contiguous"
    return I64x3(t.stride(0), t.stride(1), t.stride(2))


class AttentionPlan:
    """Prepared operands of one attention call (workspace owned by torch)."""

    def __init__(self, B, heads, Sq, Sk, mode, workspace, dtype):
        self.B, self.heads, self.Sq, self.Sk, self.mode, self.workspace, self.dtype = B, heads, Sq, Sk, mode, workspace, dtype


_WS_CACHE = {}   # (device, B, heads, Sq, Sk, mode) -> buffer; insertion-ordered, a few most recent shapes
_WS_CACHE_ENTRIES = 4


def attn_workspace(B: int, heads: int, Sq: int, Sk: int, mode: int, device) -> torch.Tensor:
    """Workspace of one attention shape.  A block alternates between self-attention and cross-attention, so a few
    shapes stay cached; every plan of the same shape shares ONE buffer: a plan is valid until the next
    ``attn_prepare`` of that shape (on the same stream)."""
    n = load().dax_attn_workspace_bytes(B, heads, Sq, Sk, mode)
    if n == 0:
        check(_lib.DAX_ERR_INVALID)
    key = (str(device), B, heads, Sq, Sk, mode)
    ws = _WS_CACHE.pop(key, None)
    if ws is None:
        while len(_WS_CACHE) >= _WS_CACHE_ENTRIES:
            _WS_CACHE.pop(next(iter(_WS_CACHE)))
        ws = torch.empty(n + 1024, dtype=torch.uint8, device=device)
    _WS_CACHE[key] = ws  # most recently used last
    off = (-ws.data_ptr()) % 1024
    return ws[off:off + n]


def attn_prepare(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mode: str = "bf16",
                 sm_scale: Optional[float] = None, parts: str = "all") -> AttentionPlan:
    """q, k, v: ``[B, heads, S, 128]`` views (any batch/head/token strides) of bf16 or fp16.  ``parts``: "all", or
    "kv" (statistics, K and V operands) and "q" (Q operands) as two calls on the same shape, for callers whose K and
    V are complete before Q is."""
    _need_cuda(q, k, v)
    B, heads, Sq, d = q.shape
    Sk = k.shape[2]
    assert d == 128 and k.shape == v.shape and k.shape[:2] == q.shape[:2] and q.dtype == k.dtype == v.dtype
    m = ATTN_MODES[mode]
    ws = attn_workspace(B, heads, Sq, Sk, m, q.device)
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(d)
    tok = TRACE.begin("attn_prepare")
    TRACE.launches -= {"all": 0, "kv": 1, "q": 4}[parts]  # five kernels in all: four on the K / V side, one for Q
    check(load().dax_attn_prepare_parts(q.data_ptr(), k.data_ptr(), v.data_ptr(), _dt(q.dtype), B, heads, Sq, Sk,
                                        _bhsd_strides(q), _bhsd_strides(k), _bhsd_strides(v), float(sm_scale), m,
                                        {"all": 3, "kv": 1, "q": 2}[parts], ws.data_ptr(), ws.numel(), _stream()))
    TRACE.end(tok, (B, heads, Sq, Sk))
    return AttentionPlan(B, heads, Sq, Sk, m, ws, q.dtype)


def attn_forward(plan: AttentionPlan, out: torch.Tensor, q_begin: int = 0, q_end: Optional[int] = None,
                 n_ranges: int = 1, range_stride: int = 0) -> torch.Tensor:
    """Run the flash pass for the query rows ``[q_begin + r*range_stride, q_end + r*range_stride)``,
    ``r < n_ranges``, into ``out`` (a ``[B, heads, Sq, 128]`` view)."""
    _need_cuda(out)
    if q_end is None:
        q_end = plan.Sq
    assert out.shape == (plan.B, plan.heads, plan.Sq, 128) and out.dtype == plan.dtype
    tok = TRACE.begin("attn_forward")
    check(load().dax_attn_forward(out.data_ptr(), _dt(out.dtype), plan.B, plan.heads, plan.Sq, plan.Sk,
                                  _bhsd_strides(out), q_begin, q_end, n_ranges, range_stride, plan.mode,
                                  plan.workspace.data_ptr(),
                                  plan.workspace.numel(), _stream()))
    TRACE.end(tok, (plan.B, plan.heads, (q_end - q_begin) * n_ranges, plan.Sk))
    return out


def attn_forward_scatter(plan: AttentionPlan, dest_ptrs, rows_per_dest: int, head_stride: int, token_stride: int,
                         q_begin: int = 0, q_end: Optional[int] = None) -> None:
    """The flash pass (batch 1) with every query row written to the destination that owns it: row ``q`` of head
    ``h`` goes to ``dest_ptrs[q // rows_per_dest] + (q % rows_per_dest) * token_stride + h * head_stride``
    (elements of the plan's dtype).  The destinations may be other GPUs' buffers (peer mappings)."""
    assert plan.B == 1
    if q_end is None:
        q_end = plan.Sq
    tok = TRACE.begin("attn_forward")
    check(load().dax_attn_forward_scatter(_ptr_array(dest_ptrs), len(dest_ptrs), rows_per_dest, _dt(plan.dtype), plan.heads,
                                          plan.Sq, plan.Sk, head_stride, token_stride, q_begin, q_end, plan.mode,
                                          plan.workspace.data_ptr(), plan.workspace.numel(), _stream()))
    TRACE.end(tok, (plan.B, plan.heads, q_end - q_begin, plan.Sk))


def direct_attention_ok(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mode: str) -> bool:
    """Whether the in-place 16-bit kernel serves this call: bf16 mode and tensors, at least one tile of queries and
    keys, (batch, head) flattening to one stride."""
    B, heads = q.shape[:2]
    return (ATTN_MODES[mode] == _lib.DAX_ATTN_QK_BF16_PV_BF16 and q.dtype == torch.bfloat16 and q.shape[2] >= 128
            and k.shape[2] >= 128 and (B == 1 or all(t.stride(0) == heads * t.stride(1) for t in (q, k, v))))


def attention_direct(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: Optional[torch.Tensor] = None, *,
                     sm_scale: Optional[float] = None, dest_ptrs=None, rows_per_dest: int = 0, head_stride: int = 0,
                     token_stride: int = 0, q_begin: int = 0, q_end: Optional[int] = None, n_ranges: int = 1,
                     range_stride: int = 0) -> Optional[torch.Tensor]:
    """The 16-bit attention reading ``q, k, v`` (``[B, heads, S, 128]`` views, bf16 or fp16) in place: one kernel, no
    prepare step, no workspace.  Result into ``out`` (a ``[B, heads, Sq, 128]`` view; allocated token-major when
    omitted) or, with ``dest_ptrs``, scattered by destination like ``attn_forward_scatter``."""
    _need_cuda(q, k, v, out)
    B, heads, Sq, d = q.shape
    Sk = k.shape[2]
    assert d == 128 and k.shape == v.shape and k.shape[:2] == q.shape[:2] and q.dtype == k.dtype == v.dtype
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(d)
    if q_end is None:
        q_end = Sq
    if dest_ptrs is not None:
        o_ptr, o_str, table, n = None, I64x3(0, head_stride, token_stride), _ptr_array(dest_ptrs), len(dest_ptrs)
    else:
        if out is None:
            out = torch.empty((B, Sq, heads, d), dtype=q.dtype, device=q.device).transpose(1, 2)
        assert out.shape == (B, heads, Sq, 128) and out.dtype == q.dtype
        o_ptr, o_str, table, n = out.data_ptr(), _bhsd_strides(out), None, 0
    tok = TRACE.begin("attn_forward")
    check(load().dax_attn_forward_direct(q.data_ptr(), k.data_ptr(), v.data_ptr(), _dt(q.dtype), B, heads, Sq, Sk,
                                         _bhsd_strides(q), _bhsd_strides(k), _bhsd_strides(v), float(sm_scale), o_ptr, o_str,
                                         table, n, rows_per_dest, q_begin, q_end, n_ranges, range_stride, _stream()))
    TRACE.end(tok, (B, heads, (q_end - q_begin) * n_ranges, Sk))
    return out


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mode: str = "bf16",
              sm_scale: Optional[float] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Non-causal attention over ``[B, heads, S, 128]``; the result has the memory layout
    ``[B, S, heads, 128]`` (token-major, as the head->sequence exchange wants it) viewed as
    ``[B, heads, S, 128]``."""
    B, heads, Sq, d = q.shape
    if direct_attention_ok(q, k, v, mode):
        return attention_direct(q, k, v, out, sm_scale=sm_scale)  # the 16-bit mode reads its operands in place
    plan = attn_prepare(q, k, v, mode, sm_scale)
    if out is None:
        out = torch.empty((B, Sq, heads, d), dtype=q.dtype, device=q.device).transpose(1, 2)
    return attn_forward(plan, out)
