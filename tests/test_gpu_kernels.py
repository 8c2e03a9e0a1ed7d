"""Parity of every CUDA entry point against the oracle, through the C ABI (ctypes).  Needs a B200."""
import math
import os

import pytest
import torch

from oracle import dax_oracle as O

pytestmark = pytest.mark.gpu

DEV = "cuda"
FP8 = {"e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}


@pytest.fixture(scope="module")
def ops(built_library):
    if not torch.cuda.is_available():
        pytest.fail("the gpu tests need a CUDA device")
    from dax_b200 import ops as _ops
    return _ops


@pytest.fixture(autouse=True)
def device_status_clean():
    yield
    from dax_b200 import _lib
    assert _lib.device_status() == 0, "a kernel reported a timed-out wait"


def bits(t):
    return t.view(torch.uint8) if t.dtype in FP8.values() else t


# ---- quantiser -------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["bf16", "f16", "f32"])
def test_quantiser_golden(ops, golden_dir, name):
    g = torch.load(os.path.join(golden_dir, f"quant_{name}.pt"))
    q, s = ops.quant_rowwise(g["x"].to(DEV), torch.int8)
    assert torch.equal(q.cpu(), g["q_int8"]) and torch.equal(s.cpu(), g["s_int8"])
    for f, dt in FP8.items():
        q, s = ops.quant_rowwise(g["x"].to(DEV), dt)
        assert torch.equal(q.cpu().view(torch.uint8), g["q_" + f]) and torch.equal(s.cpu(), g["s_" + f])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("K", [16, 256, 1536, 4096, 5120, 13824, 20480])
def test_quantiser_oracle(ops, dtype, K):
    torch.manual_seed(K)
    M = 67
    x = (torch.randn(M, K) * torch.logspace(-3, 3, M).unsqueeze(1)).to(dtype)
    x[3] = 0
    for qd in (torch.int8, torch.float8_e4m3fn, torch.float8_e5m2):
        q, s = ops.quant_rowwise(x.to(DEV), qd)
        qr, sr = O.quantize_rowwise(x, qd)
        assert torch.equal(bits(q.cpu()), bits(qr)), (dtype, K, qd)
        assert torch.equal(s.cpu(), sr)


def test_quantiser_grouped_columns_and_empty(ops):
    """Reading the head->token receive slabs [P, n, h*d] in place equals quantising the gathered matrix."""
    P, n, hd = 4, 37, 256
    slabs = torch.randn(P, n, hd).bfloat16()
    mat = slabs.permute(1, 0, 2).reshape(n, P * hd).contiguous()
    q, s = ops.quant_rowwise(slabs.to(DEV), torch.int8, col_group=hd, group_stride=n * hd, rows=n, cols=P * hd, ldx=hd)
    qr, sr = O.quantize_rowwise(mat, torch.int8)
    assert torch.equal(q.cpu(), qr) and torch.equal(s.cpu(), sr)
    # the same through the row-pipelined kernel (rows of more than 256 vectors): 8 slabs of 640 columns, FP8 and INT8
    P, n, hd = 8, 301, 640
    slabs = torch.randn(P, n, hd).bfloat16()
    mat = slabs.permute(1, 0, 2).reshape(n, P * hd).contiguous()
    for qd in (torch.int8, torch.float8_e4m3fn):
        q, s = ops.quant_rowwise(slabs.to(DEV), qd, col_group=hd, group_stride=n * hd, rows=n, cols=P * hd, ldx=hd)
        qr, sr = O.quantize_rowwise(mat, qd)
        assert torch.equal(bits(q.cpu()), bits(qr)) and torch.equal(s.cpu(), sr)
    q, s = ops.quant_rowwise(torch.empty(0, 64, device=DEV).bfloat16(), torch.int8)
    assert q.shape == (0, 64)
    with pytest.raises(ValueError):
        ops.quant_rowwise(torch.zeros(4, 24, device=DEV).bfloat16(), torch.int8)


def test_quantiser_full_size_properties(ops):
    """M = 75,600 tokens x 5120: scale * 127 bounds every row, re-quantising the de-quantised tensor is
    idempotent, and a row permutation commutes with the quantiser."""
    torch.manual_seed(1)
    M, K = 75600, 5120
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    q, s = ops.quant_rowwise(x, torch.int8)
    assert int(q.abs().max()) <= 127 + 1
    amax = x.abs().amax(-1, keepdim=True).float()
    assert torch.all((s * 127 - amax).abs() <= amax * 2 ** -8 + 1e-6)
    perm = torch.randperm(M, device=DEV)
    q2, s2 = ops.quant_rowwise(x[perm].contiguous(), torch.int8)
    assert torch.equal(q2, q[perm]) and torch.equal(s2, s[perm])
    xd = q.float() * s
    q3, s3 = ops.quant_rowwise(xd, torch.int8)
    assert torch.equal(q3, q)
    # a sample of rows against the oracle
    idx = torch.arange(0, M, 997)
    qr, sr = O.quantize_rowwise(x[idx.to(DEV)].cpu(), torch.int8)
    assert torch.equal(q[idx.to(DEV)].cpu(), qr) and torch.equal(s[idx.to(DEV)].cpu(), sr)


def test_quantiser_fp8_division_is_correctly_rounded(ops):
    """The FP8 path divides by the row scale; the kernel does it as a reciprocal multiply plus one fused
    residual correction, which must give the correctly rounded quotient: 21 million elements over nine decades
    of magnitude against true division, bit for bit."""
    torch.manual_seed(7)
    M, K = 4096, 5120
    x = (torch.randn(M, K, device=DEV) * torch.logspace(-4, 5, M, device=DEV).unsqueeze(1)).bfloat16()
    for qd, qmax in ((torch.float8_e4m3fn, 448.0), (torch.float8_e5m2, 57344.0)):
        q, s = ops.quant_rowwise(x, qd)
        sr = (x.abs().amax(-1, keepdim=True) / qmax).clamp(min=torch.finfo(torch.float32).eps).float()
        qr = (x.float() / sr).clamp(-qmax, qmax).to(qd)
        assert torch.equal(s, sr)
        assert torch.equal(q.view(torch.uint8), qr.view(torch.uint8))


# ---- GEMM --------------------------------------------------------------------------------------------
GEMM_SHAPES = [(128, 256, 128), (17, 8, 16), (300, 512, 1536), (1000, 1536, 1536), (77, 264, 208), (129, 5120, 640),
               (2500, 768, 4096)]


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_gemm_int8_bit_exact(ops, M, N, K, out_dtype):
    torch.manual_seed(M + N + K)
    x = torch.randn(M, K).to(out_dtype)
    w = (torch.randn(N, K) * 0.02).to(out_dtype)
    b = (torch.randn(N) * 0.1).to(out_dtype)
    qw, sw = O.quantize_weight(w, torch.int8)
    yr, qx, sx, acc = O.linear_int8(x, qw, sw, b, out_dtype, return_parts=True)
    dump = torch.zeros(M, N, dtype=torch.int32, device=DEV)
    ss = torch.zeros(M, 2 * ((N + 255) // 256), device=DEV)
    y = ops.gemm_dequant(qx.to(DEV), sx.to(DEV), qw.to(DEV), sw.to(DEV).reshape(-1).contiguous(), b.to(DEV), out_dtype,
                         acc_dump=dump, row_sumsq=ss)
    assert torch.equal(dump.cpu(), acc), "int32 accumulators differ"
    assert torch.equal(y.cpu(), yr), "de-quantised outputs differ"
    ref_ss = yr.double().pow(2).sum(-1)
    assert torch.allclose(ss.sum(-1).cpu().double(), ref_ss, rtol=1e-4, atol=1e-6)
    y2 = ops.gemm_dequant(qx.to(DEV), sx.to(DEV), qw.to(DEV), sw.to(DEV).reshape(-1).contiguous(), None, out_dtype)
    yr2 = O.linear_int8(x, qw, sw, None, out_dtype)
    assert torch.equal(y2.cpu(), yr2)


def test_gemm_int8_golden(ops, golden_dir):
    g = torch.load(os.path.join(golden_dir, "weight_bf16.pt"))
    l = torch.load(os.path.join(golden_dir, "linear_int8.pt"))
    x = l["x"].reshape(-1, 256)
    qx, sx = ops.quant_rowwise(x.to(DEV), torch.int8)
    y = ops.gemm_dequant(qx, sx, g["qweight_int8"].to(DEV), g["wscale_int8"].to(DEV).reshape(-1).contiguous(),
                         g["b"].to(DEV), torch.bfloat16)
    assert torch.equal(y.cpu().view(l["y"].shape), l["y"])


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (300, 512, 1536), (77, 264, 208), (1000, 5120, 1024)])
@pytest.mark.parametrize("act", ["e4m3", "e5m2"])
def test_gemm_fp8(ops, M, N, K, act):
    """FP8: fp32 accumulation order differs from any reference, so the check is the stated tolerance
    (rel-L2 <= 1e-2, cosine >= 0.999) and, for the raw accumulators, 1e-5 relative."""
    torch.manual_seed(M + K)
    x = torch.randn(M, K).bfloat16()
    w = (torch.randn(N, K) * 0.02).bfloat16()
    b = (torch.randn(N) * 0.1).bfloat16()
    qw, sw = O.quantize_weight(w, torch.float8_e4m3fn)
    yr = O.linear_fp8(x, qw, sw, b, torch.bfloat16, FP8[act])
    qx, sx = O.quantize_rowwise(x, FP8[act])
    dump = torch.zeros(M, N, dtype=torch.float32, device=DEV)
    y = ops.gemm_dequant(qx.to(DEV), sx.to(DEV), qw.to(DEV), sw.to(DEV).reshape(-1).contiguous(), b.to(DEV),
                         torch.bfloat16, acc_dump=dump)
    assert O.rel_l2(y.cpu(), yr) <= 1e-2 and O.cosine(y.cpu(), yr) >= 0.999
    acc = qx.double() @ qw.double().T
    assert O.rel_l2(dump.cpu(), acc) <= 1e-5
    assert (y.cpu().float() - yr.float()).abs().max() <= 2 ** -6 * yr.float().abs().max()


def test_gemm_writes_exchange_layout(ops):
    """out_col_group / out_group_stride: the projection lands directly in [P, s, h*d]."""
    P, s, hd, K = 4, 150, 256, 512
    N = P * hd
    x = torch.randn(s, K).bfloat16()
    w = (torch.randn(N, K) * 0.02).bfloat16()
    qw, sw = O.quantize_weight(w, torch.int8)
    yr, qx, sx, _ = O.linear_int8(x, qw, sw, None, torch.bfloat16, return_parts=True)
    send = torch.zeros(P, s, hd, dtype=torch.bfloat16, device=DEV)
    ops.gemm_dequant(qx.to(DEV), sx.to(DEV), qw.to(DEV), sw.to(DEV).reshape(-1).contiguous(), None, torch.bfloat16,
                     out=send, ldo=hd, out_col_group=hd, out_group_stride=s * hd)
    assert torch.equal(send.cpu().permute(1, 0, 2).reshape(s, N), yr)


def test_gemm_full_size_linearity(ops):
    """M = 75,600, 5120 -> 5120 (too large for the CPU oracle): the int32 accumulators are linear in the
    activations, acc(a + b) = acc(a) + acc(b), and a sample of rows matches the oracle exactly."""
    torch.manual_seed(2)
    M, N, K = 75600, 5120, 5120
    a = torch.randint(-60, 60, (M, K), dtype=torch.int8, device=DEV)
    b = torch.randint(-60, 60, (M, K), dtype=torch.int8, device=DEV)
    w = torch.randint(-127, 128, (N, K), dtype=torch.int8, device=DEV)
    ones_m = torch.ones(M, 1, device=DEV)
    ones_n = torch.ones(N, device=DEV)
    outs = []
    for qx in (a, b, a + b):
        dump = torch.empty(M, N, dtype=torch.int32, device=DEV)
        ops.gemm_dequant(qx, ones_m, w, ones_n, None, torch.float32, acc_dump=dump)
        outs.append(dump)
    assert torch.equal(outs[0] + outs[1], outs[2])
    idx = torch.arange(0, M, 2111, device=DEV)
    ref = O.int_matmul(a[idx].cpu(), w.cpu())
    assert torch.equal(outs[0][idx].cpu(), ref)


# ---- RMSNorm + RoPE + pack ---------------------------------------------------------------------------
def test_rmsnorm_rope_pack_many_rows_full_width(ops):
    """Production width (5120 = 40 heads: 320 threads x 2 vectors) and more rows than resident CTAs, so that every
    CTA strides over several rows with the next rows' copies in flight."""
    torch.manual_seed(5)
    grid = (3, 20, 25)
    S, H = 1500, 40
    D = H * 128
    x = (torch.randn(S, D) * torch.logspace(-1, 1, S).unsqueeze(1)).bfloat16()
    w = (1 + 0.1 * torch.randn(D)).bfloat16()
    fr = O.rope_table(grid)
    ref = O.rmsnorm(x.unsqueeze(0), w).unflatten(2, (H, -1)).transpose(1, 2)
    ref = O.apply_rotary_emb(ref, fr).transpose(1, 2).flatten(2, 3)[0]
    cos = fr.real.float().reshape(S, 64).contiguous().to(DEV)
    sin = fr.imag.float().reshape(S, 64).contiguous().to(DEV)
    y = ops.rmsnorm_rope_pack(x.to(DEV), norm_weight=w.to(DEV), do_norm=True, rope_cos=cos, rope_sin=sin)
    assert O.rel_l2(y.cpu(), ref) <= 2e-3
    parts = x.float().pow(2).view(S, D // 128, 128).sum(-1).to(DEV)   # 40 partials per row, as the GEMM writes them
    y2 = ops.rmsnorm_rope_pack(x.to(DEV), norm_weight=w.to(DEV), do_norm=True, rope_cos=cos, rope_sin=sin, row_sumsq=parts)
    assert O.rel_l2(y2.cpu(), ref) <= 2e-3
    # every row on its own equals the row inside the batch (no cross-row leakage through the prefetch registers)
    idx = torch.tensor([0, 1, 443, 444, 445, 887, 1499])
    for i in idx.tolist():
        yi = ops.rmsnorm_rope_pack(x[i:i + 1].to(DEV), norm_weight=w.to(DEV), do_norm=True, rope_cos=cos, rope_sin=sin,
                                   token_offset=i)
        assert torch.equal(yi[0], y[i])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_rmsnorm_rope_pack(ops, dtype):
    torch.manual_seed(3)
    grid = (3, 4, 8)
    S, H = 96, 12
    D = H * 128
    x = torch.randn(S, D).to(dtype)
    w = (1 + 0.1 * torch.randn(D)).to(dtype)
    fr = O.rope_table(grid)
    ref = O.rmsnorm(x.unsqueeze(0), w).unflatten(2, (H, -1)).transpose(1, 2)
    ref = O.apply_rotary_emb(ref, fr).transpose(1, 2).flatten(2, 3)[0]
    cos = fr.real.float().reshape(S, 64).contiguous().to(DEV)
    sin = fr.imag.float().reshape(S, 64).contiguous().to(DEV)
    y = ops.rmsnorm_rope_pack(x.to(DEV), norm_weight=w.to(DEV), do_norm=True, rope_cos=cos, rope_sin=sin)
    assert O.rel_l2(y.cpu(), ref) <= 2e-3 and O.cosine(y.cpu(), ref) >= 0.9999
    # partial sums of squares from a GEMM epilogue give the same result as the in-kernel reduction
    parts = x.float().pow(2).view(S, D // 256, 256).sum(-1).to(DEV)
    y2 = ops.rmsnorm_rope_pack(x.to(DEV), norm_weight=w.to(DEV), do_norm=True, rope_cos=cos, rope_sin=sin, row_sumsq=parts)
    assert O.rel_l2(y2.cpu(), ref) <= 2e-3
    # rank 1 of 2: its token slice, packed into [P=3, s, h*d]
    s, P = S // 2, 3
    hd = D // P
    out = torch.zeros(P, s, hd, dtype=dtype, device=DEV)
    ops.rmsnorm_rope_pack(x[s:].to(DEV), norm_weight=w.to(DEV), do_norm=True, rope_cos=cos, rope_sin=sin, token_offset=s,
                          out=out, ldo=hd, col_group=hd, group_stride=s * hd)
    assert torch.equal(out.cpu().permute(1, 0, 2).reshape(s, D), y.cpu()[s:])
    # rotation only / norm only
    y3 = ops.rmsnorm_rope_pack(x.to(DEV), norm_weight=None, do_norm=False, rope_cos=cos, rope_sin=sin)
    ref3 = O.apply_rotary_emb(x.view(1, S, H, 128).transpose(1, 2), fr).transpose(1, 2).reshape(S, D)
    assert O.rel_l2(y3.cpu(), ref3) <= 2e-3
    y4 = ops.rmsnorm_rope_pack(x.to(DEV), norm_weight=w.to(DEV), do_norm=True)
    assert O.rel_l2(y4.cpu(), O.rmsnorm(x, w)) <= 2e-3


@pytest.mark.parametrize("H", [3, 40])
def test_rmsnorm_rope_pack_strided_rows(ops, H):
    """Input rows that are a column slice of a wider matrix (leading dimension larger than the width): same results as
    the contiguous copy."""
    torch.manual_seed(13)
    grid = (2, 5, 9)
    S, D = 90, H * 128
    wide = torch.randn(S, D + 128).bfloat16().to(DEV)
    xs = wide[:, :D]
    w = (1 + 0.1 * torch.randn(D)).bfloat16().to(DEV)
    fr = O.rope_table(grid)
    cos = fr.real.float().reshape(S, 64).contiguous().to(DEV)
    sin = fr.imag.float().reshape(S, 64).contiguous().to(DEV)
    y0 = ops.rmsnorm_rope_pack(xs.contiguous(), norm_weight=w, do_norm=True, rope_cos=cos, rope_sin=sin)
    y1 = ops.rmsnorm_rope_pack(xs, norm_weight=w, do_norm=True, rope_cos=cos, rope_sin=sin)
    assert torch.equal(y0, y1)


@pytest.mark.parametrize("H", [2, 16, 24, 32, 56, 64, 72])
def test_rmsnorm_rope_pack_widths(ops, H):
    """One width per kernel variant: rows that fill the CTA exactly (no predicates) and ragged ones, 1 to 4 vectors
    per thread, and the widest CTA; more rows than the copy ring is deep."""
    torch.manual_seed(H)
    grid = (2, 5, 7)
    S, D = 70, H * 128
    x = torch.randn(S, D).bfloat16()
    w = (1 + 0.1 * torch.randn(D)).bfloat16()
    fr = O.rope_table(grid)
    ref = O.rmsnorm(x.unsqueeze(0), w).unflatten(2, (H, -1)).transpose(1, 2)
    ref = O.apply_rotary_emb(ref, fr).transpose(1, 2).flatten(2, 3)[0]
    cos = fr.real.float().reshape(S, 64).contiguous().to(DEV)
    sin = fr.imag.float().reshape(S, 64).contiguous().to(DEV)
    y = ops.rmsnorm_rope_pack(x.to(DEV), norm_weight=w.to(DEV), do_norm=True, rope_cos=cos, rope_sin=sin)
    assert O.rel_l2(y.cpu(), ref) <= 2e-3
    # one partial sum per 128 columns, as the GEMM epilogue writes them (72 of them at the widest: more than two per lane)
    parts = x.float().pow(2).view(S, H, 128).sum(-1)
    y2 = ops.rmsnorm_rope_pack(x.to(DEV), norm_weight=w.to(DEV), do_norm=True, rope_cos=cos, rope_sin=sin,
                               row_sumsq=parts.to(DEV))
    assert O.rel_l2(y2.cpu(), ref) <= 2e-3


# ---- attention ---------------------------------------------------------------------------------------
def qkv(B, H, Sq, Sk, dtype=torch.bfloat16, offset=2.0, seed=0):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, H, Sq, 128, generator=g).to(dtype)
    k = (torch.randn(B, H, Sk, 128, generator=g) + offset * torch.randn(B, H, 1, 128, generator=g)).to(dtype)
    v = torch.randn(B, H, Sk, 128, generator=g).to(dtype)
    return q, k, v


@pytest.mark.parametrize("S", [1, 128, 256, 1000, 2049])
def test_attention_high_accuracy_mode(ops, S):
    """bf16 contractions: the tolerance stated for attention against fp32 SDPA,
    rel-L2 <= 1e-2 and cosine >= 0.999."""
    q, k, v = qkv(1, 3, S, S)
    ref = O.sdpa_fp32(q, k, v)
    o = ops.attention(q.to(DEV), k.to(DEV), v.to(DEV), mode="bf16").float().cpu()
    assert not torch.isnan(o).any()
    assert O.rel_l2(o, ref) <= 1e-2 and O.cosine(o, ref) >= 0.999


@pytest.mark.parametrize("S", [1, 128, 256, 1000, 2049])
def test_attention_sage_mode(ops, S):
    """INT8 Q.K^T + FP8 P.V.  THIS MODE DOES NOT MEET the stated attention tolerance (rel-L2 <= 1e-2): single-term
    FP8 P and V carry about 2.6 % relative rounding error each, so on Gaussian data (outputs are small residual
    sums) rel-L2 sits near 3.7e-2 for any kernel with these operand formats.  Labelled bounds: cosine >= 0.999,
    rel-L2 <= 5e-2, and within 4e-2 of the oracle's model of the same quantisation."""
    q, k, v = qkv(1, 3, S, S)
    ref = O.sdpa_fp32(q, k, v)
    o = ops.attention(q.to(DEV), k.to(DEV), v.to(DEV), mode="sage").float().cpu()
    assert not torch.isnan(o).any()
    assert O.cosine(o, ref) >= 0.999 and O.rel_l2(o, ref) <= 5e-2
    model = O.sage_attention_model(q, k, v)
    assert O.rel_l2(o, model) <= 4e-2


@pytest.mark.parametrize("S", [1, 128, 1000, 2049])
def test_attention_int8_bf16_mode(ops, S):
    """INT8 Q.K^T + bf16 P.V (V unquantised).  NOT HELD to the stated tolerance either: the INT8 rounding of Q and K
    alone costs about 1e-2 rel-L2 on Gaussian data (per-token Q scales, per-128-token K scales), i.e. it sits ON
    the bound.  Labelled bounds: rel-L2 <= 2e-2, cosine >= 0.9999, within 1e-2 of the oracle's model."""
    q, k, v = qkv(1, 3, S, S)
    ref = O.sdpa_fp32(q, k, v)
    o = ops.attention(q.to(DEV), k.to(DEV), v.to(DEV), mode="int8_bf16").float().cpu()
    assert not torch.isnan(o).any()
    assert O.cosine(o, ref) >= 0.9999 and O.rel_l2(o, ref) <= 2e-2
    model = O.sage_attention_model(q, k, v, qk="int8", pv="f16")
    assert O.rel_l2(o, model) <= 1e-2


def test_attention_k_smoothing_matters(ops):
    """A large per-channel K offset (the case mean-smoothing exists for) must not hurt accuracy."""
    q, k, v = qkv(1, 2, 512, 512, offset=20.0)
    ref = O.sdpa_fp32(q, k, v)
    o = ops.attention(q.to(DEV), k.to(DEV), v.to(DEV), mode="sage").float().cpu()
    assert O.cosine(o, ref) >= 0.999


@pytest.mark.parametrize("mode", ["sage", "bf16", "int8_bf16"])
def test_attention_layouts_ranges_and_cross(ops, mode):
    tol = {"sage": 5e-2, "bf16": 1e-2, "int8_bf16": 2e-2}[mode]
    # token-major memory ([B, S, H, d] viewed as [B, H, S, d]), fp16, batch 2, Sq != Sk
    q, k, v = qkv(2, 2, 300, 77, dtype=torch.float16)
    ref = O.sdpa_fp32(q, k, v)
    tm = lambda t: t.transpose(1, 2).contiguous().to(DEV).transpose(1, 2)
    o = ops.attention(tm(q), tm(k), tm(v), mode=mode)
    assert o.stride(2) == 2 * 128  # result is token-major
    assert O.rel_l2(o.float().cpu(), ref) <= tol
    # micro-batch style launch: P ranges of the query rows, everything else untouched
    q, k, v = qkv(1, 2, 4 * 150, 4 * 150)
    ref = O.sdpa_fp32(q, k, v)
    plan = ops.attn_prepare(q.to(DEV), k.to(DEV), v.to(DEV), mode)
    out = torch.full((1, 600, 2, 128), 7.0, dtype=torch.bfloat16, device=DEV).transpose(1, 2)
    ops.attn_forward(plan, out, q_begin=75, q_end=150, n_ranges=4, range_stride=150)
    got = out.float().cpu()
    for r in range(4):
        lo, hi = r * 150 + 75, r * 150 + 150
        assert O.rel_l2(got[:, :, lo:hi], ref[:, :, lo:hi]) <= tol
        assert bool((got[:, :, r * 150:lo] == 7.0).all())
    ops.attn_forward(plan, out, q_begin=0, q_end=75, n_ranges=4, range_stride=150)
    assert O.rel_l2(out.float().cpu(), ref) <= tol


def test_attention_rows_are_convex_combinations(ops):
    """Size-independent property at a long sequence (S = 32,760, the 480p config, two heads): with V
    constant per channel the output equals that constant whatever the scores are."""
    S, H = 32760, 2
    g = torch.Generator().manual_seed(5)
    q = torch.randn(1, H, S, 128, generator=g).bfloat16().to(DEV)
    k = torch.randn(1, H, S, 128, generator=g).bfloat16().to(DEV)
    c = torch.randn(1, H, 1, 128, generator=g).bfloat16()
    v = c.expand(1, H, S, 128).contiguous().to(DEV)
    for mode, tol in (("sage", 3e-2), ("bf16", 6e-3), ("int8_bf16", 6e-3)):
        o = ops.attention(q, k, v, mode=mode).float().cpu()
        assert O.rel_l2(o, c.float().expand_as(o)) <= tol
    # and a slice of query rows against fp32 SDPA over the full key set
    v2 = torch.randn(1, H, S, 128, generator=g).bfloat16().to(DEV)
    o = ops.attention(q, k, v2, mode="f16").float().cpu()
    ref = torch.nn.functional.scaled_dot_product_attention(q[:, :, 5000:5256].float().cpu(), k.float().cpu(), v2.float().cpu())
    assert O.rel_l2(o[:, :, 5000:5256], ref) <= 1e-2


# ---- one-call dynamic linear ---------------------------------------------------------------------------
@pytest.mark.parametrize("M,N,K", [(40, 192, 256), (512, 5120, 4096), (1000, 1536, 1536)])
def test_linear_dynamic_matches_two_step(ops, M, N, K):
    torch.manual_seed(M)
    x = torch.randn(M, K).bfloat16()
    w = (torch.randn(N, K) * 0.02).bfloat16()
    b = (torch.randn(N) * 0.1).bfloat16()
    for wdt, adt in ((torch.int8, torch.int8), (torch.float8_e4m3fn, torch.float8_e4m3fn)):
        qw, sw = O.quantize_weight(w, wdt)
        swd = sw.to(DEV).reshape(-1).contiguous()
        y = ops.linear_dynamic(x.to(DEV), qw.to(DEV), swd, b.to(DEV), adt, torch.bfloat16)
        qx, sx = ops.quant_rowwise(x.to(DEV), adt)
        y2 = ops.gemm_dequant(qx, sx, qw.to(DEV), swd, b.to(DEV), torch.bfloat16)
        assert torch.equal(y, y2)
        if wdt == torch.int8:
            assert torch.equal(y.cpu(), O.linear_int8(x, qw, sw, b, torch.bfloat16))


# ---- scattered outputs (the exchange written by the producing kernels) --------------------------------
def test_scatter_entry_points_match_the_strided_ones(ops):
    """The *_scatter entry points with every group pointer in a SEPARATE allocation of this GPU (what a peer mapping
    looks like to the kernel: an unrelated address) give exactly what the strided layouts give."""
    torch.manual_seed(11)
    P, s, hd, K = 4, 150, 256, 512
    N = D = P * hd
    # GEMM epilogue -> P separate slabs
    x = torch.randn(s, K).bfloat16()
    w = (torch.randn(N, K) * 0.02).bfloat16()
    qw, sw = O.quantize_weight(w, torch.int8)
    yr, qx, sx, _ = O.linear_int8(x, qw, sw, None, torch.bfloat16, return_parts=True)
    slabs = [torch.zeros(s + 3, hd, dtype=torch.bfloat16, device=DEV) for _ in range(P)]
    ops.gemm_dequant(qx.to(DEV), sx.to(DEV), qw.to(DEV), sw.to(DEV).reshape(-1).contiguous(), None, torch.bfloat16,
                     ldo=hd, out_col_group=hd, group_ptrs=[t[3:].data_ptr() for t in slabs])
    for g in range(P):
        assert torch.equal(slabs[g][3:].cpu(), yr[:, g * hd:(g + 1) * hd]) and bool((slabs[g][:3] == 0).all())
    # RMSNorm + RoPE pack -> P separate slabs
    grid, H = (2, 5, 15), 8
    xx = torch.randn(s, D).bfloat16().to(DEV)
    wn = (1 + 0.1 * torch.randn(D)).bfloat16().to(DEV)
    fr = O.rope_table(grid)
    cos = fr.real.float().reshape(s, 64).contiguous().to(DEV)
    sin = fr.imag.float().reshape(s, 64).contiguous().to(DEV)
    want = ops.rmsnorm_rope_pack(xx, norm_weight=wn, do_norm=True, rope_cos=cos, rope_sin=sin)
    slabs = [torch.zeros(s, hd, dtype=torch.bfloat16, device=DEV) for _ in range(P)]
    ops.rmsnorm_rope_pack(xx, norm_weight=wn, do_norm=True, rope_cos=cos, rope_sin=sin, ldo=hd, col_group=hd,
                          group_ptrs=[t.data_ptr() for t in slabs])
    assert torch.equal(torch.cat(slabs, 1), want)
    # plain scatter copy (no norm, no rotation), one group
    one = torch.zeros(s, D, dtype=torch.bfloat16, device=DEV)
    ops.rmsnorm_rope_pack(xx, norm_weight=None, do_norm=False, ldo=D, col_group=D, group_ptrs=[one.data_ptr()])
    assert torch.equal(one, xx)
    # attention rows scattered by destination: 3 destinations of 100 rows, each [src slab = 1 of 2, 100, h*d]
    for mode, tol in (("bf16", 1e-2), ("sage", 5e-2)):
        q, k, v = qkv(1, 2, 300, 300, seed=3)
        ref = O.sdpa_fp32(q, k, v)
        plan = ops.attn_prepare(q.to(DEV), k.to(DEV), v.to(DEV), mode)
        dests = [torch.full((2, 100, 2 * 128), 7.0, dtype=torch.bfloat16, device=DEV) for _ in range(3)]
        ops.attn_forward_scatter(plan, [t[1].data_ptr() for t in dests], rows_per_dest=100, head_stride=128, token_stride=256)
        got = torch.cat([t[1].view(100, 2, 128) for t in dests], 0).permute(1, 0, 2).unsqueeze(0).float().cpu()
        assert O.rel_l2(got, ref) <= tol and all(bool((t[0] == 7.0).all()) for t in dests)
    with pytest.raises(ValueError):
        ops.rmsnorm_rope_pack(xx, norm_weight=None, do_norm=False, ldo=hd, col_group=hd, group_ptrs=[one.data_ptr()] * 3)


@pytest.mark.parametrize("B,H,Sq,Sk,dtype", [(1, 3, 128, 128, torch.bfloat16), (1, 3, 1000, 1000, torch.bfloat16),
                                             (2, 2, 300, 512, torch.bfloat16), (1, 2, 2049, 2049, torch.bfloat16)])
def test_attention_direct(ops, B, H, Sq, Sk, dtype):
    """The 16-bit attention reading Q, K, V in place (3-D tensor maps over the strided views, V as the MN-major operand
    of P.V, no K smoothing, no workspace): head-major and token-major memory, against fp32 SDPA at the stated
    tolerance, and against the prepared-operand variant of the same kernel."""
    q, k, v = qkv(B, H, Sq, Sk, dtype=dtype, seed=Sq + Sk)
    ref = O.sdpa_fp32(q, k, v)
    tm = lambda t: t.transpose(1, 2).contiguous().to(DEV).transpose(1, 2)
    layouts = [(q.to(DEV), k.to(DEV), v.to(DEV))]
    if B == 1:  # token-major memory of a batch does not flatten (batch, head) into one stride
        layouts.append((tm(q), tm(k), tm(v)))
    for qq, kk, vv in layouts:
        o = ops.attention_direct(qq, kk, vv).float().cpu()
        assert not torch.isnan(o).any()
        assert O.rel_l2(o, ref) <= 1e-2 and O.cosine(o, ref) >= 0.999
    plan = ops.attn_prepare(q.to(DEV), k.to(DEV), v.to(DEV), "bf16")
    o2 = torch.empty((B, Sq, H, 128), dtype=dtype, device=DEV).transpose(1, 2)
    ops.attn_forward(plan, o2)
    assert O.rel_l2(o, o2.float().cpu()) <= 6e-3
    # fp16 tensors and sequences shorter than one tile are refused by the in-place kernel (the wrapper `attention`
    # sends them through the prepared-operand path)
    with pytest.raises(NotImplementedError):
        ops.attention_direct(q.to(DEV).half(), k.to(DEV).half(), v.to(DEV).half())
    with pytest.raises(NotImplementedError):
        ops.attention_direct(q.to(DEV)[:, :, :64], k.to(DEV)[:, :, :64], v.to(DEV)[:, :, :64])


def test_attention_direct_ranges_and_destinations(ops):
    q, k, v = qkv(1, 2, 600, 600, seed=9)
    ref = O.sdpa_fp32(q, k, v)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    out = torch.full((1, 600, 2, 128), 7.0, dtype=torch.bfloat16, device=DEV).transpose(1, 2)
    ops.attention_direct(qd, kd, vd, out, q_begin=75, q_end=150, n_ranges=4, range_stride=150)
    got = out.float().cpu()
    for r in range(4):
        lo, hi = r * 150 + 75, r * 150 + 150
        assert O.rel_l2(got[:, :, lo:hi], ref[:, :, lo:hi]) <= 1e-2 and bool((got[:, :, r * 150:lo] == 7.0).all())
    dests = [torch.full((2, 200, 2 * 128), 7.0, dtype=torch.bfloat16, device=DEV) for _ in range(3)]
    ops.attention_direct(qd, kd, vd, dest_ptrs=[t[1].data_ptr() for t in dests], rows_per_dest=200, head_stride=128,
                         token_stride=256)
    got = torch.cat([t[1].view(200, 2, 128) for t in dests], 0).permute(1, 0, 2).unsqueeze(0).float().cpu()
    assert O.rel_l2(got, ref) <= 1e-2 and all(bool((t[0] == 7.0).all()) for t in dests)
