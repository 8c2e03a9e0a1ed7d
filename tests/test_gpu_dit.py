"""The kernels and adapters around the hot path (next-tier rows): LayerNorm+modulate+quantise, the GEMM's
GELU / gated-residual epilogues, the fused Wan block, and a small DiT forward with sequence split, against the
oracle.  Needs a B200."""
import pytest
import torch
import torch.nn.functional as F

from oracle import dax_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ops(built_library):
    if not torch.cuda.is_available():
        pytest.fail("the gpu tests need a CUDA device")
    from dax_b200 import ops as _ops
    return _ops


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("D", [256, 1024, 1536, 2048, 3072, 4096, 5120, 6144])
def test_layernorm_modulate_quant(ops, dtype, D):
    torch.manual_seed(D)
    s = 45
    x = (torch.randn(s, D) * 3 + 0.5).to(dtype)
    w, b = 1 + 0.1 * torch.randn(D), 0.1 * torch.randn(D)
    shift, scale = 0.2 * torch.randn(D), 0.2 * torch.randn(D)
    for kw, ref in (
        (dict(shift=shift, scale=scale), (O.layernorm(x) * (1 + scale) + shift).to(dtype)),
        (dict(ln_weight=w, ln_bias=b), O.layernorm(x, w, b).to(dtype)),
        (dict(), O.layernorm(x).to(dtype)),
    ):
        dkw = {k: v.to(DEV) for k, v in kw.items()}
        y, _, _ = ops.layernorm_modulate_quant(x.to(DEV), **dkw)
        assert O.rel_l2(y.cpu(), ref) <= 3e-3 and (y.cpu().float() - ref.float()).abs().max() <= 0.05
        for qd in (torch.int8, torch.float8_e4m3fn):
            y2, q, qs = ops.layernorm_modulate_quant(x.to(DEV), q_dtype=qd, **dkw)
            assert torch.equal(y2, y)
            # the fused codes are exactly the quantiser applied to the kernel's own y
            qr, sr = O.quantize_rowwise(y.cpu(), qd)
            assert torch.equal(q.cpu().view(torch.uint8), qr.view(torch.uint8)) and torch.equal(qs.cpu(), sr)
            _, q3, qs3 = ops.layernorm_modulate_quant(x.to(DEV), q_dtype=qd, want_y=False, **dkw)
            assert torch.equal(q3, q) and torch.equal(qs3, qs)


def test_layernorm_modulate_quant_many_rows(ops):
    """More rows than resident CTAs at the production width: the row loop with prefetch, against the oracle and
    against the same rows processed one at a time."""
    torch.manual_seed(9)
    s, D = 2000, 5120
    x = (torch.randn(s, D) * torch.logspace(-1, 1.5, s).unsqueeze(1) + 0.3).bfloat16()
    shift, scale = 0.2 * torch.randn(D), 0.2 * torch.randn(D)
    ref = (O.layernorm(x) * (1 + scale) + shift).bfloat16()
    y, q, qs = ops.layernorm_modulate_quant(x.to(DEV), shift=shift.to(DEV), scale=scale.to(DEV), q_dtype=torch.float8_e4m3fn)
    assert O.rel_l2(y.cpu(), ref) <= 3e-3
    qr, sr = O.quantize_rowwise(y.cpu(), torch.float8_e4m3fn)
    assert torch.equal(q.cpu().view(torch.uint8), qr.view(torch.uint8)) and torch.equal(qs.cpu(), sr)
    for i in (0, 1, 295, 296, 443, 444, 1999):
        yi, qi, si = ops.layernorm_modulate_quant(x[i:i + 1].to(DEV), shift=shift.to(DEV), scale=scale.to(DEV),
                                                  q_dtype=torch.float8_e4m3fn)
        assert torch.equal(yi[0], y[i]) and torch.equal(qi[0], q[i]) and torch.equal(si[0], qs[i])


@pytest.mark.parametrize("D", [256, 5120])
def test_layernorm_strided_rows(ops, D):
    """Rows that are a column slice of a wider matrix (leading dimension larger than the width): same results as the
    contiguous copy, in both kernels."""
    torch.manual_seed(11)
    s = 300
    wide = torch.randn(s, D + 64).bfloat16().to(DEV)
    xs = wide[:, :D]
    assert xs.stride(0) == D + 64
    shift, scale = (0.2 * torch.randn(D)).to(DEV), (0.2 * torch.randn(D)).to(DEV)
    for qd in (torch.int8, torch.float8_e4m3fn):
        y0, q0, s0 = ops.layernorm_modulate_quant(xs.contiguous(), shift=shift, scale=scale, q_dtype=qd)
        y1, q1, s1 = ops.layernorm_modulate_quant(xs, shift=shift, scale=scale, q_dtype=qd)
        assert torch.equal(y0, y1) and torch.equal(q0, q1) and torch.equal(s0, s1)


@pytest.mark.parametrize("D", [5120, 1000 * 8])
def test_layernorm_rows_with_a_large_mean(ops, D):
    """Rows whose mean dwarfs their spread (E[x^2] - mean^2 would cancel) and a constant row: the centred form must
    take over.  fp16 input, whose spacing near 100 is fine enough to carry a spread of 0.1.  Both kernels (a width
    that fills a CTA exactly, and one that does not)."""
    torch.manual_seed(21)
    s = 37
    x = (100.0 + 0.1 * torch.randn(s, D)).half()
    x[5] = 3.0
    x[6] = 0.0
    ref = O.layernorm(x).half()
    y, q, qs = ops.layernorm_modulate_quant(x.to(DEV), q_dtype=torch.int8)
    assert torch.isfinite(y).all()
    assert O.rel_l2(y.cpu(), ref) <= 3e-3
    assert float(y[5].abs().max()) <= 1e-3 and float(y[6].abs().max()) == 0.0
    qr, sr = O.quantize_rowwise(y.cpu(), torch.int8)
    assert torch.equal(q.cpu(), qr) and torch.equal(qs.cpu(), sr)


@pytest.mark.parametrize("wdt", [torch.int8, torch.float8_e4m3fn])
def test_gemm_epilogues(ops, wdt):
    torch.manual_seed(3)
    M, N, K = 300, 768, 512
    x = torch.randn(M, K).bfloat16()
    w = (torch.randn(N, K) * 0.05).bfloat16()
    b = (torch.randn(N) * 0.1).bfloat16()
    resid = torch.randn(M, N).bfloat16()
    gate = torch.randn(N)
    qw, sw = O.quantize_weight(w, wdt)
    qx, sx = O.quantize_rowwise(x, wdt)
    lin = (O.linear_int8(x, qw, sw, b, torch.bfloat16) if wdt == torch.int8
           else O.linear_fp8(x, qw, sw, b, torch.bfloat16, wdt))
    args = (qx.to(DEV), sx.to(DEV), qw.to(DEV), sw.to(DEV).reshape(-1).contiguous(), b.to(DEV), torch.bfloat16)
    y = ops.gemm_dequant(*args, act="gelu_tanh")
    ref = F.gelu(lin.float(), approximate="tanh").bfloat16()
    assert O.rel_l2(y.cpu(), ref) <= 2e-3
    y = ops.gemm_dequant(*args, resid=resid.to(DEV), gate=gate.to(DEV))
    ref = (resid.float() + gate * lin.float()).bfloat16()
    assert O.rel_l2(y.cpu(), ref) <= 2e-3
    # the kernel fuses gate * y + resid into one FMA (one fp32 rounding, torch has two): a few bf16 ties differ
    assert (y.cpu() != ref).float().mean() < 1e-3
    out = resid.to(DEV).clone()
    ops.gemm_dequant(*args, out=out, ldo=N, resid=out)  # in place, no gate
    assert O.rel_l2(out.cpu(), (resid.float() + lin.float()).bfloat16()) <= 2e-3
    with pytest.raises(NotImplementedError):
        ops.gemm_dequant(*args[:5], torch.float32, act="gelu_tanh")


def build_dit(layers=2, dim=256, ffn=512, heads=2, text_dim=64, seed=0):
    from dax_b200.adapters.wan.modules import WanDiT, init_wan_weights_
    torch.manual_seed(seed)
    m = WanDiT(layers=layers, dim=dim, ffn_dim=ffn, heads=heads, text_dim=text_dim)
    init_wan_weights_(m, 0.05, seed)
    g = torch.Generator().manual_seed(seed + 1)
    with torch.no_grad():
        for n_, p in m.named_parameters():
            if n_.endswith("bias") and p.dim() == 1:
                p.copy_(0.05 * torch.randn(p.shape, generator=g))
            if "norm_q.weight" in n_ or "norm_k.weight" in n_ or n_.endswith("norm2.weight"):
                p.copy_(1 + 0.1 * torch.randn(p.shape, generator=g))
    return m.bfloat16()


def oracle_block(blk, wdt, adt):
    ql = lambda lin: O.QuantLinear(lin.weight.detach().cpu(), lin.bias.detach().cpu(), wdt, adt)
    a = lambda at: (ql(at.to_q), ql(at.to_k), ql(at.to_v), ql(at.to_out[0]), at.norm_q.weight.detach().cpu(),
                    at.norm_k.weight.detach().cpu())
    return dict(table6=blk.scale_shift_table.detach().cpu(), attn1=a(blk.attn1), attn2=a(blk.attn2),
                norm2_w=blk.norm2.weight.detach().cpu(), norm2_b=blk.norm2.bias.detach().cpu(),
                ffn_up=ql(blk.ffn.net[0].proj), ffn_down=ql(blk.ffn.net[2]))


@pytest.mark.parametrize("linear", ["int8", "fp8_e4m3"])
def test_fused_block_matches_oracle(ops, linear):
    from dax_b200.adapters.wan import optimize_pipe
    from dax_b200.adapters.wan.modules import _Pipe, wan_rope_table
    wdt = torch.int8 if linear == "int8" else torch.float8_e4m3fn
    m = build_dit(layers=1)
    blk = m.blocks[0]
    ob = oracle_block(blk, wdt, wdt)
    grid, D, H = (2, 8, 8), 256, 2
    S = 128
    g = torch.Generator().manual_seed(9)
    h = torch.randn(1, S, D, generator=g).bfloat16()
    ctx = torch.randn(1, 19, D, generator=g).bfloat16()
    temb = (0.3 * torch.randn(1, 6, D, generator=g)).bfloat16()
    fr = O.rope_table(grid)
    ref = O.wan_block(h, ctx, temb, heads=H, freqs=fr, **ob)
    pipe = _Pipe(m.to(DEV))
    optimize_pipe(pipe, sequence_parallel=False, compile=False, overlap_comm=False, int8_linear=linear == "int8",
                  fp8_linear=linear != "int8", attention_mode="bf16")
    y = blk(h.to(DEV), ctx.to(DEV), temb.to(DEV), wan_rope_table(grid, device=DEV))
    assert y.shape == h.shape and y.dtype == torch.bfloat16
    # quantised linears re-quantise slightly different inputs at every stage: FP8 (3-bit mantissa) amplifies more
    tol = 1.5e-2 if linear == "int8" else 3e-2
    assert O.cosine(y.cpu(), ref) >= 0.999 and O.rel_l2(y.cpu(), ref) <= tol, O.rel_l2(y.cpu(), ref)


def test_fused_block_equals_unfused_composition(ops):
    """The fused forward against the plain torch composition of the same (quantised) modules on the GPU."""
    from dax_b200.adapters.wan import optimize_pipe
    from dax_b200.adapters.wan.modules import WanTransformerBlock, _Pipe, wan_rope_table
    m = build_dit(layers=1, seed=4)
    pipe = _Pipe(m.to(DEV))
    optimize_pipe(pipe, sequence_parallel=False, compile=False, overlap_comm=False, int8_linear=True,
                  attention_mode="bf16")
    blk = m.blocks[0]
    g = torch.Generator().manual_seed(2)
    h = torch.randn(2, 300, 256, generator=g).bfloat16().to(DEV)
    ctx = torch.randn(2, 33, 256, generator=g).bfloat16().to(DEV)
    temb = (0.3 * torch.randn(2, 6, 256, generator=g)).bfloat16().to(DEV)
    fused = blk(h, ctx, temb, None)
    plain = WanTransformerBlock.forward(blk, h, ctx, temb, None)
    assert O.rel_l2(fused.float().cpu(), plain.float().cpu()) <= 1e-2


def test_fused_block_without_cross_attention_norm(ops):
    """cross_attn_norm=False makes norm2 an identity: the fused forward must skip that LayerNorm (and still
    quantise the cross-attention input) instead of applying a default one."""
    from dax_b200.adapters.wan import optimize_pipe
    from dax_b200.adapters.wan.modules import WanTransformerBlock, _Pipe
    m = build_dit(layers=1, seed=8)
    m.blocks[0].norm2 = torch.nn.Identity()
    pipe = _Pipe(m.to(DEV))
    optimize_pipe(pipe, sequence_parallel=False, compile=False, overlap_comm=False, int8_linear=True,
                  attention_mode="bf16")
    blk = m.blocks[0]
    g = torch.Generator().manual_seed(3)
    h = torch.randn(1, 200, 256, generator=g).bfloat16().to(DEV)
    ctx = torch.randn(1, 33, 256, generator=g).bfloat16().to(DEV)
    temb = (0.3 * torch.randn(1, 6, 256, generator=g)).bfloat16().to(DEV)
    fused = blk(h, ctx, temb, None)
    plain = WanTransformerBlock.forward(blk, h, ctx, temb, None)
    assert O.rel_l2(fused.float().cpu(), plain.float().cpu()) <= 1e-2


def test_dit_forward_and_teacache(ops):
    """A small DiT through `optimize_pipe` (fused blocks, INT8 linears, bf16 attention) against the oracle's
    restatement of the reference forward (patch embedding, condition embedder, quantised blocks with fp32 SDPA,
    modulated output norm, projection, unpatchify); then the TeaCache path: a skipped step returns input +
    cached residual without running the blocks."""
    from dax_b200.adapters.wan import optimize_pipe
    from dax_b200.adapters.wan.modules import _Pipe
    m = build_dit(layers=2, seed=7)
    sd = {k: v.detach().clone() for k, v in m.state_dict().items()}
    g = torch.Generator().manual_seed(21)
    lat_c = torch.randn(1, 16, 2, 16, 16, generator=g).bfloat16()
    text_c = torch.randn(1, 11, 64, generator=g).bfloat16()
    ref = O.dit_forward(lat_c, torch.tensor([321]), text_c, sd, heads=2).float()
    m = m.to(DEV)
    lat, text, t = lat_c.to(DEV), text_c.to(DEV), torch.tensor([321], device=DEV)
    pipe = _Pipe(m)
    optimize_pipe(pipe, sequence_parallel=False, compile=False, overlap_comm=False, int8_linear=True,
                  attention_mode="bf16", cache_strategy="teacache", teacache_thresh=1e9, num_inference_steps=4)
    with torch.no_grad():
        out = m(lat, t, text, return_dict=True).sample.float().cpu()
    assert out.shape == lat.shape
    assert O.cosine(out, ref) >= 0.999 and O.rel_l2(out, ref) <= 2e-2, O.rel_l2(out, ref)
    # ret_steps = 10 calls always compute; with an infinite threshold every later call before the cut-off skips
    cls = type(m)
    cls.ret_steps, cls.cutoff_steps = 2, 100
    m.cnt = 0
    with torch.no_grad():
        outs = [m(lat, t, text, return_dict=False)[0] for _ in range(4)]
    # call 2 (even branch) is skipped: input + residual cached by call 0, equal to call 0 up to bf16 rounding
    assert m.should_calc_even is False and m.should_calc_odd is False
    assert O.rel_l2(outs[2].float().cpu(), outs[0].float().cpu()) <= 1e-2
    cls.enable_teacache = False


def test_denoise_loop_with_teacache(ops):
    """Ten guided denoising steps of a small DiT through the optimised forward: the cache must skip some of the
    twenty forwards, never during the first ten calls, and the sample must stay finite and close to the one
    computed without the cache."""
    from dax_b200.adapters.wan import optimize_pipe
    from dax_b200.adapters.wan.modules import _Pipe
    from dax_b200.adapters.wan.sampling import denoise
    from dax_b200.cache import teacache
    m = build_dit(layers=2, seed=11).to(DEV)
    pipe = _Pipe(m)
    optimize_pipe(pipe, sequence_parallel=False, compile=False, overlap_comm=False, int8_linear=True,
                  attention_mode="bf16")
    g = torch.Generator().manual_seed(5)
    lat = torch.randn(1, 16, 2, 16, 16, generator=g).bfloat16().to(DEV)
    pos = torch.randn(1, 11, 64, generator=g).bfloat16().to(DEV)
    neg = torch.randn(1, 11, 64, generator=g).bfloat16().to(DEV)
    plain = denoise(pipe, lat, pos, neg, num_inference_steps=10, guidance_scale=3.0, flow_shift=3.0)
    teacache.configure(m, teacache_thresh=0.05, num_inference_steps=10)
    calc = []
    cached = denoise(pipe, lat, pos, neg, num_inference_steps=10, guidance_scale=3.0, flow_shift=3.0,
                     on_step=lambda i, x: calc.append((bool(m.should_calc_even), bool(m.should_calc_odd))))
    type(m).enable_teacache = False
    assert m.cnt == 20 and len(calc) == 10
    assert all(c == (True, True) for c in calc[:5])      # ret_steps = 10 forwards
    assert torch.isfinite(cached.float()).all() and torch.isfinite(plain.float()).all()
    if any(c != (True, True) for c in calc):             # skipped forwards reuse a residual: close, not equal
        assert O.rel_l2(cached.float().cpu(), plain.float().cpu()) <= 0.2
    else:
        assert torch.equal(cached, plain)
