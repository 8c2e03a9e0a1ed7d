"""The benchmark configurations at their stated sizes, through the C ABI, against the oracle on row / slice
samples (the full problems are far too large for the CPU): the standalone attention at 40 heads x 32,760 tokens
with a per-channel K offset, and the dynamic-linear sweep at M = 75,600 rows.  Needs a B200."""
import pytest
import torch

from oracle import dax_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"

# tolerance against fp32 SDPA: (rel-L2, cosine).  Only the 16-bit mode is held to the stated contract
# (rel-L2 <= 1e-2, cosine >= 0.999); the two quantised modes are labelled with what their operand formats allow
# on Gaussian data (single-term e4m3 P and V: about 3.7e-2; INT8 Q.K^T alone: about 1e-2).
ATTN_BOUNDS = {"bf16": (1e-2, 0.999), "int8_bf16": (2e-2, 0.999), "sage": (5e-2, 0.999)}


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


@pytest.fixture(scope="module")
def attention_problem():
    """B=1, 40 heads, head_dim 128, S=32,760 (grid 21x30x52): Q, V ~ N(0,1), K ~ N(0,1) + per-channel offset of
    std 2 broadcast over the tokens; fp32 SDPA on three slices of query rows (first tile, a middle tile that
    straddles two 256-row CTAs, the ragged last tile)."""
    S, H = 32760, 40
    g = torch.Generator().manual_seed(2)
    q = torch.randn(1, H, S, 128, generator=g).bfloat16()
    k = (torch.randn(1, H, S, 128, generator=g) + 2.0 * torch.randn(1, H, 1, 128, generator=g)).bfloat16()
    v = torch.randn(1, H, S, 128, generator=g).bfloat16()
    idx = torch.cat([torch.arange(0, 96), torch.arange(16300, 16396), torch.arange(S - 96, S)])
    ref = O.sdpa_fp32(q[:, :, idx], k, v)
    return q.to(DEV), k.to(DEV), v.to(DEV), idx, ref


@pytest.mark.parametrize("mode", ["bf16", "int8_bf16", "sage"])
def test_standalone_attention_40_heads_32760_tokens(ops, attention_problem, mode):
    q, k, v, idx, ref = attention_problem
    o = ops.attention(q, k, v, mode=mode)
    assert torch.isfinite(o.float()).all()
    got = o[:, :, idx.to(DEV)].float().cpu()
    rel, cos = O.rel_l2(got, ref), O.cosine(got, ref)
    bound_rel, bound_cos = ATTN_BOUNDS[mode]
    assert rel <= bound_rel and cos >= bound_cos, (mode, rel, cos)
    # per slice too: an error confined to the ragged last tile must not hide in the average
    for lo in (0, 96, 192):
        assert O.rel_l2(got[:, :, lo:lo + 96], ref[:, :, lo:lo + 96]) <= bound_rel, (mode, lo)


LINEAR_SHAPES = [(5120, 5120), (5120, 13824), (13824, 5120), (4096, 5120)]  # K -> N


@pytest.mark.parametrize("K,N", LINEAR_SHAPES)
@pytest.mark.parametrize("arith", ["int8", "fp8_e4m3"])
def test_dynamic_linear_at_75600_rows(ops, K, N, arith):
    """x bf16 ~ N(0,1) [75,600, K], W ~ N(0, 0.02), through the one-call dynamic linear (quantiser + GEMM).  A sample
    of rows against the oracle: INT8 bit-exact outputs; FP8 outputs within bf16 rounding and raw accumulators within
    1e-5 of exact products of the same codes."""
    M = 75600
    wdt = torch.int8 if arith == "int8" else torch.float8_e4m3fn
    g = torch.Generator(device=DEV).manual_seed(K + N)
    x = torch.randn(M, K, generator=g, device=DEV).bfloat16()
    w = (torch.randn(N, K, generator=g, device=DEV) * 0.02).bfloat16().cpu()
    b = (torch.randn(N, generator=g, device=DEV) * 0.1).bfloat16().cpu()
    qw, sw = O.quantize_weight(w, wdt)
    swd = sw.to(DEV).reshape(-1).contiguous()
    y = ops.linear_dynamic(x, qw.to(DEV), swd, b.to(DEV), wdt, torch.bfloat16)
    idx = torch.cat([torch.arange(0, M, 2521), torch.tensor([127, 128, M - 81, M - 1])])  # 34 rows, incl. the ragged last tile
    xs = x[idx.to(DEV)].cpu()
    got = y[idx.to(DEV)].cpu()
    if arith == "int8":
        want = O.linear_int8(xs, qw, sw, b, torch.bfloat16)
        assert torch.equal(got, want)
    else:
        want = O.linear_fp8(xs, qw, sw, b, torch.bfloat16, wdt)
        assert O.rel_l2(got, want) <= 2e-3 and O.cosine(got, want) >= 0.99999
        assert (got != want).float().mean() < 0.02  # a few bf16 ties from the fp32 summation order
    del y
    # the two launches separately, with the raw accumulators of the full-size GEMM
    qx, sx = ops.quant_rowwise(x, wdt)
    qxr, sxr = O.quantize_rowwise(xs, wdt)
    bits = (lambda t: t.view(torch.uint8)) if arith != "int8" else (lambda t: t)
    assert torch.equal(bits(qx[idx.to(DEV)].cpu()), bits(qxr)) and torch.equal(sx[idx.to(DEV)].cpu(), sxr)
    dump = torch.empty(M, N, dtype=torch.int32 if arith == "int8" else torch.float32, device=DEV)
    ops.gemm_dequant(qx, sx, qw.to(DEV), swd, None, torch.bfloat16, acc_dump=dump)
    acc = dump[idx.to(DEV)].cpu()
    if arith == "int8":
        assert torch.equal(acc, O.int_matmul(qxr, qw))
    else:
        exact = qxr.double() @ qw.double().T
        assert O.rel_l2(acc, exact) <= 1e-5
