"""The oracle against the golden vectors produced by the reference's own code
(tests/golden/make_golden.py).  CPU only."""
import math
import os

import pytest
import torch

from oracle import dax_oracle as O

FP8 = {"e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}


def load(golden_dir, name):
    return torch.load(os.path.join(golden_dir, name))


@pytest.mark.parametrize("name", ["bf16", "f16", "f32"])
def test_quantiser_bit_exact(golden_dir, name):
    g = load(golden_dir, f"quant_{name}.pt")
    q, s = O.quantize_rowwise(g["x"], torch.int8)
    assert torch.equal(q, g["q_int8"]) and torch.equal(s, g["s_int8"])
    for f, dt in FP8.items():
        q, s = O.quantize_rowwise(g["x"], dt)
        assert torch.equal(q.view(torch.uint8), g["q_" + f]) and torch.equal(s, g["s_" + f])


def test_quantiser_edge_rows(golden_dir):
    g = load(golden_dir, "quant_bf16.pt")
    # all-zero row: scale is floored at fp32 eps, values quantise to 0
    assert float(g["s_int8"][5]) == pytest.approx(torch.finfo(torch.float32).eps)
    assert int(g["q_int8"][5].abs().max()) == 0
    # constant row: every element maps to +127
    assert bool((g["q_int8"][6] == 127).all())


def test_extreme_code_is_minus_127_for_16bit_inputs():
    """Sweep every bf16 value of eight binades as the row maximum: rounding amax/127 to bf16 moves the
    scale by at most 2^-9 relative, so the largest code is +-127; the clamp bound -128 of the
    reference (quantize_to_int8) is never the result for a row's own maximum."""
    bits = torch.arange(0x3C00, 0x4400, dtype=torch.int32).to(torch.int16)
    vals = bits.view(torch.bfloat16)
    x = torch.stack([-vals, torch.zeros_like(vals)], 1)
    q, _ = O.quantize_rowwise(x, torch.int8)
    assert int(q[:, 0].min()) == -127 and int(q[:, 0].max()) == -127


@pytest.mark.parametrize("name", ["bf16", "f32"])
def test_weight_quantisation_bit_exact(golden_dir, name):
    g = load(golden_dir, f"weight_{name}.pt")
    q, s = O.quantize_weight(g["w"], torch.int8)
    assert torch.equal(q, g["qweight_int8"]) and torch.equal(s, g["wscale_int8"])
    q, s = O.quantize_weight(g["w"], torch.float8_e4m3fn)
    assert torch.equal(q.view(torch.uint8), g["qweight_e4m3"]) and torch.equal(s, g["wscale_e4m3"])


def test_int8_linear_bit_exact(golden_dir):
    g = load(golden_dir, "weight_bf16.pt")
    l = load(golden_dir, "linear_int8.pt")
    y = O.linear_int8(l["x"], g["qweight_int8"], g["wscale_int8"], g["b"], torch.bfloat16)
    assert y.dtype == l["y"].dtype and torch.equal(y, l["y"])


def test_int_matmul_is_exact():
    torch.manual_seed(0)
    a = torch.randint(-128, 128, (37, 512), dtype=torch.int8)
    b = torch.randint(-128, 128, (29, 512), dtype=torch.int8)
    ref = a.to(torch.int64) @ b.to(torch.int64).T
    assert torch.equal(O.int_matmul(a, b).to(torch.int64), ref)


def test_exchange_layouts(golden_dir):
    g = load(golden_dir, "layout.pt")
    P = len(g["shards"])
    for r in range(P):
        assert torch.equal(O.collect_tokens_ref(g["shards"], r), g["tokens"][r])
        assert torch.equal(O.collect_heads_ref(g["tokens"], r), g["heads"][r])
        assert torch.equal(g["heads"][r], g["shards"][r])  # the two exchanges are inverse


def test_micro_batches(golden_dir):
    g = load(golden_dir, "microbatch.pt")
    idx = O.micro_batch_indices(g["t"].shape[1], 2, 4)
    for i, ref in enumerate(g["mb"]):
        assert torch.equal(g["t"][:, idx[i]], ref)
    # concatenating each rank's slices in micro-batch order gives back that rank's block
    s = g["t"].shape[1] // 4
    for j in range(4):
        got = torch.cat([g["mb"][i][:, j * (s // 2):(j + 1) * (s // 2)] for i in range(2)], dim=1)
        assert torch.equal(got, g["t"][:, j * s:(j + 1) * s])


def test_rope_table_properties():
    grid = (3, 4, 5)
    fr = O.rope_table(grid)
    assert fr.shape == (1, 1, 60, 64) and O.rope_axis_dims(128) == (44, 42, 42)
    assert torch.allclose(fr.abs(), torch.ones_like(fr.abs()))
    assert torch.allclose(fr[0, 0, 0], torch.ones(64, dtype=fr.dtype))  # token (0,0,0) is not rotated
    # token (f, h, w): pair 0 rotates by f, pair 22 by h, pair 43 by w (frequency 1 each)
    f, h, w = 2, 3, 4
    t = (f * 4 + h) * 5 + w
    for pair, pos in ((0, f), (22, h), (43, w)):
        assert fr[0, 0, t, pair].angle().item() == pytest.approx(math.remainder(pos, 2 * math.pi), abs=1e-9)
    x = torch.randn(1, 2, 60, 128)
    y = O.apply_rotary_emb(x, fr)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), rtol=1e-5)  # rotations preserve norms


def test_rmsnorm_unit_rms():
    x = torch.randn(4, 7, 256) * 3
    y = O.rmsnorm(x, None)
    assert torch.allclose(y.pow(2).mean(-1), torch.ones(4, 7), atol=1e-4)


def test_sage_model_error_budget():
    """The quantised-attention model on config-2-like data: K offsets are removed by the smoothing,
    INT8 Q.K^T + FP8 P.V lands near 4e-2 rel-L2 / 0.9993 cosine, fp16 contractions near 1e-3."""
    torch.manual_seed(0)
    H, S = 2, 1024
    q = torch.randn(1, H, S, 128).bfloat16()
    v = torch.randn(1, H, S, 128).bfloat16()
    k = (torch.randn(1, H, S, 128) + 2 * torch.randn(1, H, 1, 128)).bfloat16()
    ref = O.sdpa_fp32(q, k, v)
    sage = O.sage_attention_model(q, k, v)
    assert O.cosine(sage, ref) >= 0.999 and O.rel_l2(sage, ref) < 5e-2
    hi = O.sage_attention_model(q, k, v, qk="f16", pv="f16")
    assert O.rel_l2(hi, ref) <= 1e-2 and O.cosine(hi, ref) >= 0.999


def test_block_int8_linear_error_vs_float():
    """Wan2.1-1.3B layer shape (1536 hidden, 12 heads): the quantised block stays within the
    quantisation error of the float block (sanity of the whole restatement)."""
    torch.manual_seed(0)
    S, D, H = 256, 1536, 12
    x = torch.randn(1, S, D)
    ws = [torch.randn(D, D) * 0.02 for _ in range(4)]
    zero = torch.zeros(D)
    lw = O.LayerWeights(*ws, zero, zero, zero, zero, torch.ones(D), torch.ones(D))
    fr = O.rope_table((1, 16, 16))
    y = O.self_attention_block(x, lw, H, fr, attention="sdpa")
    # float reference of the same block
    q = O.rmsnorm(x @ ws[0].T, torch.ones(D)).unflatten(2, (H, -1)).transpose(1, 2)
    k = O.rmsnorm(x @ ws[1].T, torch.ones(D)).unflatten(2, (H, -1)).transpose(1, 2)
    v = (x @ ws[2].T).unflatten(2, (H, -1)).transpose(1, 2)
    o = O.sdpa_fp32(O.apply_rotary_emb(q, fr), O.apply_rotary_emb(k, fr), v).transpose(1, 2).flatten(2, 3)
    yf = o @ ws[3].T
    assert O.rel_l2(y, yf) < 5e-2
