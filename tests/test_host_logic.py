"""Host-side logic on the CPU: module swap, qconfig propagation, state-dict names, error behaviour,
and the C-ABI library (loads, exports every declared symbol, validates arguments before launching)."""
import ctypes
import os
import re

import pytest
import torch
from torch import nn

from dax_b200 import _lib
from dax_b200.quant.nn.dynamic import Linear as QLinear
from dax_b200.quant.qscheme import get_block_size, per_channel_symmetric, per_tensor_symmetric, per_token_symmetric
from dax_b200.quant.quantization import (
    get_default_dynamic_int8_qconfig,
    get_dynamic_fp8_per_token_act_per_channel_weight_qconfig as fp8_cfg,
    get_dynamic_int8_per_token_act_per_channel_weight_qconfig as int8_cfg,
    quantize_dynamic,
)

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class Block(nn.Module):
    def __init__(self):
        super().__init__()
        self.to_q = nn.Linear(32, 32)
        self.proj_out = nn.Linear(32, 8)


class Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.blocks = nn.ModuleList([Block(), Block()])
        self.condition_embedder = nn.Sequential(nn.Linear(32, 32))
        self.proj_out = nn.Linear(32, 8)


def test_module_swap_matches_reference(golden_dir):
    net = Net()
    quantize_dynamic(net, {"": int8_cfg(), "condition_embedder": None, "proj_out": None})
    got = {n: (type(m).__name__, hasattr(m, "qweight")) for n, m in net.named_modules()}
    assert got == torch.load(os.path.join(golden_dir, "swap.pt"))
    assert not any(hasattr(m, "qconfig") for m in net.modules())


def test_swap_not_inplace_and_type_keys():
    net = Net()
    out = quantize_dynamic(net, {nn.Linear: int8_cfg()}, inplace=False)
    assert isinstance(out.proj_out, QLinear) and isinstance(net.proj_out, nn.Linear)


@pytest.mark.parametrize("name", ["bf16", "f32"])
def test_from_float_matches_reference(golden_dir, name):
    g = torch.load(os.path.join(golden_dir, f"weight_{name}.pt"))
    for cfg, qk, sk in ((int8_cfg(), "qweight_int8", "wscale_int8"),
                        (fp8_cfg(activation_dtype=torch.float8_e4m3fn), "qweight_e4m3", "wscale_e4m3")):
        m = nn.Linear(256, 192).to(g["w"].dtype)
        m.weight.data.copy_(g["w"])
        m.bias.data.copy_(g["b"])
        m.qconfig = cfg
        ql = QLinear.from_float(m)
        assert torch.equal(ql.qweight.view(torch.uint8), g[qk].view(torch.uint8))
        assert torch.equal(ql.weight_scale, g[sk]) and ql.weight_scale.shape == (1, 192)
        assert set(ql.state_dict()) == {"qweight", "weight_scale", "bias"}
        assert not hasattr(m, "weight")  # the float weight is released
    assert ql.bias.dtype == torch.bfloat16  # FP8 row-wise linears keep a bf16 bias


def test_state_dict_round_trip():
    m = nn.Linear(64, 48).bfloat16()
    m.qconfig = int8_cfg()
    a = QLinear.from_float(m)
    b = QLinear(64, 48, True, None, torch.int8, torch.int8, torch.bfloat16, per_channel_symmetric, per_token_symmetric)
    b.load_state_dict(a.state_dict())
    assert torch.equal(a.qweight, b.qweight) and torch.equal(a.weight_scale, b.weight_scale)
    assert torch.allclose(a.weight.float(), a.qweight.float() * a.weight_scale.T, rtol=2e-2, atol=1e-6)


def test_fp8_default_activation_is_e5m2():
    assert fp8_cfg().activation().dtype == torch.float8_e5m2
    assert fp8_cfg(activation_dtype=torch.float8_e4m3fn).activation().dtype == torch.float8_e4m3fn


def test_bad_combinations_raise():
    with pytest.raises(ValueError):
        QLinear(8, 8, True, None, torch.int8, torch.float8_e4m3fn, torch.bfloat16, per_channel_symmetric, per_token_symmetric)
    with pytest.raises(ValueError):
        QLinear(8, 8, True, None, torch.float8_e4m3fn, torch.float8_e4m3fn, torch.bfloat16, per_channel_symmetric,
                per_tensor_symmetric)
    m = nn.Linear(16, 16)
    m.qconfig = get_default_dynamic_int8_qconfig()
    q = QLinear.from_float(m)  # per-tensor scheme: swap works, forward is rejected before any launch
    with pytest.raises(NotImplementedError):
        q._check_supported()


def test_no_cpu_fallback():
    m = nn.Linear(32, 32).bfloat16()
    m.qconfig = int8_cfg()
    q = QLinear.from_float(m)
    with pytest.raises(RuntimeError, match="CUDA"):
        q(torch.randn(20, 32).bfloat16())
    from dax_b200.adapters.wan import DAXWanAttnProcessor2_0
    from dax_b200.adapters.wan.modules import Attention
    attn = Attention(256, 2)
    proc = DAXWanAttnProcessor2_0()
    with pytest.raises(RuntimeError, match="CUDA"):
        proc(attn, torch.randn(1, 8, 256).bfloat16())
    with pytest.raises(NotImplementedError):
        proc(attn, torch.randn(1, 8, 256).bfloat16(), attention_mask=torch.ones(1))


def test_optimize_pipe_argument_checks():
    from dax_b200.adapters.wan import optimize_pipe
    from dax_b200.adapters.wan.modules import WanSelfAttentionStack, _Pipe
    pipe = _Pipe(WanSelfAttentionStack(1, 256, 2))
    with pytest.raises(ValueError, match="Overlap"):
        optimize_pipe(pipe, sequence_parallel=False, overlap_comm=True)
    optimize_pipe(pipe, sequence_parallel=False, overlap_comm=False, int8_linear=True)
    blk = pipe.transformer.blocks[0]
    assert isinstance(blk.to_q, QLinear) and isinstance(blk.to_out[0], QLinear)
    assert type(blk.processor).__name__ == "DAXWanAttnProcessor2_0"


def test_block_sizes():
    assert get_block_size((2, 3, 8), per_token_symmetric) == (1, 1, 8)
    assert get_block_size((4, 8), per_channel_symmetric) == (4, 1)
    assert get_block_size((4, 8), per_tensor_symmetric) == (4, 8)
    with pytest.raises(ValueError):
        get_block_size((4, 8), "nope")


# ---- C ABI ---------------------------------------------------------------------------------------
def declared_symbols():
    text = open(os.path.join(ROOT, "include", "dax_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dax_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(built_library):
    lib = ctypes.CDLL(built_library)
    names = declared_symbols()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/dax_b200.h but not exported"
    assert set(names) == set(_lib.SIGNATURES), "python prototypes and the header disagree"


def test_library_validates_before_launching(built_library):
    lib = _lib.load()
    assert lib.dax_version() >= 100
    one = ctypes.c_void_p(4096)  # never dereferenced: validation fails first
    # K not a multiple of 16
    assert lib.dax_quant_rowwise(one, _lib.DAX_BF16, 4, 24, 24, 24, 0, one, _lib.DAX_I8, one, None) == _lib.DAX_ERR_ALIGN
    assert b"multiple of 16" in lib.dax_last_error()
    # unknown dtype
    assert lib.dax_quant_rowwise(one, 99, 4, 32, 32, 32, 0, one, _lib.DAX_I8, one, None) == _lib.DAX_ERR_UNSUPPORTED
    # mixed INT8 / FP8 operands
    rc = lib.dax_gemm_dequant(one, _lib.DAX_I8, one, one, _lib.DAX_E4M3, one, None, 0, one, _lib.DAX_BF16, 32, 32, 32, 32,
                              32, 0, None, None, None)
    assert rc == _lib.DAX_ERR_UNSUPPORTED
    with pytest.raises(NotImplementedError):
        _lib.check(rc)
    # null pointer
    assert lib.dax_gemm_dequant(None, _lib.DAX_I8, one, one, _lib.DAX_I8, one, None, 0, one, _lib.DAX_BF16, 32, 32, 32, 32,
                                32, 0, None, None, None) == _lib.DAX_ERR_INVALID
    # empty problem is a no-op
    assert lib.dax_quant_rowwise(one, _lib.DAX_BF16, 0, 32, 32, 32, 0, one, _lib.DAX_I8, one, None) == _lib.DAX_OK
    assert lib.dax_attn_workspace_bytes(1, 2, 300, 300, 0) > 0
    assert lib.dax_attn_workspace_bytes(1, 2, 0, 300, 0) == 0


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_LIB", None)
    monkeypatch.setattr(_lib, "library_path", lambda: str(tmp_path / "absent.so"))
    with pytest.raises(_lib.DaxLibraryError, match="no CPU"):
        _lib.load()


def test_rope_table_cache_survives_address_reuse():
    """Two rotary tables of identical shape and different content, the second allocated after the first was
    dropped (the allocator may hand out the same address): each gets its own cos/sin; an in-place update of a
    cached table is noticed through the version counter."""
    from dax_b200.adapters.wan.attn_adapter import _rope_tables
    from dax_b200.adapters.wan.modules import wan_rope_table
    seen = []
    for grid in ((2, 3, 4), (2, 4, 3), (4, 3, 2)):
        table = wan_rope_table(grid).clone()
        cos, sin = _rope_tables(table)
        want = torch.view_as_real(table.reshape(-1, 64))
        assert torch.equal(cos, want[..., 0].float()) and torch.equal(sin, want[..., 1].float())
        seen.append(cos)
        del table
    assert not torch.equal(seen[0], seen[1])
    table = wan_rope_table((2, 3, 4)).clone()
    cos0, _ = _rope_tables(table)
    table.mul_(1j)  # rotate every entry by 90 degrees, in place
    cos1, sin1 = _rope_tables(table)
    assert torch.allclose(cos1, -torch.view_as_real(wan_rope_table((2, 3, 4)).reshape(-1, 64))[..., 1].float())
    assert not torch.equal(cos0, cos1)


def test_unknown_cache_strategy_disables_teacache():
    from dax_b200.adapters.wan.transformer_adapter import replace_transformer

    class T(nn.Module):
        pass

    t = replace_transformer(T(), cache_strategy="something_else")
    assert type(t).enable_teacache is False


def test_scatter_entry_points_validate_their_pointer_tables(built_library):
    """The *_scatter entry points reject a bad table of group pointers before anything is launched."""
    lib = _lib.load()
    one = ctypes.c_void_p(4096)

    def table(*vals):
        return (ctypes.c_void_p * len(vals))(*vals)

    args = (one, _lib.DAX_BF16, 4, 512, 512, None, 0, 0, None, ctypes.c_float(1e-6), None, None, 0)
    # nine groups: more than the table holds
    assert lib.dax_rmsnorm_rope_pack_scatter(*args, table(*([4096] * 9)), 9, 64, 64, None) == _lib.DAX_ERR_INVALID
    assert b"group pointers" in lib.dax_last_error()
    # a pointer that is not 16-byte aligned, a null entry
    assert lib.dax_rmsnorm_rope_pack_scatter(*args, table(4096, 4104), 2, 256, 256, None) == _lib.DAX_ERR_ALIGN
    assert lib.dax_rmsnorm_rope_pack_scatter(*args, table(4096, None), 2, 256, 256, None) == _lib.DAX_ERR_ALIGN
    # number of pointers must equal the number of column groups
    assert lib.dax_rmsnorm_rope_pack_scatter(*args, table(4096, 8192, 12288), 3, 256, 256, None) == _lib.DAX_ERR_INVALID
    rc = lib.dax_gemm_dequant_scatter(one, _lib.DAX_I8, one, one, _lib.DAX_I8, one, None, 0, table(4096, 8192, 12288), 3,
                                      _lib.DAX_BF16, 32, 512, 64, 256, 256, None)
    assert rc == _lib.DAX_ERR_INVALID
    # attention rows: destinations must cover every query row
    ws_bytes = lib.dax_attn_workspace_bytes(1, 2, 300, 300, _lib.DAX_ATTN_QK_BF16_PV_BF16)
    rc = lib.dax_attn_forward_scatter(table(4096, 8192), 2, 100, _lib.DAX_BF16, 2, 300, 300, 128, 256, 0, 300,
                                      _lib.DAX_ATTN_QK_BF16_PV_BF16, ctypes.c_void_p(1 << 20), ws_bytes, None)
    assert rc == _lib.DAX_ERR_INVALID and b"destinations" in lib.dax_last_error()
    assert lib.dax_peer_copy(None, one, 16, None) == _lib.DAX_ERR_INVALID
    assert lib.dax_peer_copy(one, one, 0, None) == _lib.DAX_OK
