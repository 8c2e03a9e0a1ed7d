"""The allocation-free dynamic linear (dax_linear_dynamic_static) against the workspace-taking entry
point (dax_linear_dynamic), through the C ABI.

Who needs it: hosts that give the library only inputs and outputs and may not call cudaMalloc while a
layer runs (a runtime with a fixed memory pool, a foreign-language binding without a CUDA allocator).
The test makes two calls in a row, the second smaller than the first, so that stale bytes left in the
shared built-in buffer by the first call would show up if the second depended on them, and requires
bit-identical outputs (the same two kernels run in both entry points).  This file sorts last on
purpose: a run that stops at the first failure has then already run every other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"
LIMIT = 8 << 20


def _inputs(M, N, K, seed, fp8):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g).bfloat16().to(DEV)
    if fp8:
        qw = (torch.randn(N, K, generator=g) * 60).clamp(-448, 448).to(torch.float8_e4m3fn).to(DEV)
    else:
        qw = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8).to(DEV)
    sw = (torch.rand(N, generator=g) * 1e-3 + 1e-4).to(DEV)
    bias = (torch.randn(N, generator=g) * 0.1).bfloat16().to(DEV)
    return x, qw, sw, bias


def _call_pair(lib, _lib, M, N, K, seed, fp8):
    x, qw, sw, bias = _inputs(M, N, K, seed, fp8)
    wdt = _lib.DAX_E4M3 if fp8 else _lib.DAX_I8
    stream = torch.cuda.current_stream().cuda_stream
    # existing entry point, workspace from torch
    n = lib.dax_linear_dynamic_workspace_bytes(M, K)
    ws = torch.empty(n + 256, dtype=torch.uint8, device=DEV)
    off = (-ws.data_ptr()) % 256
    ref = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    _lib.check(lib.dax_linear_dynamic(x.data_ptr(), _lib.DAX_BF16, M, K, K, qw.data_ptr(), wdt, wdt, sw.data_ptr(),
                                      bias.data_ptr(), _lib.DAX_BF16, ref.data_ptr(), _lib.DAX_BF16, N, N,
                                      ws.data_ptr() + off, n, stream))
    # allocation-free entry point: inputs and outputs only
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    _lib.check(lib.dax_linear_dynamic_static(x.data_ptr(), _lib.DAX_BF16, M, K, K, qw.data_ptr(), wdt, wdt, sw.data_ptr(),
                                             bias.data_ptr(), _lib.DAX_BF16, out.data_ptr(), _lib.DAX_BF16, N, N, stream))
    torch.cuda.synchronize()
    return out, ref


@pytest.mark.parametrize("fp8", [False, True])
def test_static_linear_matches_workspace_linear_twice(built_library, fp8):
    if not torch.cuda.is_available():
        pytest.fail("the gpu tests need a CUDA device")
    from dax_b200 import _lib
    lib = _lib.load()
    # first call: the 512 x 4096 text-context projection shape; second call: smaller and ragged
    for M, N, K, seed in ((512, 5120, 4096, 11), (77, 264, 208, 12)):
        out, ref = _call_pair(lib, _lib, M, N, K, seed, fp8)
        assert torch.isfinite(out.float()).all()
        assert torch.equal(out, ref), f"outputs differ for M={M} N={N} K={K}"
    assert _lib.device_status() == 0


def test_static_linear_rejects_oversized_problems(built_library):
    if not torch.cuda.is_available():
        pytest.fail("the gpu tests need a CUDA device")
    from dax_b200 import _lib
    lib = _lib.load()
    M, K = 4096, 4096  # 16 MiB of codes: beyond the built-in 8 MiB
    assert lib.dax_linear_dynamic_workspace_bytes(M, K) > LIMIT
    one = ctypes.c_void_p(4096)  # never dereferenced: the size check comes first
    rc = lib.dax_linear_dynamic_static(one, _lib.DAX_BF16, M, K, K, one, _lib.DAX_I8, _lib.DAX_I8, one, None, 0, one,
                                       _lib.DAX_BF16, 256, 256, None)
    assert rc == _lib.DAX_ERR_UNSUPPORTED
    assert b"built-in buffer" in lib.dax_last_error()
    with pytest.raises(NotImplementedError):
        _lib.check(rc)
