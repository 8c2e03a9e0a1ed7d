"""A bounded device-side wait that actually runs out.  Every mbarrier / slot wait of the library has a poll
limit after which the kernel raises its abort flag, tears down and stores DAX_ERR_TIMEOUT in the device status
word.  Here a test-only kernel (tests/csrc/expire_wait.cu, compiled with a poll limit of 64) waits on a barrier
nothing arrives on: it must return by itself within milliseconds, the status word must read DAX_ERR_TIMEOUT
once and DAX_OK afterwards, and the context must stay usable.  Nothing here traps, faults or hangs the GPU."""
import ctypes
import os
import subprocess
import time

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _build(libdir):
    from dax_b200.build import CSRC, NVCC_FLAGS, nvcc_path
    src = os.path.join(HERE, "csrc", "expire_wait.cu")
    out = os.path.join(HERE, "csrc", "libdax_test_expire_wait.so")
    deps = [src, os.path.join(CSRC, "sm100_ptx.cuh"), os.path.join(CSRC, "common.cuh")]
    if not os.path.exists(out) or any(os.path.getmtime(d) > os.path.getmtime(out) for d in deps):
        cmd = [nvcc_path()] + [f for f in NVCC_FLAGS if f not in ("-Xptxas", "-v")] + [
            "-DDAX_SPIN_LIMIT=64", "-I", CSRC, "-shared", "-cudart", "static", src, "-o", out,
            "-L", libdir, "-ldax_b200", "-Xlinker", "-rpath", "-Xlinker", libdir]
        r = subprocess.run(cmd, capture_output=True, text=True)
        assert r.returncode == 0, r.stdout + r.stderr
    return out


def test_expired_wait_sets_status_and_returns(built_library):
    if not torch.cuda.is_available():
        pytest.fail("the gpu tests need a CUDA device")
    from dax_b200 import _lib
    _lib.load()  # libdax_b200.so first: the test library resolves the status word through it
    lib = ctypes.CDLL(_build(os.path.dirname(built_library)))
    lib.dax_test_expire_wait.restype = ctypes.c_int
    lib.dax_test_expire_wait.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    assert _lib.device_status() == 0
    polls = torch.zeros(1, dtype=torch.int32, device="cuda")
    t0 = time.perf_counter()
    assert lib.dax_test_expire_wait(polls.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    assert int(polls.item()) == 64, "the kernel was not built with the lowered poll limit"
    assert elapsed < 2.0, f"the bounded wait took {elapsed:.3f} s to give up"
    assert _lib.device_status() == _lib.DAX_ERR_TIMEOUT
    assert _lib.device_status() == 0, "reading the status word must clear it"
    # the context is intact: a production kernel runs and reports no timeout
    from dax_b200 import ops
    q, s = ops.quant_rowwise(torch.randn(8, 64, device="cuda").bfloat16(), torch.int8)
    torch.cuda.synchronize()
    assert q.shape == (8, 64) and _lib.device_status() == 0
