"""The allocation-free GEMM entry point, called through its exported C symbol.

Some embedders of the kernel library may not allocate device memory when they call it (fixed memory
budgets, latency-critical paths where cudaMalloc would stall the device, a device heap owned by a
different allocator).  ``mlcb_gemm_noalloc`` serves them: its split-K scratch is a fixed array inside
the library.  The test checks it against the regular entry point (which gets its scratch from the
caller) and against an fp32 product, on two consecutive calls, because the built-in scratch is shared
by all calls and keeps the previous call's contents.  Every call passes a real status word and the
test asserts that no bounded wait inside the kernel ran out.  The file name sorts last so a run that
stops at the first failure has already executed every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from mlc_llm_b200.ops import _lib as loader

    lib = loader.lib()
    lib.mlcb_gemm_noalloc.restype = ctypes.c_int
    lib.mlcb_gemm_noalloc_last_error.restype = ctypes.c_char_p
    return lib


def _noalloc(lib, x, w, y, ab_fmt, status=None):
    m, k = x.shape
    n = w.shape[0]
    return lib.mlcb_gemm_noalloc(ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(w.data_ptr()),
                                 ctypes.c_void_p(y.data_ptr()), ctypes.c_int(m), ctypes.c_int(n), ctypes.c_int(k),
                                 ctypes.c_int(x.stride(0)), ctypes.c_int(y.stride(0)), ctypes.c_int(ab_fmt),
                                 ctypes.c_void_p(0 if status is None else status.data_ptr()),
                                 ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def _check(y, x, w, status):
    torch.cuda.synchronize()
    assert int(status.item()) == 0, f"a bounded device wait ran out (status {int(status.item())})"
    want = x.float() @ w.float().t()
    err = (y.float() - want).abs()
    tol = 2e-2 + 2e-2 * want.abs()
    assert bool((err <= tol).all()), f"max err vs fp32 product {err.max().item()}"


@pytest.mark.parametrize("dtype,ab_fmt", [(torch.float16, 0), (torch.bfloat16, 1)])
def test_noalloc_matches_regular_entry_point_twice(dtype, ab_fmt):
    from mlc_llm_b200 import ops

    lib = _lib()
    dev = torch.device("cuda")
    torch.manual_seed(0)
    # first a larger problem, then a smaller one with different data: the second call must not be
    # affected by what the first left in the shared scratch
    for m, n, k in [(200, 512, 1024), (48, 256, 2048)]:
        x = (torch.randn(m, k, device=dev) * 0.5).to(dtype)
        w = (torch.randn(n, k, device=dev) * 0.05).to(dtype)
        y = torch.empty(m, n, dtype=dtype, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        rc = _noalloc(lib, x, w, y, ab_fmt, status)
        assert rc == 0, lib.mlcb_gemm_noalloc_last_error().decode()
        _check(y, x, w, status)
        ref = ops.linear(x, ops.dense_weight(w))
        torch.cuda.synchronize()
        err = (y.float() - ref.float()).abs()
        tol = 2e-2 + 2e-2 * ref.float().abs()
        assert bool((err <= tol).all()), f"max err vs the regular entry point {err.max().item()}"


@pytest.mark.parametrize("m,n,k", [(64, 12800, 512),   # 100 tiles: more than half the SMs, runs unsplit
                                   (64, 4096, 2048),   # 32 tiles: split-K through the built-in scratch
                                   (96, 384, 64)])     # a single K block: nothing to split, no scratch
def test_noalloc_many_tiles_and_single_k_block(m, n, k):
    lib = _lib()
    dev = torch.device("cuda")
    torch.manual_seed(1)
    for _ in range(2):
        x = (torch.randn(m, k, device=dev) * 0.5).to(torch.float16)
        w = (torch.randn(n, k, device=dev) * 0.05).to(torch.float16)
        y = torch.empty(m, n, dtype=torch.float16, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        rc = _noalloc(lib, x, w, y, 0, status)
        assert rc == 0, lib.mlcb_gemm_noalloc_last_error().decode()
        _check(y, x, w, status)


def test_noalloc_rejects_oversized_problem():
    lib = _lib()
    dev = torch.device("cuda")
    # 8192 x 8192 outputs are 2048 tiles: more than the built-in counter array holds
    x = torch.zeros(8192, 64, dtype=torch.float16, device=dev)
    w = torch.zeros(8192, 64, dtype=torch.float16, device=dev)
    y = torch.zeros(8192, 8192, dtype=torch.float16, device=dev)
    rc = _noalloc(lib, x, w, y, 0)
    assert rc == -2
    assert b"exceed" in lib.mlcb_gemm_noalloc_last_error()
    # 64 tiles of 256 x 128 split two ways need 16 MiB of partial sums: more than the built-in 8 MiB
    x = torch.zeros(2048, 2048, dtype=torch.float16, device=dev)
    w = torch.zeros(1024, 2048, dtype=torch.float16, device=dev)
    y = torch.zeros(2048, 1024, dtype=torch.float16, device=dev)
    rc = _noalloc(lib, x, w, y, 0)
    assert rc == -2
    assert b"exceed" in lib.mlcb_gemm_noalloc_last_error()
