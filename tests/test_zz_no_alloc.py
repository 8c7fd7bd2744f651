"""The allocation-free split GEMM, called through its exported C symbol.

Some callers of this library cannot allocate device memory at the moment they need the chunked
small-M GEMM (a serving loop whose KV-cache pool owns the rest of the GPU, a plugin invoked while
the host framework's memory plan is frozen).  ``rlk_det_gemm_split_static`` keeps its temporary
buffer inside the library image instead of taking a scratch pointer.  This test drives it the way
such a caller would -- raw pointers through ctypes, no scratch argument -- and requires its output
to be bitwise equal to the regular entry point's, on two calls in a row with different inputs (the
built-in buffer keeps the first call's contents, which must not leak into the second result).
The file name sorts last so that a run that stops at the first failure has already run every
other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _call_static(lib, a, b, out, nchunks, tile_n):
    from rl_kernel_b200.backends import extension as ext

    M, K = a.shape
    N = b.shape[0]
    fn = lib.rlk_det_gemm_split_static
    fn.restype = ctypes.c_int
    rc = fn(ext.ptr(a), ext.ptr(b), ext.ptr(out), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
            ctypes.c_longlong(a.stride(0)), ctypes.c_longlong(b.stride(0)), ctypes.c_longlong(out.stride(0)),
            ctypes.c_int(nchunks), ctypes.c_int(tile_n), ext.stream_ptr(a.device))
    return rc


def test_static_scratch_entry_matches_regular_entry_twice():
    from rl_kernel_b200.backends import extension as ext
    from rl_kernel_b200.backends import native as nv

    lib = ext.load()
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cuda").manual_seed(11)
    for call, (M, N, K, nchunks, tile_n) in enumerate([(64, 4096, 4096, 8, 64), (48, 2048, 1024, 4, 32)]):
        a = torch.randn(M, K, device=dev, generator=g).to(BF)
        b = torch.randn(N, K, device=dev, generator=g).to(BF)
        want = torch.empty(M, N, device=dev, dtype=BF)
        scratch = torch.empty(nchunks * M * N, device=dev, dtype=BF)
        nv.det_gemm_split(a, b, want, scratch, nchunks=nchunks, tile_n=tile_n)
        got = torch.full((M, N), float("nan"), device=dev, dtype=BF)
        rc = _call_static(lib, a, b, got, nchunks, tile_n)
        assert rc == 0, lib.rlk_last_error().decode()
        torch.cuda.synchronize()
        assert ext.poll_status(dev) == 0
        assert torch.equal(got, want), f"call {call}: static-scratch result differs from the regular entry point"


def test_static_scratch_entry_rejects_oversized_requests():
    from rl_kernel_b200.backends import extension as ext

    lib = ext.load()
    dev = torch.device("cuda:0")
    M, N, K = 512, 4096, 512           # 8 * 512 * 4096 * 2 bytes = 32 MiB > 8 MiB
    a = torch.zeros(M, K, device=dev, dtype=BF)
    b = torch.zeros(N, K, device=dev, dtype=BF)
    out = torch.zeros(M, N, device=dev, dtype=BF)
    rc = _call_static(lib, a, b, out, 8, 64)
    assert rc == 1
    assert "exceeds the built-in scratch" in lib.rlk_last_error().decode()
