"""The allocation-free split GEMM, called through its exported C symbol.

Some callers of this library cannot allocate device memory at the moment they need the chunked
small-M GEMM (a serving loop whose KV-cache pool owns the rest of the GPU, a plugin invoked while
the host framework's memory plan is frozen).  ``rlk_det_gemm_split_static`` keeps its temporary
buffer inside the library image instead of taking a scratch pointer.  This test drives it the way
such a caller would -- raw pointers through ctypes, no scratch argument -- and requires its output
to be bitwise equal to the regular entry point's, on consecutive calls with different inputs and
sizes (the built-in buffer keeps the previous call's contents, which must not leak into the next
result), with the free device memory unchanged across a call.
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


def test_static_scratch_entry_matches_regular_entry_on_consecutive_calls():
    """Four calls in a row through the exported symbol: a large one, a smaller one (stale partials of
    the first call sit behind its own), a larger one again, and one whose output pitch is wider than
    N.  Every result must equal the regular entry point's bit for bit, and from the second call on
    the amount of free device memory must not move: the point of the entry is that it allocates
    nothing.  (The static entry has no status word, so a device-side wait that gave up could not be
    polled here; the bitwise comparison is what catches a kernel that ended early.)"""
    from rl_kernel_b200.backends import extension as ext
    from rl_kernel_b200.backends import native as nv

    lib = ext.load()
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cuda").manual_seed(11)
    cases = [(64, 4096, 4096, 8, 64, 0), (48, 2048, 1024, 4, 32, 0), (96, 4096, 2048, 8, 64, 0),
             (40, 1024, 2048, 2, 64, 256)]
    for call, (M, N, K, nchunks, tile_n, pad) in enumerate(cases):
        a = torch.randn(M, K, device=dev, generator=g).to(BF)
        b = torch.randn(N, K, device=dev, generator=g).to(BF)
        ldc = N + pad
        want = torch.zeros(M, ldc, device=dev, dtype=BF)[:, :N]
        scratch = torch.empty(nchunks * M * ldc, device=dev, dtype=BF)
        nv.det_gemm_split(a, b, want, scratch, nchunks=nchunks, tile_n=tile_n)
        got = torch.full((M, ldc), float("nan"), device=dev, dtype=BF)[:, :N]
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info(dev)[0]
        rc = _call_static(lib, a, b, got, nchunks, tile_n)
        assert rc == 0, lib.rlk_last_error().decode()
        torch.cuda.synchronize()
        free_after = torch.cuda.mem_get_info(dev)[0]
        if call > 0:        # the first call of a process may load the kernel's module
            assert free_after == free_before, f"call {call}: free device memory moved by {free_before - free_after} bytes"
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


def test_static_scratch_entry_rejects_null_output_and_narrow_pitch():
    """No leaves-only mode and no pitch below N: both are refused before anything is launched."""
    from rl_kernel_b200.backends import extension as ext

    lib = ext.load()
    dev = torch.device("cuda:0")
    M, N, K = 16, 256, 512
    a = torch.zeros(M, K, device=dev, dtype=BF)
    b = torch.zeros(N, K, device=dev, dtype=BF)
    out = torch.zeros(M, N, device=dev, dtype=BF)
    fn = lib.rlk_det_gemm_split_static
    fn.restype = ctypes.c_int
    common = (ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K), ctypes.c_longlong(K), ctypes.c_longlong(K))
    rc = fn(ext.ptr(a), ext.ptr(b), ctypes.c_void_p(0), *common, ctypes.c_longlong(N), ctypes.c_int(4),
            ctypes.c_int(64), ext.stream_ptr(dev))
    assert rc == 1 and "must not be null" in lib.rlk_last_error().decode()
    rc = fn(ext.ptr(a), ext.ptr(b), ext.ptr(out), *common, ctypes.c_longlong(N - 8), ctypes.c_int(4),
            ctypes.c_int(64), ext.stream_ptr(dev))
    assert rc == 1 and "must be at least N" in lib.rlk_last_error().decode()
    torch.cuda.synchronize()
