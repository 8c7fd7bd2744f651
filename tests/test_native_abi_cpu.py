"""Argument checks of the native library that run before any CUDA call, exercised on a machine
without a GPU: a rejected request must return RLK_ERR_BAD_ARG (1) and launch nothing."""
import ctypes

from rl_kernel_b200.backends import extension as ext


def _static(lib, a, b, c, M, N, K, ldc, nchunks):
    fn = lib.rlk_det_gemm_split_static
    fn.restype = ctypes.c_int
    return fn(ctypes.c_void_p(a), ctypes.c_void_p(b), ctypes.c_void_p(c), ctypes.c_int(M), ctypes.c_int(N),
              ctypes.c_int(K), ctypes.c_longlong(K), ctypes.c_longlong(K), ctypes.c_longlong(ldc),
              ctypes.c_int(nchunks), ctypes.c_int(64), ctypes.c_void_p(0))


def test_static_split_gemm_rejects_bad_requests_before_touching_the_device():
    lib = ext.load()
    lib.rlk_last_error.restype = ctypes.c_char_p
    fake = 0x10000            # never dereferenced: every case below is refused first
    assert _static(lib, fake, fake, 0, 16, 256, 512, 256, 4) == 1
    assert b"must not be null" in lib.rlk_last_error()
    assert _static(lib, 0, fake, fake, 16, 256, 512, 256, 4) == 1
    assert _static(lib, fake, fake, fake, 16, 256, 512, 248, 4) == 1
    assert b"must be at least N" in lib.rlk_last_error()
    assert _static(lib, fake, fake, fake, 512, 4096, 512, 4096, 8) == 1
    assert b"exceeds the built-in scratch" in lib.rlk_last_error()
    assert _static(lib, fake, fake, fake, 16, 256, 512, 256, 3) == 1


def test_split_gemm_with_scratch_rejects_a_pitch_below_n():
    lib = ext.load()
    lib.rlk_last_error.restype = ctypes.c_char_p
    fn = lib.rlk_det_gemm_split
    fn.restype = ctypes.c_int
    fake = ctypes.c_void_p(0x10000)
    rc = fn(fake, fake, fake, fake, ctypes.c_int(16), ctypes.c_int(256), ctypes.c_int(512), ctypes.c_longlong(512),
            ctypes.c_longlong(512), ctypes.c_longlong(128), ctypes.c_int(4), ctypes.c_int(64), ctypes.c_void_p(0))
    assert rc == 1 and b"must be at least N" in lib.rlk_last_error()
