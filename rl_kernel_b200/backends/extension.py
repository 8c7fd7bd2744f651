"""Loader for the native library ``librlk_b200.so`` (plain C ABI, loaded with ctypes).

Plays the role of the reference's soft import of ``rl_engine._C``
(rl_engine/backends/extension.py:12-19) with one difference: on a machine that has a CUDA
device the library is REQUIRED — a missing or stale library raises instead of silently
falling back to PyTorch, so a GPU run can never pass on an eager fallback.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

import torch

_LIB_PATH = Path(__file__).resolve().parent.parent / "librlk_b200.so"
_lock = threading.Lock()
_lib: ctypes.CDLL | None = None
_load_error: str | None = None

ABI_VERSION = 1


class NativeLibraryError(RuntimeError):
    """The sm_100a library is missing, stale, or a native call reported an error."""


class DeviceWaitTimeout(NativeLibraryError):
    """A bounded device-side wait gave up; the context is still usable."""


def library_path() -> Path:
    return _LIB_PATH


def _try_build() -> None:
    if os.environ.get("RLK_NO_AUTOBUILD") == "1":
        return
    from rl_kernel_b200.csrc.build import build

    build()


def load(required: bool = True) -> ctypes.CDLL | None:
    """Return the loaded library, building it in-tree first if it does not exist."""
    global _lib, _load_error
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        try:
            if not _LIB_PATH.exists():
                _try_build()
            lib = ctypes.CDLL(str(_LIB_PATH))
            lib.rlk_last_error.restype = ctypes.c_char_p
            lib.rlk_abi_version.restype = ctypes.c_int
            if lib.rlk_abi_version() != ABI_VERSION:
                raise NativeLibraryError(
                    f"{_LIB_PATH} has ABI {lib.rlk_abi_version()}, expected {ABI_VERSION}; rebuild "
                    "with `python -m rl_kernel_b200.csrc.build --force`"
                )
            if os.environ.get("RLK_PDL", "1") == "0":
                lib.rlk_set_pdl(ctypes.c_int(0))     # programmatic dependent launch off
            _lib = lib
        except Exception as exc:  # noqa: BLE001 - reported below
            _load_error = f"{type(exc).__name__}: {exc}"
            if required:
                raise NativeLibraryError(
                    f"cannot load {_LIB_PATH}: {_load_error}. Build it with "
                    "`python -m rl_kernel_b200.csrc.build`."
                ) from exc
            return None
    return _lib


def available() -> bool:
    """True when the native library is loadable AND a CUDA device is present."""
    return torch.cuda.is_available() and load(required=False) is not None


def check(rc: int, what: str = "native call") -> None:
    if rc == 0:
        return
    lib = load()
    msg = lib.rlk_last_error().decode("utf-8", "replace")
    if rc == 4:
        raise DeviceWaitTimeout(f"{what}: {msg}")
    raise NativeLibraryError(f"{what} failed (code {rc}): {msg}")


def stream_ptr(device: torch.device | None = None) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def poll_status(device: torch.device | None = None) -> int:
    """Synchronise the current stream and return (and clear) the device status word.

    Non-zero means a bounded wait inside a kernel timed out; the value identifies the wait.
    """
    lib = load()
    code = ctypes.c_int(0)
    check(lib.rlk_status_poll(stream_ptr(device), ctypes.byref(code)), "status poll")
    return code.value


def raise_on_device_timeout(device: torch.device | None = None) -> None:
    code = poll_status(device)
    if code != 0:
        raise DeviceWaitTimeout(f"a device-side wait timed out (wait id {code})")
