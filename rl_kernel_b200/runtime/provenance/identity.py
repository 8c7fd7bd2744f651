"""Stable operator identities and code fingerprints (parity: rl_engine/runtime/provenance/
identity.py:14-17 and the fingerprints of semantic_registry.py:467-790)."""
from __future__ import annotations

import hashlib
import inspect
from pathlib import Path


def stable_operator_path(obj) -> str:
    """``module.QualName`` of an operator object or class, with the public alias package name."""
    cls = obj if inspect.isclass(obj) or inspect.isfunction(obj) else type(obj)
    mod = cls.__module__.replace("rl_kernel_b200", "rl_engine", 1)
    return f"{mod}.{cls.__qualname__}"


def code_fingerprint(*objs) -> str:
    """SHA-256 over the source of the given Python objects plus the native library image."""
    h = hashlib.sha256()
    for o in objs:
        try:
            h.update(inspect.getsource(o if inspect.isclass(o) or inspect.isfunction(o) else type(o)).encode())
        except (OSError, TypeError):
            h.update(repr(o).encode())
    return h.hexdigest()


def native_library_fingerprint() -> str | None:
    from rl_kernel_b200.backends.extension import library_path

    p: Path = library_path()
    if not p.exists():
        return None
    h = hashlib.sha256()
    with open(p, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()
