"""Device facts the validation gates need (parity: rl_engine/validation/operators/accelerator.py:43-290), for the two
device types this framework runs on: ``cuda`` (B200, sm_100a kernels) and ``cpu`` (reference operators).

Rules enforced here: a required profile never falls back silently (asking for the B200 profile on a host without a GPU
is an error, not a CPU run); TF32 is off whenever a gate runs; ``arch_key`` pins the silicon in every piece of evidence."""
from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Any

import torch

PROFILE_DEVICE = {"b200_bf16": "cuda", "cuda_bf16": "cuda", "cpu_fp32": "cpu", "reference_fp32": "cpu"}
CANDIDATE_FAMILY = {"b200": "cuda", "cuda": "cuda", "sm100": "cuda", "pytorch": "any", "reference": "any", "native": "any"}


class AcceleratorUnavailable(RuntimeError):
    pass


def is_available(device_type: str) -> bool:
    if device_type == "cpu":
        return True
    if device_type == "cuda":
        return torch.cuda.is_available()
    return False


def device_type_for_profile(profile: str) -> str:
    try:
        return PROFILE_DEVICE[profile]
    except KeyError:
        raise ValueError(f"unknown backend profile {profile!r}; known: {sorted(PROFILE_DEVICE)}") from None


def family_for_profile(profile: str) -> str:
    return device_type_for_profile(profile)


def candidate_family(candidate: str) -> str:
    try:
        return CANDIDATE_FAMILY[candidate.strip().lower()]
    except KeyError:
        raise ValueError(f"unknown candidate {candidate!r}") from None


@dataclass(frozen=True)
class AcceleratorInfo:
    device_type: str
    device_index: int | None
    name: str
    arch_key: str
    compute_capability: str
    runtime_version: str | None
    tf32_enabled: bool
    total_memory_bytes: int | None

    def to_dict(self) -> dict[str, Any]:
        return asdict(self)


def resolve_device(device: str | torch.device | None = None, *, profile: str | None = None, required: bool = True) -> torch.device:
    """The device of a gate.  With ``profile`` the device type is the profile's; ``required`` (default) makes an
    unavailable device an ``AcceleratorUnavailable`` instead of a quiet CPU run."""
    want = device_type_for_profile(profile) if profile else None
    dev = torch.device(device) if device is not None else torch.device(want or ("cuda" if torch.cuda.is_available() else "cpu"))
    if want and dev.type != want:
        raise AcceleratorUnavailable(f"profile {profile!r} runs on {want}, not on {dev.type}")
    if not is_available(dev.type):
        if required:
            raise AcceleratorUnavailable(f"device type {dev.type!r} is not available on this host")
        return torch.device("cpu")
    if dev.type == "cuda" and dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    return dev


def current_device(device_type: str) -> int:
    return torch.cuda.current_device() if device_type == "cuda" else 0


def set_device(device: torch.device) -> None:
    if device.type == "cuda":
        torch.cuda.set_device(device)


def device_name(device: torch.device) -> str:
    return torch.cuda.get_device_name(device) if device.type == "cuda" else "cpu"


def compute_capability(device: torch.device) -> str:
    if device.type != "cuda":
        return "cpu"
    major, minor = torch.cuda.get_device_capability(device)
    return f"{major}.{minor}"


def arch_key(device: torch.device) -> str:
    """``sm100`` on a B200; ``cpu`` otherwise."""
    return "sm" + compute_capability(device).replace(".", "") if device.type == "cuda" else "cpu"


def runtime_version(device_type: str) -> str | None:
    return torch.version.cuda if device_type == "cuda" else None


def tf32_enabled() -> bool:
    return bool(torch.backends.cuda.matmul.allow_tf32 or torch.backends.cudnn.allow_tf32)


def disable_tf32(device_type: str) -> bool:
    """Switch TF32 off for library matmuls and convolutions; returns the state after the call (always False)."""
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    return tf32_enabled()


def describe(device: torch.device) -> AcceleratorInfo:
    mem = torch.cuda.get_device_properties(device).total_memory if device.type == "cuda" else None
    return AcceleratorInfo(device.type, device.index, device_name(device), arch_key(device), compute_capability(device),
                           runtime_version(device.type), tf32_enabled(), mem)


def manual_seed_all(device_type: str, seed: int) -> None:
    torch.manual_seed(seed)
    if device_type == "cuda" and torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def synchronize(device: torch.device) -> None:
    if device.type == "cuda":
        torch.cuda.synchronize(device)


def empty_cache(device_type: str) -> None:
    if device_type == "cuda" and torch.cuda.is_available():
        torch.cuda.empty_cache()


__all__ = ["AcceleratorInfo", "AcceleratorUnavailable", "arch_key", "candidate_family", "compute_capability", "current_device", "describe",
           "device_name", "device_type_for_profile", "disable_tf32", "empty_cache", "family_for_profile", "is_available", "manual_seed_all",
           "resolve_device", "runtime_version", "set_device", "synchronize", "tf32_enabled"]
