"""Enums of the platform layer (parity: rl_engine/platforms/constants.py:7-110, reduced to the
single backend this library targets)."""
from __future__ import annotations

import enum


class DeviceType(str, enum.Enum):
    CUDA = "cuda"
    CPU = "cpu"


class PlatformName(str, enum.Enum):
    B200 = "b200"        # sm_100a with the native library loaded
    CUDA_OTHER = "cuda"  # some other CUDA GPU: only the PyTorch references run
    CPU = "cpu"


SM100 = (10, 0)
HBM_BYTES_B200 = 180 * 1000 ** 3
L2_BYTES_B200 = 126 * 1024 * 1024
SM_COUNT_B200 = 148
