"""Device context singleton (parity: DeviceContext, rl_engine/platforms/device.py:35-101)."""
from __future__ import annotations

import functools

import torch

from rl_kernel_b200.platforms.constants import SM100, DeviceType, PlatformName


class DeviceContext:
    def __init__(self) -> None:
        self._refresh()

    def _refresh(self) -> None:
        self.has_cuda = torch.cuda.is_available()
        self.capability = torch.cuda.get_device_capability() if self.has_cuda else None
        self.device_count = torch.cuda.device_count() if self.has_cuda else 0

    @property
    def device_type(self) -> DeviceType:
        return DeviceType.CUDA if self.has_cuda else DeviceType.CPU

    @property
    def is_sm100(self) -> bool:
        return self.capability is not None and tuple(self.capability) == SM100

    @functools.cached_property
    def native_available(self) -> bool:
        from rl_kernel_b200.backends import extension

        return self.is_sm100 and extension.available()

    @property
    def platform(self) -> PlatformName:
        if self.native_available:
            return PlatformName.B200
        return PlatformName.CUDA_OTHER if self.has_cuda else PlatformName.CPU

    def current_device(self) -> torch.device:
        return torch.device("cuda", torch.cuda.current_device()) if self.has_cuda else torch.device("cpu")

    def describe(self) -> dict:
        d = {"platform": self.platform.value, "device_type": self.device_type.value,
             "device_count": self.device_count, "capability": self.capability}
        if self.has_cuda:
            p = torch.cuda.get_device_properties(0)
            d.update(name=p.name, total_memory=p.total_memory, sm_count=p.multi_processor_count)
        return d


device_ctx = DeviceContext()
