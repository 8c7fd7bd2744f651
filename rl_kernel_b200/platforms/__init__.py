"""Platform layer: one accelerator family (NVIDIA Blackwell, sm_100a) plus CPU for references."""
from rl_kernel_b200.platforms.constants import DeviceType, PlatformName  # noqa: F401
from rl_kernel_b200.platforms.device import DeviceContext, device_ctx  # noqa: F401
