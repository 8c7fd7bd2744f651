"""Small shared utilities: logging, raw-bit comparison, device timing."""
from rl_kernel_b200.utils.bits import bit_equal, bit_mismatch_count, raw_bits  # noqa: F401
from rl_kernel_b200.utils.logger import init_logger  # noqa: F401
