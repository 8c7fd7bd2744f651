from rl_kernel_b200.models.qwen3_moe.engine import MoEPackedParams, Qwen3MoeEngine  # noqa: F401
from rl_kernel_b200.models.qwen3_moe.spec import Qwen3MoeSpec  # noqa: F401
