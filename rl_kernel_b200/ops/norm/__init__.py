from rl_kernel_b200.ops.norm.canonical_rmsnorm import RMSNormOp, rms_norm  # noqa: F401
from rl_kernel_b200.ops.norm import reproducible  # noqa: F401
