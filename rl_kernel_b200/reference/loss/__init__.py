from rl_kernel_b200.reference.loss.ratio_kl import NativeRatioKLOp  # noqa: F401
from rl_kernel_b200.reference.loss.grpo_loss import NativeGRPOLossOp, grpo_loss_from_logps  # noqa: F401
from rl_kernel_b200.reference.loss.distributed_grpo_loss import DistributedGRPOLossOp  # noqa: F401
