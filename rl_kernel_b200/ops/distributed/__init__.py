"""Operator objects for the multi-GPU kernels, so that ``kernel_registry`` hands out the sm_100a
implementations of ``cp_attention``, ``vocab_parallel_logp``, ``ratio_kl`` and
``distributed_grpo_loss`` instead of their PyTorch references
(parity: the native entries of the reference's registry, rl_engine/runtime/registry.py:581-788,
1098-1287)."""
from rl_kernel_b200.ops.distributed.cp_attention import CPAttentionOp  # noqa: F401
from rl_kernel_b200.ops.distributed.losses import DistributedGRPOLossNativeOp, RatioKLNativeOp  # noqa: F401
from rl_kernel_b200.ops.distributed.vocab_parallel_logp import VocabParallelLinearLogpOp  # noqa: F401
