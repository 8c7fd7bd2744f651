"""Fixed-order collectives and the fused compute+collective operators.

``create_deterministic_collective`` keeps the reference's factory name
(rl_engine/distributed/__init__.py:4-16).
"""
from rl_kernel_b200.distributed.algorithms.collectives import (  # noqa: F401
    CollectiveMismatchError, CollectiveTimeout, TorchDistributedDeterministicCollective, balanced_tree_sum, collective_for_group,
    create_deterministic_collective)
