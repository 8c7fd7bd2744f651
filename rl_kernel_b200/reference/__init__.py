"""PyTorch definitions of every operator: the mathematical contract and the fp32 gold.

They run on CPU, are written for clarity rather than speed, and restate the reduction orders the
sm_100a kernels promise where an order is part of the contract (canonical K-chunk tree, 128-key
attention blocks, 128-id vocab tiles).  Parity: ``rl_engine/reference`` in RL-Kernel.
"""
from rl_kernel_b200.reference.definitions import (  # noqa: F401
    masked_mean, selected_logprobs_reference, summarize_kernel_drift)
