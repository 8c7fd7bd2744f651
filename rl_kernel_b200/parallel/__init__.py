"""Parallelism entry points (tensor / context / vocab / data parallel). ``rl_kernel_b200.parallel``
and ``rl_kernel_b200.distributed`` expose the same collectives; model-level parallel layouts live
in ``rl_kernel_b200.models.qwen3.engine.ParallelContext``."""
from rl_kernel_b200.distributed import *  # noqa: F401,F403
from rl_kernel_b200.distributed import (collective_for_group, create_deterministic_collective)  # noqa: F401
