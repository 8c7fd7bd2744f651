"""Deterministic collectives by transport (parity: rl_engine/distributed/transports/collectives.py:1-20): the
``torch.distributed`` implementation (gather + fixed balanced tree; any backend) and the peer-memory implementation over
NVLink symmetric memory (``SymmetricMemoryCollective``; CUDA only), behind one factory."""
from rl_kernel_b200.distributed.algorithms.collectives import (TorchDistributedDeterministicCollective,  # noqa: F401
                                                               create_deterministic_collective)
from rl_kernel_b200.distributed.transports.symm import SymmetricMemoryCollective  # noqa: F401

NVLinkDeterministicCollective = SymmetricMemoryCollective
RCCLDeterministicCollective = TorchDistributedDeterministicCollective      # name kept for callers written against ROCm builds

__all__ = ["NVLinkDeterministicCollective", "RCCLDeterministicCollective", "SymmetricMemoryCollective",
           "TorchDistributedDeterministicCollective", "create_deterministic_collective"]
