"""Numerical contracts: typed, validated descriptions of what an operator promises (reduction
order, sharding, masking, dtype policy), their cross-rank fingerprints and the tolerance profile
used by validation (parity: rl_engine/contracts)."""
from rl_kernel_b200.contracts.numerical import ToleranceSpec, load_precision_profile, resolve_tolerance  # noqa: F401
from rl_kernel_b200.contracts.operators.attention import (AttentionBackendCapability, AttentionContract,  # noqa: F401
                                                          KVCacheSpec, ReductionSpec, RoPESpec, ShardingSpec)
from rl_kernel_b200.contracts.operators.logprob import LogprobBackendCapability, LogprobContract, MaskSpec  # noqa: F401
from rl_kernel_b200.contracts.operators.loss import GRPOLossContract  # noqa: F401
