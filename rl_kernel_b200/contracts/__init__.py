"""Numerical contracts: typed, validated descriptions of what an operator promises (reduction
order, sharding, masking, dtype policy), their cross-rank fingerprints and the tolerance profile
used by validation (parity: rl_engine/contracts)."""
from rl_kernel_b200.contracts.numerical import ToleranceSpec, load_precision_profile, resolve_tolerance  # noqa: F401
from rl_kernel_b200.contracts.operators.attention import (AttentionBackendCapability, AttentionContract,  # noqa: F401
                                                          AttentionContractError, KVCacheSpec, ReductionSpec, RoPESpec,
                                                          ShardingSpec, SplitKVSpec)
from rl_kernel_b200.contracts.operators.logprob import (LogprobBackendCapability, LogprobContract,  # noqa: F401
                                                        LogprobContractError, MaskSpec)
from rl_kernel_b200.contracts.operators.loss import GRPOLossContract, LossContractError  # noqa: F401
