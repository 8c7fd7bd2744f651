"""GRPO / PPO loss contract (parity: rl_engine/contracts/operators/loss.py:39-503)."""
from __future__ import annotations

import enum
from dataclasses import dataclass

from rl_kernel_b200.contracts.operators._base import ContractBase, assert_same_across_ranks

GRPO_CONTRACT_ID = "grpo_loss.sequence_major.v1"


class KLEstimator(str, enum.Enum):
    K1 = "k1"
    K3 = "k3"


class LossNormaliser(str, enum.Enum):
    ACTIVE_TOKENS = "active_tokens"
    SEQUENCES = "sequences"


@dataclass(frozen=True)
class GRPOLossContract(ContractBase):
    clip_eps_low: float = 0.2
    clip_eps_high: float = 0.2
    kl_coef: float = 0.001
    kl_estimator: KLEstimator = KLEstimator.K3
    normaliser: LossNormaliser = LossNormaliser.ACTIVE_TOKENS
    samples_per_prompt: int = 8
    advantage_eps: float = 1e-6
    variance: str = "two_pass"
    token_sum: str = "lane_strided_then_xor_butterfly"
    sequence_sum: str = "ascending_sequence"
    dp_gather: str = "rank_ordered_all_gather"
    counts: str = "integer"
    contract_id: str = GRPO_CONTRACT_ID

    def __post_init__(self):
        if self.clip_eps_low < 0 or self.clip_eps_high < 0:
            raise ValueError("clip ranges must be non-negative")
        if self.samples_per_prompt < 2:
            raise ValueError("group-relative advantages need at least 2 samples per prompt")

    def cross_rank_fingerprint(self) -> str:
        return self.fingerprint()

    def preflight(self, group=None) -> None:
        assert_same_across_ranks(self.cross_rank_fingerprint(), group, "GRPO loss contract")
