"""Selected-token log-prob contract (parity: rl_engine/contracts/operators/logprob.py:54-494)."""
from __future__ import annotations

import enum
from dataclasses import dataclass, field

from rl_kernel_b200.contracts.operators._base import ContractBase, assert_same_across_ranks

LOGPROB_CONTRACT_ID = "logprob.vocab_tile128.v1"


class LogpInput(str, enum.Enum):
    LOGITS = "logits"
    HIDDEN = "hidden"           # fused linear -> logp


class TopPReplay(str, enum.Enum):
    NONE = "none"
    KEEP_THRESHOLD = "keep_threshold"


@dataclass(frozen=True)
class VocabShardingSpec(ContractBase):
    tp_size: int = 1
    real_vocab: int = 151936
    padded_vocab: int = 152576
    tile: int = 128

    def __post_init__(self):
        if self.tp_size not in (1, 2, 4, 8):
            raise ValueError("tp_size must be 1, 2, 4 or 8")
        if self.padded_vocab % (self.tile * self.tp_size):
            raise ValueError("padded vocab must be a multiple of tile * tp_size so tiles never straddle a shard")
        if not 0 < self.real_vocab <= self.padded_vocab:
            raise ValueError("real_vocab must be in (0, padded_vocab]")

    @property
    def num_tiles(self) -> int:
        return self.padded_vocab // self.tile


@dataclass(frozen=True)
class MaskSpec(ContractBase):
    mask_before_normalisation: bool = True
    masked_value: float = 0.0
    clamp_non_positive: bool = True


@dataclass(frozen=True)
class LogprobContract(ContractBase):
    input_kind: LogpInput = LogpInput.HIDDEN
    logits_dtype: str = "bfloat16"
    output_dtype: str = "float32"
    temperature: float = 1.0
    temperature_scales: str = "logits_before_max"
    tile_sum: str = "four_interleaved_chains"
    row_merge: str = "ascending_tile_fma"
    exp: str = "__expf"
    sharding: VocabShardingSpec = field(default_factory=VocabShardingSpec)
    mask: MaskSpec = field(default_factory=MaskSpec)
    top_p_replay: TopPReplay = TopPReplay.NONE
    contract_id: str = LOGPROB_CONTRACT_ID

    def __post_init__(self):
        if self.temperature <= 0:
            raise ValueError("temperature must be positive")

    def cross_rank_fingerprint(self) -> str:
        return self.fingerprint()

    def preflight(self, group=None) -> None:
        assert_same_across_ranks(self.cross_rank_fingerprint(), group, "logprob contract")


@dataclass(frozen=True)
class LogprobBackendCapability(ContractBase):
    backend_id: str
    fused_linear: bool = True
    batch_invariant: bool = True
    vocab_parallel: bool = True
    backward: bool = True

    def incompatibilities(self, contract: LogprobContract) -> list[str]:
        why = []
        if contract.input_kind == LogpInput.HIDDEN and not self.fused_linear:
            why.append("backend cannot fuse the LM head")
        if contract.sharding.tp_size > 1 and not self.vocab_parallel:
            why.append("backend is not vocab-parallel")
        if not self.batch_invariant:
            why.append("backend is not batch-invariant")
        return why


B200_LOGPROB_CAPABILITY = LogprobBackendCapability(backend_id="b200-tcgen05")
REFERENCE_LOGPROB_CAPABILITY = LogprobBackendCapability(backend_id="reference")
