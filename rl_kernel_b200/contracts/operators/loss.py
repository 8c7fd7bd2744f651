"""GRPO loss contract (parity: rl_engine/contracts/operators/loss.py:35-784).

A ``GRPOLossContract`` nests the log-prob contract of the calling rank's rows and adds: which
sequences of the global batch the data-parallel rank owns and how they fall into advantage groups
(``LossShardingSpec``); the objective (``ObjectiveSpec``: asymmetric ratio clipping, reference-KL
estimator and weight, group-relative advantage normalisation with the two-pass variance); how
per-token terms become one scalar (``LossReductionSpec``: fp32, tokens of a sequence on the rank
that owns it, sequences in ascending global index, partial sums moved by all-gather and never
reduced by a collective, one of three denominators); and the fp32 replicated output.

``KernelSummation`` additionally pins the in-kernel order of the sm_100a loss kernel
(lane-strided token sums folded by an xor butterfly, integer counts), which the PyTorch reference
reproduces.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from enum import Enum
from typing import Any

from rl_kernel_b200.contracts.operators._base import ContractBase, assert_same_across_ranks, is_plain_int, make_validators, stable_hash
from rl_kernel_b200.contracts.operators.logprob import (RESERVED_DISPATCH_POLICIES, DeterminismScope, DowncastPoint,
                                                         LogprobContract, LogprobDType)

GRPO_CONTRACT_ID = "grpo_loss.sequence_major.v1"


class LossContractError(ValueError):
    """Loss metadata does not describe a valid GRPO invocation."""


(_enum_value, _positive_int, _non_negative_int, _plain_int, _integer_tuple, _coerce,
 _world_sizes) = make_validators(LossContractError)


def _non_negative_float(value: Any, name: str) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise LossContractError(f"{name} must be a real number; got {value!r}")
    value = float(value)
    if not math.isfinite(value) or value < 0.0:
        raise LossContractError(f"{name} must be finite and non-negative; got {value!r}")
    return value


class TokenNormalizer(str, Enum):
    """Denominator of the summed per-token terms: the active tokens of the global batch (long sequences
    weigh more), each sequence's own active count followed by a mean over sequences (equal weights), or a
    declared constant.  They differ by more than a scale once lengths vary, so the choice is part of the
    numerical identity."""
    GLOBAL_ACTIVE_TOKENS = "global_active_tokens"
    PER_SEQUENCE_THEN_MEAN = "per_sequence_then_mean"
    FIXED_CONSTANT = "fixed_constant"


class SummationOrder(str, Enum):
    """Tokens of a sequence combine over the full padded length on the one rank that owns the sequence;
    sequences combine in ascending global index.  Both extents are contract-fixed, so the grouping is the
    same at every DP degree -- only which rank computes a sequence changes."""
    SEQUENCE_MAJOR_FIXED = "sequence_major_fixed"


class LossTransport(str, Enum):
    """Collectives move partial sums, they never add them (an all-reduce's order depends on world size
    and topology)."""
    ALL_GATHER = "all_gather"


class KLEstimator(str, Enum):
    K3_UNBIASED = "k3_unbiased"        # exp(ref - pol) - (ref - pol) - 1
    K1_LOG_RATIO = "k1_log_ratio"      # pol - ref


class ClipMode(str, Enum):
    MIN_OF_UNCLIPPED_AND_CLIPPED = "min_of_unclipped_and_clipped"


class AdvantageNormalizer(str, Enum):
    MEAN_STD_POPULATION = "mean_std_population"     # (r - mean) / std, biased std: the original GRPO form
    MEAN_ONLY = "mean_only"                         # r - mean (Dr.GRPO)


class VarianceFormula(str, Enum):
    TWO_PASS = "two_pass"              # subtract the mean before squaring; E[x^2] - E[x]^2 cancels catastrophically


class GroupReplication(str, Enum):
    REPLICATED_ALL_GATHER = "replicated_all_gather"     # rewards are gathered and every rank normalises every group


class LossPlacement(str, Enum):
    REPLICATED = "replicated"


@dataclass(frozen=True)
class ClipSpec:
    """Asymmetric PPO ratio clipping; equal epsilons give the symmetric [1 - eps, 1 + eps]."""
    clip_eps_low: float = 0.2
    clip_eps_high: float = 0.2
    mode: ClipMode = ClipMode.MIN_OF_UNCLIPPED_AND_CLIPPED

    def __post_init__(self) -> None:
        object.__setattr__(self, "mode", _enum_value(ClipMode, self.mode, "clip.mode"))
        low = _non_negative_float(self.clip_eps_low, "clip_eps_low")
        high = _non_negative_float(self.clip_eps_high, "clip_eps_high")
        if low >= 1.0:
            raise LossContractError(f"clip_eps_low={low} must be smaller than 1.0; the lower clip bound 1 - clip_eps_low "
                                    "must stay positive")
        object.__setattr__(self, "clip_eps_low", low)
        object.__setattr__(self, "clip_eps_high", high)

    @property
    def lower_bound(self) -> float:
        return 1.0 - self.clip_eps_low

    @property
    def upper_bound(self) -> float:
        return 1.0 + self.clip_eps_high


@dataclass(frozen=True)
class AdvantageSpec:
    normalizer: AdvantageNormalizer = AdvantageNormalizer.MEAN_STD_POPULATION
    variance: VarianceFormula = VarianceFormula.TWO_PASS
    std_eps: float = 1e-6
    replication: GroupReplication = GroupReplication.REPLICATED_ALL_GATHER

    def __post_init__(self) -> None:
        object.__setattr__(self, "normalizer", _enum_value(AdvantageNormalizer, self.normalizer, "advantage.normalizer"))
        object.__setattr__(self, "variance", _enum_value(VarianceFormula, self.variance, "advantage.variance"))
        object.__setattr__(self, "replication", _enum_value(GroupReplication, self.replication, "advantage.replication"))
        eps = _non_negative_float(self.std_eps, "advantage.std_eps")
        if eps <= 0.0:
            raise LossContractError(f"advantage.std_eps={eps} must be strictly positive; it is the floor that keeps a "
                                    "zero-variance group from dividing by zero")
        object.__setattr__(self, "std_eps", eps)


@dataclass(frozen=True)
class ObjectiveSpec:
    clip: ClipSpec = field(default_factory=ClipSpec)
    advantage: AdvantageSpec = field(default_factory=AdvantageSpec)
    kl_estimator: KLEstimator = KLEstimator.K3_UNBIASED
    beta: float = 0.0

    def __post_init__(self) -> None:
        if not isinstance(self.clip, ClipSpec):
            raise LossContractError("objective.clip must be a ClipSpec")
        if not isinstance(self.advantage, AdvantageSpec):
            raise LossContractError("objective.advantage must be an AdvantageSpec")
        object.__setattr__(self, "kl_estimator", _enum_value(KLEstimator, self.kl_estimator, "objective.kl_estimator"))
        object.__setattr__(self, "beta", _non_negative_float(self.beta, "objective.beta"))

    @property
    def uses_reference_model(self) -> bool:
        """beta == 0 drops the KL term from the loss (the KL is still reported when reference log-probs exist)."""
        return self.beta > 0.0


@dataclass(frozen=True)
class LossReductionSpec:
    token_normalizer: TokenNormalizer = TokenNormalizer.GLOBAL_ACTIVE_TOKENS
    summation_order: SummationOrder = SummationOrder.SEQUENCE_MAJOR_FIXED
    acc_dtype: LogprobDType = LogprobDType.FP32
    transport: LossTransport = LossTransport.ALL_GATHER
    downcast_at: DowncastPoint = DowncastPoint.FINAL_WRITE
    determinism_scope: DeterminismScope = DeterminismScope.CROSS_TP_BITWISE
    fixed_normalizer_constant: int | None = None

    def __post_init__(self) -> None:
        _coerce(self, token_normalizer=TokenNormalizer, summation_order=SummationOrder, acc_dtype=LogprobDType,
                transport=LossTransport, downcast_at=DowncastPoint, determinism_scope=DeterminismScope)
        if self.acc_dtype is not LogprobDType.FP32:
            raise LossContractError(f"loss accumulation must be fp32; got {self.acc_dtype.value}")
        if self.token_normalizer is TokenNormalizer.FIXED_CONSTANT:
            object.__setattr__(self, "fixed_normalizer_constant",
                               _positive_int(self.fixed_normalizer_constant, "fixed_normalizer_constant"))
        elif self.fixed_normalizer_constant is not None:
            raise LossContractError("fixed_normalizer_constant is only meaningful for "
                                    f"token_normalizer={TokenNormalizer.FIXED_CONSTANT.value}; got {self.token_normalizer.value}")


@dataclass(frozen=True)
class LossOutputSpec:
    loss_dtype: LogprobDType = LogprobDType.FP32
    placement: LossPlacement = LossPlacement.REPLICATED

    def __post_init__(self) -> None:
        _coerce(self, loss_dtype=LogprobDType, placement=LossPlacement)
        if self.loss_dtype is not LogprobDType.FP32:
            raise LossContractError(f"loss output must be fp32; got {self.loss_dtype.value}")


@dataclass(frozen=True)
class KernelSummation(ContractBase):
    """In-kernel order of the device loss kernel (rl_kernel_b200/csrc/loss/grpo_loss.cu)."""
    token_sum: str = "lane_strided_then_xor_butterfly"
    sequence_sum: str = "ascending_sequence"
    dp_gather: str = "rank_ordered_all_gather"
    counts: str = "integer"
    contract_id: str = GRPO_CONTRACT_ID


@dataclass(frozen=True)
class LossShardingSpec:
    """Which sequences of the global batch (``num_sequences`` x ``padded_seq_len`` token slots) this DP rank
    owns.  ``sequence_shard_bounds[r]`` is rank r's half-open range; the table partitions
    [0, num_sequences) contiguously in rank order.  ``group_boundaries`` are the num_groups + 1 offsets of the
    advantage groups."""
    dp_rank: int
    dp_world_size: int
    num_sequences: int
    padded_seq_len: int
    sequence_shard_bounds: tuple[tuple[int, int], ...]
    group_boundaries: tuple[int, ...]
    cp_rank: int = 0
    cp_world_size: int = 1

    def __post_init__(self) -> None:
        dp = _positive_int(self.dp_world_size, "dp_world_size")
        if _non_negative_int(self.dp_rank, "dp_rank") >= dp:
            raise LossContractError(f"dp_rank={self.dp_rank} must be smaller than dp_world_size={dp}")
        cp = _positive_int(self.cp_world_size, "cp_world_size")
        _non_negative_int(self.cp_rank, "cp_rank")
        if cp != 1:
            raise LossContractError(f"cp_world_size={cp} is unsupported: context parallelism splits a sequence's tokens "
                                    "across ranks, so the loss reduction would span an axis this contract does not model. "
                                    "Reduce across CP outside this operator.")
        if self.cp_rank != 0:
            raise LossContractError(f"cp_rank must be 0 when cp_world_size=1; got {self.cp_rank}")
        n = _positive_int(self.num_sequences, "num_sequences")
        _positive_int(self.padded_seq_len, "padded_seq_len")
        object.__setattr__(self, "sequence_shard_bounds", self._validated_bounds(self.sequence_shard_bounds, dp, n))
        object.__setattr__(self, "group_boundaries", self._validated_groups(self.group_boundaries, n))

    @staticmethod
    def _validated_bounds(raw: Any, dp: int, n: int) -> tuple[tuple[int, int], ...]:
        try:
            bounds = tuple((p[0], p[1]) for p in raw)
        except (TypeError, IndexError, KeyError) as exc:
            raise LossContractError("sequence_shard_bounds must be an iterable of (start, end) integer pairs") from exc
        if len(bounds) != dp:
            raise LossContractError("sequence_shard_bounds must declare exactly one (start, end) pair per DP rank; "
                                    f"got {len(bounds)} pairs for dp_world_size={dp}")
        expect = 0
        for r, (s, e) in enumerate(bounds):
            for name, v in ((f"sequence_shard_bounds[{r}][0]", s), (f"sequence_shard_bounds[{r}][1]", e)):
                if not is_plain_int(v):
                    raise LossContractError(f"{name} must be an integer; got {v!r}")
            if e <= s:
                raise LossContractError(f"sequence_shard_bounds[{r}] must satisfy end > start; got [{s}, {e})")
            if s != expect:
                raise LossContractError("sequence_shard_bounds must form a contiguous [0, num_sequences) partition in "
                                        f"DP-rank order; rank {r} starts at {s}, expected {expect}")
            expect = e
        if expect != n:
            raise LossContractError(f"sequence_shard_bounds must cover num_sequences exactly; covered {expect}, declared {n}")
        return bounds

    @staticmethod
    def _validated_groups(raw: Any, n: int) -> tuple[int, ...]:
        try:
            offs = tuple(raw)
        except TypeError as exc:
            raise LossContractError("group_boundaries must be an iterable of integers") from exc
        if len(offs) < 2:
            raise LossContractError("group_boundaries must hold num_groups + 1 offsets, so at least 2 entries")
        for i, v in enumerate(offs):
            if not is_plain_int(v):
                raise LossContractError(f"group_boundaries[{i}] must be an integer")
        if offs[0] != 0 or offs[-1] != n:
            raise LossContractError(f"group_boundaries must start at 0 and end at num_sequences={n}; "
                                    f"got [{offs[0]}, ..., {offs[-1]}]")
        for i in range(1, len(offs)):
            if offs[i] <= offs[i - 1]:
                raise LossContractError(f"group_boundaries must be strictly increasing; offset {i} is {offs[i]} after "
                                        f"{offs[i - 1]}")
        return offs

    @classmethod
    def even(cls, *, dp_rank: int, dp_world_size: int, num_sequences: int, padded_seq_len: int,
             samples_per_prompt: int) -> "LossShardingSpec":
        """Equal sequence shards and equal groups of ``samples_per_prompt`` consecutive sequences."""
        if num_sequences % dp_world_size or num_sequences % samples_per_prompt:
            raise LossContractError("num_sequences must divide evenly into DP ranks and into groups")
        per = num_sequences // dp_world_size
        return cls(dp_rank, dp_world_size, num_sequences, padded_seq_len,
                   tuple((r * per, (r + 1) * per) for r in range(dp_world_size)),
                   tuple(range(0, num_sequences + 1, samples_per_prompt)))

    @property
    def num_groups(self) -> int:
        return len(self.group_boundaries) - 1

    @property
    def group_sizes(self) -> tuple[int, ...]:
        g = self.group_boundaries
        return tuple(g[i + 1] - g[i] for i in range(self.num_groups))

    @property
    def local_sequence_start(self) -> int:
        return self.sequence_shard_bounds[self.dp_rank][0]

    @property
    def local_sequence_end(self) -> int:
        return self.sequence_shard_bounds[self.dp_rank][1]

    @property
    def local_num_sequences(self) -> int:
        s, e = self.sequence_shard_bounds[self.dp_rank]
        return e - s

    @property
    def local_num_token_slots(self) -> int:
        return self.local_num_sequences * self.padded_seq_len


@dataclass(frozen=True)
class GRPOLossContract:
    """Complete semantic request of one deterministic GRPO loss invocation."""
    logprob: LogprobContract
    sharding: LossShardingSpec
    objective: ObjectiveSpec = field(default_factory=ObjectiveSpec)
    reduction: LossReductionSpec = field(default_factory=LossReductionSpec)
    output: LossOutputSpec = field(default_factory=LossOutputSpec)
    kernel: KernelSummation = field(default_factory=KernelSummation)

    def __post_init__(self) -> None:
        for name, kind in (("logprob", LogprobContract), ("sharding", LossShardingSpec), ("objective", ObjectiveSpec),
                           ("reduction", LossReductionSpec), ("output", LossOutputSpec), ("kernel", KernelSummation)):
            if not isinstance(getattr(self, name), kind):
                raise LossContractError(f"{name} must be a {kind.__name__}")
        want = self.sharding.local_num_token_slots
        if self.logprob.mask.num_tokens != want:
            raise LossContractError(f"logprob.mask.num_tokens={self.logprob.mask.num_tokens} must equal the {want} token "
                                    f"slots this rank owns ({self.sharding.local_num_sequences} sequences x "
                                    f"{self.sharding.padded_seq_len} slots per sequence)")
        if self.logprob.reduction.determinism_scope is not self.reduction.determinism_scope:
            raise LossContractError("the loss cannot claim a stronger or weaker determinism scope than the logprob path it "
                                    f"consumes; loss={self.reduction.determinism_scope.value}, "
                                    f"logprob={self.logprob.reduction.determinism_scope.value}")
        if self.logprob.sharding.cp_world_size != self.sharding.cp_world_size:
            raise LossContractError(f"cp_world_size disagrees between the logprob contract "
                                    f"({self.logprob.sharding.cp_world_size}) and the loss sharding "
                                    f"({self.sharding.cp_world_size})")
        if self.objective.advantage.normalizer is AdvantageNormalizer.MEAN_STD_POPULATION:
            small = [i for i, n in enumerate(self.sharding.group_sizes) if n < 2]
            if small:        # a singleton group has zero variance: its sequences would contribute nothing
                raise LossContractError(f"advantage normalizer {AdvantageNormalizer.MEAN_STD_POPULATION.value} needs at "
                                        f"least 2 sequences per group; groups {small} are smaller")

    @property
    def global_token_slots(self) -> int:
        return self.sharding.num_sequences * self.sharding.padded_seq_len

    def to_dict(self) -> dict[str, Any]:
        sh, ob, rd = self.sharding, self.objective, self.reduction
        return {
            "semantic_operator": "grpo_loss", "logprob": self.logprob.to_dict(),
            "sharding": {"dp_rank": sh.dp_rank, "dp_world_size": sh.dp_world_size, "cp_rank": sh.cp_rank,
                         "cp_world_size": sh.cp_world_size, "num_sequences": sh.num_sequences,
                         "padded_seq_len": sh.padded_seq_len,
                         "sequence_shard_bounds": [list(p) for p in sh.sequence_shard_bounds],
                         "group_boundaries": list(sh.group_boundaries), "local_sequence_start": sh.local_sequence_start,
                         "local_sequence_end": sh.local_sequence_end},
            "objective": {"clip_eps_low": ob.clip.clip_eps_low, "clip_eps_high": ob.clip.clip_eps_high,
                          "clip_mode": ob.clip.mode.value, "kl_estimator": ob.kl_estimator.value, "beta": ob.beta,
                          "advantage_normalizer": ob.advantage.normalizer.value,
                          "advantage_variance": ob.advantage.variance.value, "advantage_std_eps": ob.advantage.std_eps,
                          "advantage_replication": ob.advantage.replication.value},
            "reduction": {"token_normalizer": rd.token_normalizer.value, "summation_order": rd.summation_order.value,
                          "acc_dtype": rd.acc_dtype.value, "transport": rd.transport.value,
                          "downcast_at": rd.downcast_at.value, "determinism_scope": rd.determinism_scope.value,
                          "fixed_normalizer_constant": rd.fixed_normalizer_constant, "cp_is_merge_axis": False,
                          "dp_is_merge_axis": True},
            "output": {"loss_dtype": self.output.loss_dtype.value, "placement": self.output.placement.value},
            "kernel": self.kernel.to_dict(),
        }

    def cross_rank_fingerprint(self) -> str:
        """Identity shared by all dp x tp ranks of one invocation: rank fields, local bounds and the nested
        log-prob mask (every DP rank holds other sequences) are left out; the global geometry stays pinned by
        num_sequences, padded_seq_len and the full shard table."""
        payload = self.to_dict()
        lp = payload["logprob"]
        lp.pop("mask", None)
        lp["sharding"] = {k: v for k, v in lp["sharding"].items()
                          if k not in {"tp_rank", "cp_rank", "local_vocab_start", "local_vocab_end"}}
        payload["sharding"] = {k: v for k, v in payload["sharding"].items()
                               if k not in {"dp_rank", "cp_rank", "local_sequence_start", "local_sequence_end"}}
        return stable_hash(payload)

    def preflight(self, group=None) -> None:
        assert_same_across_ranks(self.cross_rank_fingerprint(), group, "GRPO loss contract")

    @classmethod
    def simple(cls, *, num_sequences: int, padded_seq_len: int, samples_per_prompt: int = 8, real_vocab_size: int = 151936,
               padded_vocab_size: int | None = None, dp_rank: int = 0, dp_world_size: int = 1, tp_rank: int = 0,
               tp_world_size: int = 1, clip_eps_low: float = 0.2, clip_eps_high: float = 0.2, beta: float = 0.001,
               kl_estimator: KLEstimator = KLEstimator.K3_UNBIASED,
               token_normalizer: TokenNormalizer = TokenNormalizer.GLOBAL_ACTIVE_TOKENS, temperature: float = 1.0
               ) -> "GRPOLossContract":
        """Equal shards, equal groups, every token slot active."""
        if samples_per_prompt < 2:
            raise LossContractError("group-relative advantages need at least 2 samples per prompt")
        sh = LossShardingSpec.even(dp_rank=dp_rank, dp_world_size=dp_world_size, num_sequences=num_sequences,
                                   padded_seq_len=padded_seq_len, samples_per_prompt=samples_per_prompt)
        lp = LogprobContract.for_tokens(sh.local_num_token_slots, real_vocab_size=real_vocab_size,
                                        padded_vocab_size=padded_vocab_size, tp_rank=tp_rank, tp_world_size=tp_world_size,
                                        temperature=temperature)
        return cls(lp, sh, ObjectiveSpec(ClipSpec(clip_eps_low, clip_eps_high), kl_estimator=kl_estimator, beta=beta),
                   LossReductionSpec(token_normalizer=token_normalizer))


@dataclass(frozen=True)
class LossBackendCapability:
    backend_id: str
    token_normalizers: frozenset
    kl_estimators: frozenset
    advantage_normalizers: frozenset
    determinism_scopes: frozenset
    dp_world_sizes: tuple[int, ...] | None = None
    supports_variable_group_sizes: bool = False
    supports_asymmetric_clip: bool = False
    implementation_kind: str = "production"

    def __post_init__(self) -> None:
        if not isinstance(self.backend_id, str) or not self.backend_id.strip():
            raise LossContractError("backend_id must be a non-empty string")
        if self.backend_id.strip().lower() in RESERVED_DISPATCH_POLICIES:
            raise LossContractError(f"backend_id={self.backend_id!r} shadows a reserved dispatch policy keyword")
        object.__setattr__(self, "backend_id", self.backend_id.strip())
        for name, kind in (("token_normalizers", TokenNormalizer), ("kl_estimators", KLEstimator),
                           ("advantage_normalizers", AdvantageNormalizer), ("determinism_scopes", DeterminismScope)):
            try:
                values = frozenset(_enum_value(kind, v, name) for v in getattr(self, name))
            except TypeError as exc:
                raise LossContractError(f"{name} must be an iterable of enum values") from exc
            if not values:
                raise LossContractError(f"{name} must not be empty")
            object.__setattr__(self, name, values)
        object.__setattr__(self, "dp_world_sizes", _world_sizes(self.dp_world_sizes, "dp_world_sizes"))
        for flag in ("supports_variable_group_sizes", "supports_asymmetric_clip"):
            if not isinstance(getattr(self, flag), bool):
                raise LossContractError(f"{flag} must be a bool")
        if self.implementation_kind not in {"production", "reference"}:
            raise LossContractError("implementation_kind must be production or reference")

    def incompatibilities(self, contract: GRPOLossContract) -> tuple[str, ...]:
        why: list[str] = []
        rd, ob, sh = contract.reduction, contract.objective, contract.sharding
        if rd.token_normalizer not in self.token_normalizers:
            why.append(f"token_normalizer={rd.token_normalizer.value} is unsupported")
        if ob.kl_estimator not in self.kl_estimators:
            why.append(f"kl_estimator={ob.kl_estimator.value} is unsupported")
        if ob.advantage.normalizer not in self.advantage_normalizers:
            why.append(f"advantage normalizer={ob.advantage.normalizer.value} is unsupported")
        if rd.determinism_scope not in self.determinism_scopes:
            why.append(f"determinism_scope={rd.determinism_scope.value} is unsupported")
        if self.dp_world_sizes is not None and sh.dp_world_size not in self.dp_world_sizes:
            why.append(f"DP={sh.dp_world_size} is unsupported")
        if len(set(sh.group_sizes)) > 1 and not self.supports_variable_group_sizes:
            why.append("variable advantage group sizes are unsupported")
        if ob.clip.clip_eps_low != ob.clip.clip_eps_high and not self.supports_asymmetric_clip:
            why.append("asymmetric ratio clipping is unsupported")
        return tuple(why)

    def supports(self, contract: GRPOLossContract) -> bool:
        return not self.incompatibilities(contract)

    def to_dict(self) -> dict[str, Any]:
        return {"backend_id": self.backend_id, "token_normalizers": sorted(v.value for v in self.token_normalizers),
                "kl_estimators": sorted(v.value for v in self.kl_estimators),
                "advantage_normalizers": sorted(v.value for v in self.advantage_normalizers),
                "determinism_scopes": sorted(v.value for v in self.determinism_scopes),
                "dp_world_sizes": list(self.dp_world_sizes) if self.dp_world_sizes else None,
                "supports_variable_group_sizes": self.supports_variable_group_sizes,
                "supports_asymmetric_clip": self.supports_asymmetric_clip, "implementation_kind": self.implementation_kind}


@dataclass(frozen=True)
class LossDispatchResult:
    op: Any
    capability: LossBackendCapability
    provenance: dict[str, Any]


B200_LOSS_CAPABILITY = LossBackendCapability(
    backend_id="b200-grpo-loss", token_normalizers=frozenset({TokenNormalizer.GLOBAL_ACTIVE_TOKENS, TokenNormalizer.FIXED_CONSTANT}),
    kl_estimators=frozenset({KLEstimator.K3_UNBIASED}), advantage_normalizers=frozenset(AdvantageNormalizer),
    determinism_scopes=frozenset(DeterminismScope), dp_world_sizes=(1, 2, 4, 8), supports_asymmetric_clip=True)
REFERENCE_LOSS_CAPABILITY = LossBackendCapability(
    backend_id="pytorch-distributed-grpo-loss", token_normalizers=frozenset(TokenNormalizer), kl_estimators=frozenset(KLEstimator),
    advantage_normalizers=frozenset(AdvantageNormalizer), determinism_scopes=frozenset(DeterminismScope),
    supports_variable_group_sizes=True, supports_asymmetric_clip=True, implementation_kind="reference")

__all__ = ["AdvantageNormalizer", "AdvantageSpec", "B200_LOSS_CAPABILITY", "ClipMode", "ClipSpec", "GRPOLossContract",
           "GRPO_CONTRACT_ID", "GroupReplication", "KLEstimator", "KernelSummation", "LossBackendCapability",
           "LossContractError", "LossDispatchResult", "LossOutputSpec", "LossPlacement", "LossReductionSpec",
           "LossShardingSpec", "LossTransport", "ObjectiveSpec", "REFERENCE_LOSS_CAPABILITY", "SummationOrder",
           "TokenNormalizer", "VarianceFormula"]
