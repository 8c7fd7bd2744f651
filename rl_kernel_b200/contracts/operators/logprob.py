"""Selected-token log-prob contract (parity: rl_engine/contracts/operators/logprob.py:34-652).

A ``LogprobContract`` is the complete semantic request of one selected-log-prob invocation under
vocabulary-parallel tensor parallelism: who owns which vocabulary range (``ShardingSpec``), which
tokens count (``MaskSpec``), how the per-shard (max, sum-exp) partials are merged
(``ReductionSpec``: fp32, global order, all-gather as pure transport, one downcast at the final
write) and what comes out (``LogprobOutputSpec``: fp32 log-prob and vocabulary-domain LSE,
replicated across the TP group).  ``LogprobBackendCapability`` is what a backend declares;
``incompatibilities`` explains every reason it cannot serve a contract.

Additions of this package: ``TileNumerics`` pins the 128-id tile arithmetic that the sm_100a
kernels and the PyTorch reference share, ``LogpInput`` / ``TopPReplay`` name the operand kind and
how a restricted sampling support is replayed, and ``VocabShardingSpec`` builds the even,
tile-aligned partition these kernels require.
"""
from __future__ import annotations

import enum
import hashlib
from dataclasses import dataclass, field
from enum import Enum
from typing import Any

from rl_kernel_b200.contracts.operators._base import (ContractBase, assert_same_across_ranks, make_validators,
                                                       stable_hash)

RESERVED_DISPATCH_POLICIES = frozenset({"auto", "production", "reference", "deterministic"})
IMPLEMENTATION_KINDS = frozenset({"production", "reference"})
LOGPROB_CONTRACT_ID = "logprob.vocab_tile128.v1"


class LogprobContractError(ValueError):
    """Log-prob metadata does not describe a valid invocation."""


(_enum_value, _positive_int, _non_negative_int, _plain_int, _integer_tuple, _coerce,
 _world_sizes) = make_validators(LogprobContractError)


class LogprobRole(str, Enum):
    TRAIN = "train"
    INFER = "infer"


class LogprobDType(str, Enum):
    BF16 = "bf16"
    FP16 = "fp16"
    FP32 = "fp32"


class LogprobMerge(str, Enum):
    MAX_SUMEXP = "max_sumexp"


class MergeAxis(str, Enum):
    TP_VOCAB = "tp_vocab"            # the only reduction axis; CP never merges log-probs


class ReductionOrder(str, Enum):
    GLOBAL_VOCAB_SHARD_INDEX = "global_vocab_shard_index"


class ReductionTransport(str, Enum):
    ALL_GATHER = "all_gather"        # collectives move partials, they never reduce numerically
    PEER_STORE = "peer_store"        # the same partials written into every rank's buffer from the GEMM epilogue


class DowncastPoint(str, Enum):
    FINAL_WRITE = "final_write"


class ReductionEngine(str, Enum):
    IN_OP_REFERENCE = "in_op_reference"
    FUSED_EPILOGUE = "fused_epilogue"


class DeterminismScope(str, Enum):
    """``fixed_topology``: bit-reproducible at one TP degree.  ``cross_tp_bitwise``: additionally the
    same bits at every TP degree, which needs a tile decomposition and merge tree that do not depend
    on the partition (the TP degree only selects who computes which tiles)."""
    FIXED_TOPOLOGY = "fixed_topology"
    CROSS_TP_BITWISE = "cross_tp_bitwise"


class MaskMode(str, Enum):
    EXPLICIT_ACTIVE_MASK = "explicit_active_mask"
    IGNORE_INDEX = "ignore_index"


class TPPlacement(str, Enum):
    REPLICATED = "replicated"


class LogpInput(str, enum.Enum):
    LOGITS = "logits"
    HIDDEN = "hidden"               # fused linear -> log-prob: the logits are never materialised


class TopPReplay(str, enum.Enum):
    NONE = "none"
    KEEP_THRESHOLD = "keep_threshold"   # one scaled-logit threshold per token, applied in the kernel
    ID_LIST = "id_list"                 # a compact (<= 64) id list per token


@dataclass(frozen=True)
class ShardingSpec:
    """Vocabulary ownership of one invocation.  ``vocab_shard_bounds[r]`` is rank r's half-open id
    range; the table is required on every rank and partitions [0, padded_vocab_size) contiguously in
    rank order.  Ids in [real_vocab_size, padded_vocab_size) are padding."""
    tp_rank: int
    tp_world_size: int
    vocab_shard_bounds: tuple[tuple[int, int], ...]
    real_vocab_size: int
    padded_vocab_size: int
    cp_rank: int = 0
    cp_world_size: int = 1

    def __post_init__(self) -> None:
        tp = _positive_int(self.tp_world_size, "tp_world_size")
        if _non_negative_int(self.tp_rank, "tp_rank") >= tp:
            raise LogprobContractError(f"tp_rank={self.tp_rank} must be smaller than tp_world_size={tp}")
        cp = _positive_int(self.cp_world_size, "cp_world_size")
        if _non_negative_int(self.cp_rank, "cp_rank") >= cp:
            raise LogprobContractError(f"cp_rank={self.cp_rank} must be smaller than cp_world_size={cp}")
        real = _positive_int(self.real_vocab_size, "real_vocab_size")
        padded = _positive_int(self.padded_vocab_size, "padded_vocab_size")
        if padded < real:
            raise LogprobContractError(f"padded_vocab_size={padded} must not be smaller than real_vocab_size={real}")
        try:
            bounds = tuple((pair[0], pair[1]) for pair in self.vocab_shard_bounds)
        except (TypeError, IndexError) as exc:
            raise LogprobContractError("vocab_shard_bounds must be an iterable of (start, end) integer pairs") from exc
        if len(bounds) != tp:
            raise LogprobContractError("vocab_shard_bounds must declare exactly one (start, end) pair per TP rank; "
                                       f"got {len(bounds)} pairs for tp_world_size={tp}")
        expect = 0
        for r, (start, end) in enumerate(bounds):
            _plain_int(start, f"vocab_shard_bounds[{r}][0]")
            _plain_int(end, f"vocab_shard_bounds[{r}][1]")
            if end <= start:
                raise LogprobContractError(f"vocab_shard_bounds[{r}] must satisfy end > start; got [{start}, {end})")
            if start != expect:
                raise LogprobContractError("vocab_shard_bounds must form a contiguous [0, padded_vocab_size) partition in "
                                           f"TP-rank order; rank {r} starts at {start}, expected {expect}")
            expect = end
        if expect != padded:
            raise LogprobContractError(f"vocab_shard_bounds must cover padded_vocab_size exactly; covered {expect}, "
                                       f"declared {padded}")
        object.__setattr__(self, "vocab_shard_bounds", bounds)

    @classmethod
    def even(cls, *, tp_rank: int, tp_world_size: int, real_vocab_size: int, padded_vocab_size: int,
             cp_rank: int = 0, cp_world_size: int = 1) -> "ShardingSpec":
        """The equal-sized partition (what Megatron and vLLM produce)."""
        if padded_vocab_size % tp_world_size:
            raise LogprobContractError(f"padded_vocab_size={padded_vocab_size} is not divisible by TP={tp_world_size}")
        per = padded_vocab_size // tp_world_size
        return cls(tp_rank, tp_world_size, tuple((r * per, (r + 1) * per) for r in range(tp_world_size)),
                   real_vocab_size, padded_vocab_size, cp_rank, cp_world_size)

    @property
    def local_vocab_start(self) -> int:
        return self.vocab_shard_bounds[self.tp_rank][0]

    @property
    def local_vocab_end(self) -> int:
        return self.vocab_shard_bounds[self.tp_rank][1]

    @property
    def local_vocab_size(self) -> int:
        start, end = self.vocab_shard_bounds[self.tp_rank]
        return end - start

    def owner_rank(self, token_id: int) -> int:
        token_id = _plain_int(token_id, "token_id")
        if not 0 <= token_id < self.real_vocab_size:
            raise LogprobContractError(f"token_id={token_id} is outside the real vocabulary [0, {self.real_vocab_size}); "
                                       "mask it as inactive instead")
        for r, (start, end) in enumerate(self.vocab_shard_bounds):
            if start <= token_id < end:
                return r
        raise LogprobContractError(f"token_id={token_id} is not covered by any declared vocab shard")

    def tile_aligned(self, tile: int) -> bool:
        return all(start % tile == 0 for start, _ in self.vocab_shard_bounds)


@dataclass(frozen=True)
class MaskSpec:
    """Which tokens are active.  Inactive tokens are excluded from drift aggregates and from the
    single-owner target gather; their targets may hold ``ignore_index`` or anything else."""
    num_tokens: int
    active_mask: tuple[bool, ...]
    ignore_index: int = -100
    _active_token_count: int = field(init=False, repr=False, compare=False)
    _active_mask_sha256: str = field(init=False, repr=False, compare=False)

    def __post_init__(self) -> None:
        n = _positive_int(self.num_tokens, "num_tokens")
        _plain_int(self.ignore_index, "ignore_index")
        try:
            mask = tuple(self.active_mask)
        except TypeError as exc:
            raise LogprobContractError("active_mask must be an iterable of booleans") from exc
        for i, v in enumerate(mask):
            if not isinstance(v, bool):
                raise LogprobContractError(f"active_mask[{i}] must be a bool; got {v!r}")
        if len(mask) != n:
            raise LogprobContractError(f"active_mask must contain exactly one entry per token; got {len(mask)} entries for "
                                       f"num_tokens={n}")
        object.__setattr__(self, "active_mask", mask)
        object.__setattr__(self, "_active_token_count", sum(mask))
        object.__setattr__(self, "_active_mask_sha256", hashlib.sha256(bytes(mask)).hexdigest())

    @classmethod
    def all_active(cls, num_tokens: int, ignore_index: int = -100) -> "MaskSpec":
        return cls(num_tokens, (True,) * num_tokens, ignore_index)

    @classmethod
    def from_tensor(cls, mask, ignore_index: int = -100) -> "MaskSpec":
        flat = [bool(v) for v in mask.reshape(-1).tolist()]
        return cls(len(flat), tuple(flat), ignore_index)

    @property
    def active_token_count(self) -> int:
        return self._active_token_count

    @property
    def active_mask_sha256(self) -> str:
        return self._active_mask_sha256


@dataclass(frozen=True)
class ReductionSpec:
    """How shard partials become one log-sum-exp.  Columns at or beyond the real vocabulary are -inf
    before anything else; every rank computes fp32 (m, s) partials; partials are moved, never reduced,
    by the transport; every rank merges them in global order:
    M = max m, S = sum s * exp(m - M), LSE = M + log S, logp = target_logit - LSE.  The identity
    partial of an all-padding range is (-inf, 0) and is used directly (never exp(-inf - -inf))."""
    merge: LogprobMerge = LogprobMerge.MAX_SUMEXP
    merge_axis: MergeAxis = MergeAxis.TP_VOCAB
    acc_dtype: LogprobDType = LogprobDType.FP32
    order: ReductionOrder = ReductionOrder.GLOBAL_VOCAB_SHARD_INDEX
    transport: ReductionTransport = ReductionTransport.ALL_GATHER
    downcast_at: DowncastPoint = DowncastPoint.FINAL_WRITE
    engine: ReductionEngine = ReductionEngine.IN_OP_REFERENCE
    determinism_scope: DeterminismScope = DeterminismScope.CROSS_TP_BITWISE

    def __post_init__(self) -> None:
        _coerce(self, determinism_scope=DeterminismScope, merge=LogprobMerge, merge_axis=MergeAxis, acc_dtype=LogprobDType,
                order=ReductionOrder, transport=ReductionTransport, downcast_at=DowncastPoint, engine=ReductionEngine)
        if self.acc_dtype is not LogprobDType.FP32:
            raise LogprobContractError(f"TP logprob accumulation must be fp32; got {self.acc_dtype.value}")


@dataclass(frozen=True)
class LogprobOutputSpec:
    selected_logp_dtype: LogprobDType = LogprobDType.FP32
    lse_dtype: LogprobDType = LogprobDType.FP32
    tp_placement: TPPlacement = TPPlacement.REPLICATED

    def __post_init__(self) -> None:
        _coerce(self, selected_logp_dtype=LogprobDType, lse_dtype=LogprobDType, tp_placement=TPPlacement)
        if self.selected_logp_dtype is not LogprobDType.FP32:
            raise LogprobContractError(f"selected logprob output must be fp32; got {self.selected_logp_dtype.value}")
        if self.lse_dtype is not LogprobDType.FP32:
            raise LogprobContractError(f"vocab LSE output must be fp32; got {self.lse_dtype.value}")


@dataclass(frozen=True)
class TileNumerics(ContractBase):
    """The in-tile arithmetic shared by the kernels and the PyTorch reference: bf16 logits, scaled by
    1/temperature before the maximum with one fp32 multiply; 128 consecutive global ids per tile; four
    interleaved sequential chains (position mod 4) combined as (c0+c1)+(c2+c3); tiles folded into the
    row sum with one fma each in ascending order; the fast hardware exponential."""
    tile: int = 128
    temperature: float = 1.0
    temperature_scales: str = "logits_before_max"
    tile_sum: str = "four_interleaved_chains"
    row_merge: str = "ascending_tile_fma"
    exp: str = "__expf"
    clamp_non_positive: bool = True
    input_kind: LogpInput = LogpInput.HIDDEN
    top_p_replay: TopPReplay = TopPReplay.NONE
    contract_id: str = LOGPROB_CONTRACT_ID

    def __post_init__(self) -> None:
        if self.temperature <= 0:
            raise LogprobContractError("temperature must be positive")
        if self.tile <= 0 or self.tile % 4:
            raise LogprobContractError("tile must be a positive multiple of 4")
        _coerce(self, input_kind=LogpInput, top_p_replay=TopPReplay)


@dataclass(frozen=True)
class LogprobContract:
    """Complete semantic request consumed by contract-aware dispatch."""
    role: LogprobRole
    dtype: LogprobDType
    mask: MaskSpec
    sharding: ShardingSpec
    reduction: ReductionSpec = field(default_factory=ReductionSpec)
    output: LogprobOutputSpec = field(default_factory=LogprobOutputSpec)
    export_lse: bool = True
    numerics: TileNumerics = field(default_factory=TileNumerics)

    def __post_init__(self) -> None:
        _coerce(self, role=LogprobRole, dtype=LogprobDType)
        for name, kind in (("mask", MaskSpec), ("sharding", ShardingSpec), ("reduction", ReductionSpec),
                           ("output", LogprobOutputSpec), ("numerics", TileNumerics)):
            if not isinstance(getattr(self, name), kind):
                raise LogprobContractError(f"{name} must be a {kind.__name__}")
        if not isinstance(self.export_lse, bool) or not self.export_lse:
            raise LogprobContractError("export_lse must be True for the vocab-domain LSE drift contract")
        if 0 <= self.mask.ignore_index < self.sharding.real_vocab_size:
            raise LogprobContractError(f"ignore_index={self.mask.ignore_index} must not collide with the real vocabulary "
                                       f"[0, {self.sharding.real_vocab_size})")

    @property
    def temperature(self) -> float:
        return self.numerics.temperature

    def to_dict(self) -> dict[str, Any]:
        """Stable, JSON-compatible provenance of the request (the mask is represented by its digest)."""
        sh, red, out = self.sharding, self.reduction, self.output
        return {
            "semantic_operator": "selected_token_logprob",
            "role": self.role.value, "dtype": self.dtype.value, "export_lse": self.export_lse, "lse_domain": "vocab",
            "mask": {"num_tokens": self.mask.num_tokens, "active_token_count": self.mask.active_token_count,
                     "active_mask_sha256": self.mask.active_mask_sha256, "ignore_index": self.mask.ignore_index},
            "sharding": {"tp_rank": sh.tp_rank, "tp_world_size": sh.tp_world_size, "cp_rank": sh.cp_rank,
                         "cp_world_size": sh.cp_world_size, "vocab_shard_bounds": [list(p) for p in sh.vocab_shard_bounds],
                         "real_vocab_size": sh.real_vocab_size, "padded_vocab_size": sh.padded_vocab_size,
                         "local_vocab_start": sh.local_vocab_start, "local_vocab_end": sh.local_vocab_end},
            "reduction": {"merge": red.merge.value, "merge_axis": red.merge_axis.value, "acc_dtype": red.acc_dtype.value,
                          "order": red.order.value, "transport": red.transport.value, "downcast_at": red.downcast_at.value,
                          "engine": red.engine.value, "determinism_scope": red.determinism_scope.value,
                          "cp_is_merge_axis": False},
            "output": {"selected_logp_dtype": out.selected_logp_dtype.value, "lse_dtype": out.lse_dtype.value,
                       "tp_placement": out.tp_placement.value},
            "numerics": self.numerics.to_dict(),
        }

    def cross_rank_fingerprint(self) -> str:
        """Rank-independent identity: the rank fields and the local bounds derived from them are left out,
        so every rank of one logical invocation computes the same value."""
        payload = self.to_dict()
        payload["sharding"] = {k: v for k, v in payload["sharding"].items()
                               if k not in {"tp_rank", "cp_rank", "local_vocab_start", "local_vocab_end"}}
        return stable_hash(payload)

    def preflight(self, group=None) -> None:
        assert_same_across_ranks(self.cross_rank_fingerprint(), group, "logprob contract")

    @classmethod
    def for_tokens(cls, num_tokens: int, *, real_vocab_size: int, padded_vocab_size: int | None = None, tp_rank: int = 0,
                   tp_world_size: int = 1, role: LogprobRole = LogprobRole.TRAIN, dtype: LogprobDType = LogprobDType.BF16,
                   temperature: float = 1.0, active_mask=None, engine: ReductionEngine = ReductionEngine.IN_OP_REFERENCE
                   ) -> "LogprobContract":
        """The common case: an even partition, every token active unless a mask is given."""
        padded = padded_vocab_size or real_vocab_size
        mask = MaskSpec.all_active(num_tokens) if active_mask is None else MaskSpec.from_tensor(active_mask)
        return cls(role, dtype, mask, ShardingSpec.even(tp_rank=tp_rank, tp_world_size=tp_world_size,
                                                        real_vocab_size=real_vocab_size, padded_vocab_size=padded),
                   ReductionSpec(engine=engine), numerics=TileNumerics(temperature=temperature))


@dataclass(frozen=True)
class LogprobBackendCapability:
    """What a concrete backend declares to contract-aware dispatch."""
    backend_id: str
    roles: frozenset
    dtypes: frozenset
    tp_world_sizes: tuple[int, ...] | None = None
    cp_world_sizes: tuple[int, ...] | None = None
    supports_vocab_padding: bool = False
    mask_modes: frozenset = frozenset()
    exports_vocab_lse: bool = False
    determinism_scopes: frozenset = frozenset()
    implementation_kind: str = "production"
    requires_tile_aligned_shards: int = 0       # 0 = no requirement, else the tile size shard starts must divide by
    top_p_replay: frozenset = frozenset({TopPReplay.NONE})

    def __post_init__(self) -> None:
        if not isinstance(self.backend_id, str) or not self.backend_id.strip():
            raise LogprobContractError("backend_id must be a non-empty string")
        if self.backend_id.strip().lower() in RESERVED_DISPATCH_POLICIES:
            raise LogprobContractError(f"backend_id={self.backend_id!r} shadows a reserved dispatch policy keyword")
        object.__setattr__(self, "backend_id", self.backend_id.strip())
        try:
            roles = frozenset(_enum_value(LogprobRole, v, "roles") for v in self.roles)
            dtypes = frozenset(_enum_value(LogprobDType, v, "dtypes") for v in self.dtypes)
        except TypeError as exc:
            raise LogprobContractError("roles and dtypes must be iterables of enum values") from exc
        if not roles or not dtypes:
            raise LogprobContractError("backend roles and dtypes must not be empty")
        try:
            modes = frozenset(_enum_value(MaskMode, v, "mask_modes") for v in self.mask_modes)
            scopes = frozenset(_enum_value(DeterminismScope, v, "determinism_scopes") for v in self.determinism_scopes)
            replay = frozenset(_enum_value(TopPReplay, v, "top_p_replay") for v in self.top_p_replay)
        except TypeError as exc:
            raise LogprobContractError("mask_modes and determinism_scopes must be iterables of enum values") from exc
        for flag in ("supports_vocab_padding", "exports_vocab_lse"):
            if not isinstance(getattr(self, flag), bool):
                raise LogprobContractError(f"{flag} must be a bool")
        if self.implementation_kind not in IMPLEMENTATION_KINDS:
            raise LogprobContractError(f"implementation_kind must be one of: {', '.join(sorted(IMPLEMENTATION_KINDS))}")
        for name, value in (("roles", roles), ("dtypes", dtypes), ("mask_modes", modes), ("determinism_scopes", scopes),
                            ("top_p_replay", replay),
                            ("tp_world_sizes", _world_sizes(self.tp_world_sizes, "tp_world_sizes")),
                            ("cp_world_sizes", _world_sizes(self.cp_world_sizes, "cp_world_sizes"))):
            object.__setattr__(self, name, value)

    def incompatibilities(self, contract: LogprobContract) -> tuple[str, ...]:
        """Every reason this backend cannot materialise ``contract``."""
        why: list[str] = []
        if contract.role not in self.roles:
            why.append(f"role={contract.role.value} is unsupported")
        if contract.dtype not in self.dtypes:
            why.append(f"dtype={contract.dtype.value} is unsupported")
        tp, cp = contract.sharding.tp_world_size, contract.sharding.cp_world_size
        if self.tp_world_sizes is not None and tp not in self.tp_world_sizes:
            why.append(f"TP={tp} is unsupported")
        if self.cp_world_sizes is not None and cp not in self.cp_world_sizes:
            why.append(f"CP={cp} is unsupported")
        if contract.sharding.padded_vocab_size != contract.sharding.real_vocab_size and not self.supports_vocab_padding:
            why.append("padded-vs-real vocab masking is unsupported")
        if contract.mask.active_token_count != contract.mask.num_tokens and MaskMode.EXPLICIT_ACTIVE_MASK not in self.mask_modes:
            why.append("explicit active-token masking is unsupported")
        if contract.export_lse and not self.exports_vocab_lse:
            why.append("vocab-domain LSE export is unsupported")
        if contract.reduction.determinism_scope not in self.determinism_scopes:
            why.append(f"determinism_scope={contract.reduction.determinism_scope.value} is unsupported")
        if self.requires_tile_aligned_shards and not contract.sharding.tile_aligned(self.requires_tile_aligned_shards):
            why.append(f"vocab shards must start on {self.requires_tile_aligned_shards}-id tile boundaries")
        if contract.numerics.top_p_replay not in self.top_p_replay:
            why.append(f"top_p_replay={contract.numerics.top_p_replay.value} is unsupported")
        return tuple(why)

    def supports(self, contract: LogprobContract) -> bool:
        return not self.incompatibilities(contract)

    def to_dict(self) -> dict[str, Any]:
        return {"backend_id": self.backend_id, "roles": sorted(r.value for r in self.roles),
                "dtypes": sorted(d.value for d in self.dtypes),
                "tp_world_sizes": list(self.tp_world_sizes) if self.tp_world_sizes else None,
                "cp_world_sizes": list(self.cp_world_sizes) if self.cp_world_sizes else None,
                "supports_vocab_padding": self.supports_vocab_padding, "mask_modes": sorted(m.value for m in self.mask_modes),
                "exports_vocab_lse": self.exports_vocab_lse,
                "determinism_scopes": sorted(s.value for s in self.determinism_scopes),
                "implementation_kind": self.implementation_kind,
                "requires_tile_aligned_shards": self.requires_tile_aligned_shards,
                "top_p_replay": sorted(t.value for t in self.top_p_replay)}


@dataclass(frozen=True)
class LogprobDispatchResult:
    """A concrete backend plus the provenance bound to the request."""
    op: Any
    capability: LogprobBackendCapability
    provenance: dict[str, Any]


@dataclass(frozen=True)
class VocabShardingSpec(ContractBase):
    """The even, tile-aligned partition the sm_100a kernels use: no 128-id tile straddles a shard when the
    padded vocabulary is a multiple of ``tile * tp_size``.  ``sharding(rank)`` gives the general spec."""
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

    def sharding(self, tp_rank: int = 0) -> ShardingSpec:
        return ShardingSpec.even(tp_rank=tp_rank, tp_world_size=self.tp_size, real_vocab_size=self.real_vocab,
                                 padded_vocab_size=self.padded_vocab)


_ALL_ROLES = frozenset(LogprobRole)
B200_LOGPROB_CAPABILITY = LogprobBackendCapability(
    backend_id="b200-tcgen05", roles=_ALL_ROLES, dtypes=frozenset({LogprobDType.BF16}), tp_world_sizes=(1, 2, 4, 8),
    supports_vocab_padding=True, mask_modes=frozenset(MaskMode), exports_vocab_lse=True,
    determinism_scopes=frozenset(DeterminismScope), implementation_kind="production", requires_tile_aligned_shards=128,
    top_p_replay=frozenset(TopPReplay))
REFERENCE_LOGPROB_CAPABILITY = LogprobBackendCapability(
    backend_id="pytorch-vocab-parallel-logp", roles=_ALL_ROLES, dtypes=frozenset(LogprobDType), supports_vocab_padding=True,
    mask_modes=frozenset(MaskMode), exports_vocab_lse=True, determinism_scopes=frozenset(DeterminismScope),
    implementation_kind="reference", requires_tile_aligned_shards=128, top_p_replay=frozenset(TopPReplay))

__all__ = ["IMPLEMENTATION_KINDS", "RESERVED_DISPATCH_POLICIES", "LOGPROB_CONTRACT_ID", "DeterminismScope", "DowncastPoint",
           "LogprobBackendCapability", "LogprobContract", "LogprobContractError", "LogprobDType", "LogprobDispatchResult",
           "LogprobMerge", "LogprobOutputSpec", "LogprobRole", "LogpInput", "MaskMode", "MaskSpec", "MergeAxis",
           "ReductionEngine", "ReductionOrder", "ReductionSpec", "ReductionTransport", "ShardingSpec", "TPPlacement",
           "TileNumerics", "TopPReplay", "VocabShardingSpec", "B200_LOGPROB_CAPABILITY", "REFERENCE_LOGPROB_CAPABILITY"]
