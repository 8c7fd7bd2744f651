"""Attention contract (parity: rl_engine/contracts/operators/attention.py:27-1789).

An ``AttentionContract`` is the complete semantic request of one attention invocation under
tensor / context / sequence parallelism: which heads and which logical token blocks the calling
rank owns (``ShardingSpec``), how partial ``(out, lse)`` states merge (``ReductionSpec``: fp32,
global block order, one downcast at the final write), whether the key axis may be split
(``SplitKVSpec`` and the runtime plans that prove what actually ran), the paged KV-cache identity
(``KVCacheSpec``), where RoPE sits (``RoPESpec``) and how the QKV / output projections execute
(``AttentionProjectionSpec``).  ``AttentionBackendCapability.incompatibilities`` explains every
reason a backend cannot serve a contract.

The one schedule of the sm_100a kernels is ``canonical_128_key_blocks_no_splitkv``: every query
row walks 128-key blocks in ascending global order with one running (max, sum) pair, whatever the
batch, the packing, the page table or the CP degree.  Split-KV is therefore never requested
here, but the policy objects exist so that a contract coming from another engine can be compared
field by field.  ``CPLayout`` and ``ShardingSpec.for_layout`` build the block tables of the two
context-parallel layouts this library runs (contiguous and Megatron zigzag).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Iterable

from rl_kernel_b200.contracts.operators._base import assert_same_across_ranks, is_plain_int, make_validators, stable_hash

STRICT_ATTENTION_PRODUCTION_CORE_ID = "rlkernel.attention.b200_tcgen05.canonical_128_key_blocks.v1"
STRICT_ATTENTION_REFERENCE_CORE_ID = "rlkernel.attention.deterministic_core.v1"
STRICT_ATTENTION_CORE_ID = STRICT_ATTENTION_REFERENCE_CORE_ID
STRICT_ATTENTION_SCHEDULE_ID = "canonical_128_key_blocks_no_splitkv"
STRICT_ATTENTION_FA4_SCHEDULE_ID = STRICT_ATTENTION_SCHEDULE_ID
STRICT_ATTENTION_RING_SCHEDULE_ID = "rlkernel.attention.strict_ring_state.v1"
ATTENTION_CONTRACT_ID = "attention.canonical_block128.v1"
CANONICAL_KV_BLOCK = 128


class AttentionContractError(ValueError):
    """Attention metadata does not describe a valid invocation."""


(_enum_value, _positive_int, _non_negative_int, _plain_int, _integer_tuple, _coerce,
 _world_sizes) = make_validators(AttentionContractError)


class AttentionRole(str, Enum):
    TRAIN = "train"
    INFER = "infer"


class AttentionMode(str, Enum):
    PREFILL = "prefill"
    CHUNKED_PREFILL = "chunked_prefill"
    DECODE = "decode"


class AttentionDType(str, Enum):
    BF16 = "bf16"
    FP16 = "fp16"
    FP32 = "fp32"


class AttentionMerge(str, Enum):
    ONLINE_SOFTMAX_LSE = "online_softmax_lse"


class ReductionOrder(str, Enum):
    GLOBAL_BLOCK_INDEX = "global_block_index"


class DowncastPoint(str, Enum):
    FINAL_WRITE = "final_write"


class ReductionEngine(str, Enum):
    IN_OP_REFERENCE = "in_op_reference"
    IN_KERNEL = "in_kernel"              # one kernel walks local and remote blocks: nothing is merged afterwards


class SplitKVMode(str, Enum):
    DISABLED = "disabled"
    FIXED = "fixed"
    AUTO = "auto"


class ProjectionCollective(str, Enum):
    NONE = "none"
    ALL_REDUCE = "all_reduce"
    ALL_GATHER = "all_gather"
    REDUCE_SCATTER = "reduce_scatter"


class RoPEState(str, Enum):
    PRE_ROPE = "pre_rope"
    POST_ROPE = "post_rope"


class RoPECastPoint(str, Enum):
    NONE = "none"
    BEFORE_ROPE = "before_rope"
    AFTER_ROPE = "after_rope"


class RoPEFusionBoundary(str, Enum):
    UNFUSED_ROPE_ATTENTION = "unfused_rope_attention"
    FUSED_ROPE_ATTENTION = "fused_rope_attention"


class CPLayout(str, enum.Enum):
    NONE = "none"
    CONTIGUOUS = "contiguous"                  # rank c owns tokens [c S/cp, (c+1) S/cp)
    ZIGZAG = "zigzag"                          # Megatron: rank c owns chunks c and 2cp-1-c of 2cp
    TOKEN_INTERLEAVED = "token_interleaved"    # rollout prefill-CP pages


class MergeOrder(str, enum.Enum):
    ASCENDING_GLOBAL_BLOCK = "ascending_global_block"


def _strictly_increasing(values: tuple) -> bool:
    return all(a < b for a, b in zip(values, values[1:]))


def _range_ok(start, end, upper=None) -> bool:
    return is_plain_int(start) and is_plain_int(end) and 0 <= start < end and (upper is None or end <= upper)


# ------------------------------------------------------------------------------------ sharding
@dataclass(frozen=True)
class ShardingSpec:
    """Logical TP / CP / SP ownership of the calling rank.

    TP head shards are equal and contiguous.  CP sequence ownership may be uneven, but every local
    block carries its global block index and global first token, so partial states can be merged by
    logical order, never by arrival order."""
    tp_rank: int
    tp_world_size: int
    cp_rank: int
    cp_world_size: int
    global_q_heads: int
    global_kv_heads: int
    local_q_head_start: int
    local_q_heads: int
    local_kv_head_start: int
    local_kv_heads: int
    global_sequence_length: int
    local_sequence_length: int
    global_block_indices: tuple[int, ...]
    global_block_token_starts: tuple[int, ...]
    local_block_offsets: tuple[int, ...]
    packed_sequence_offsets: tuple[int, ...] | None = None
    sp_rank: int = 0
    sp_world_size: int = 1

    def __post_init__(self) -> None:
        tp = _positive_int(self.tp_world_size, "tp_world_size")
        for rank_name, world_name in (("tp_rank", "tp_world_size"), ("cp_rank", "cp_world_size"), ("sp_rank", "sp_world_size")):
            world = _positive_int(getattr(self, world_name), world_name)
            if _non_negative_int(getattr(self, rank_name), rank_name) >= world:
                raise AttentionContractError(f"{rank_name}={getattr(self, rank_name)} must be smaller than {world_name}={world}")
        hq = _positive_int(self.global_q_heads, "global_q_heads")
        hkv = _positive_int(self.global_kv_heads, "global_kv_heads")
        if hq % hkv:
            raise AttentionContractError(f"global_q_heads={hq} must be divisible by global_kv_heads={hkv} for GQA")
        if hq % tp or hkv % tp:
            raise AttentionContractError("global Q/KV heads must be evenly divisible by tp_world_size; "
                                         f"got Hq={hq}, Hkv={hkv}, TP={tp}")
        want_heads = (hq // tp, hkv // tp)
        got_heads = (_positive_int(self.local_q_heads, "local_q_heads"), _positive_int(self.local_kv_heads, "local_kv_heads"))
        if got_heads != want_heads:
            raise AttentionContractError("local TP head counts do not preserve the global Q/KV mapping; "
                                         f"expected {want_heads}, got {got_heads}")
        want_starts = (self.tp_rank * want_heads[0], self.tp_rank * want_heads[1])
        got_starts = (_non_negative_int(self.local_q_head_start, "local_q_head_start"),
                      _non_negative_int(self.local_kv_head_start, "local_kv_head_start"))
        if got_starts != want_starts:
            raise AttentionContractError("local TP head starts do not match contiguous rank ownership; "
                                         f"expected {want_starts}, got {got_starts}")
        total = _positive_int(self.global_sequence_length, "global_sequence_length")
        local = _positive_int(self.local_sequence_length, "local_sequence_length")
        blocks = _integer_tuple(self.global_block_indices, "global_block_indices")
        if not blocks:
            raise AttentionContractError("global_block_indices must not be empty")
        if any(b < 0 for b in blocks):
            raise AttentionContractError("global_block_indices must be non-negative")
        if not _strictly_increasing(blocks):
            raise AttentionContractError("global_block_indices must be unique and strictly increasing")
        starts = _integer_tuple(self.global_block_token_starts, "global_block_token_starts")
        offsets = _integer_tuple(self.local_block_offsets, "local_block_offsets")
        if len(starts) != len(blocks):
            raise AttentionContractError("global_block_token_starts must contain one entry per global_block_indices entry")
        if any(s < 0 for s in starts):
            raise AttentionContractError("global_block_token_starts must be non-negative")
        if len(offsets) != len(blocks) + 1:
            raise AttentionContractError("local_block_offsets must contain one boundary more than global_block_indices")
        if offsets[0] != 0 or offsets[-1] != local:
            raise AttentionContractError("local_block_offsets must start at 0 and end at local_sequence_length")
        if not _strictly_increasing(offsets):
            raise AttentionContractError("local_block_offsets must be strictly increasing")
        prev_end = 0
        for i, (g0, l0, l1) in enumerate(zip(starts, offsets[:-1], offsets[1:])):
            g1 = g0 + (l1 - l0)
            if g1 > total:
                raise AttentionContractError(f"global block {blocks[i]} exceeds global_sequence_length")
            if i > 0 and g0 < prev_end:
                raise AttentionContractError("global block token ranges must be non-overlapping and ordered")
            prev_end = g1
        object.__setattr__(self, "global_block_indices", blocks)
        object.__setattr__(self, "global_block_token_starts", starts)
        object.__setattr__(self, "local_block_offsets", offsets)
        if self.packed_sequence_offsets is not None:
            packed = _integer_tuple(self.packed_sequence_offsets, "packed_sequence_offsets")
            if len(packed) < 2 or packed[0] != 0:
                raise AttentionContractError("packed_sequence_offsets must start at 0 and contain an end offset")
            if not _strictly_increasing(packed):
                raise AttentionContractError("packed_sequence_offsets must be strictly increasing")
            if packed[-1] != local:
                raise AttentionContractError("the final packed_sequence_offsets value must equal local_sequence_length; "
                                             f"got {packed[-1]} and {local}")
            object.__setattr__(self, "packed_sequence_offsets", packed)

    # shorthand used by registry checks and bindings
    @property
    def tp_size(self) -> int:
        return self.tp_world_size

    @property
    def cp_size(self) -> int:
        return self.cp_world_size

    @classmethod
    def for_layout(cls, *, num_q_heads: int, num_kv_heads: int, seq_len: int, tp_rank: int = 0, tp_world_size: int = 1,
                   cp_rank: int = 0, cp_world_size: int = 1, layout: CPLayout | str = CPLayout.NONE,
                   block: int = CANONICAL_KV_BLOCK, packed_sequence_offsets=None) -> "ShardingSpec":
        """Block tables of one rank for a sequence of ``seq_len`` tokens cut into ``block``-token blocks and
        distributed by ``layout`` (chunks of the layouts are whole numbers of blocks)."""
        layout = CPLayout(layout)
        if (cp_world_size == 1) != (layout is CPLayout.NONE):
            raise AttentionContractError("cp layout must be NONE exactly when cp_world_size == 1")
        if layout is CPLayout.TOKEN_INTERLEAVED:
            raise AttentionContractError("token-interleaved ownership is a paged-cache layout; describe it with KVCacheSpec")
        nchunk = {CPLayout.NONE: 1, CPLayout.CONTIGUOUS: cp_world_size, CPLayout.ZIGZAG: 2 * cp_world_size}[layout]
        if seq_len % nchunk:
            raise AttentionContractError(f"sequence length {seq_len} must divide into {nchunk} chunks for layout {layout.value}")
        chunk = seq_len // nchunk
        mine = {CPLayout.NONE: [0], CPLayout.CONTIGUOUS: [cp_rank],
                CPLayout.ZIGZAG: [cp_rank, 2 * cp_world_size - 1 - cp_rank]}[layout]
        idx, starts, offs = [], [], [0]
        for c in sorted(mine):
            t = c * chunk
            while t < (c + 1) * chunk:
                n = min(block - t % block, (c + 1) * chunk - t)
                idx.append(t // block)
                starts.append(t)
                offs.append(offs[-1] + n)
                t += n
        # two pieces of one global block (a chunk boundary inside a block) get distinct, ordered indices
        dedup = []
        for i, b in enumerate(idx):
            dedup.append(b if not dedup or b > dedup[-1] else dedup[-1] + 1)
        hq_l, hkv_l = num_q_heads // max(tp_world_size, 1), num_kv_heads // max(tp_world_size, 1)
        return cls(tp_rank, tp_world_size, cp_rank, cp_world_size, num_q_heads, num_kv_heads, tp_rank * hq_l, hq_l,
                   tp_rank * hkv_l, hkv_l, seq_len, offs[-1], tuple(dedup), tuple(starts), tuple(offs),
                   packed_sequence_offsets)


@dataclass(frozen=True)
class ReductionSpec:
    """Deterministic CP ``(out, lse)`` merge semantics."""
    merge: AttentionMerge = AttentionMerge.ONLINE_SOFTMAX_LSE
    acc_dtype: AttentionDType = AttentionDType.FP32
    order: ReductionOrder = ReductionOrder.GLOBAL_BLOCK_INDEX
    downcast_at: DowncastPoint = DowncastPoint.FINAL_WRITE
    engine: ReductionEngine = ReductionEngine.IN_OP_REFERENCE
    kv_block: int = CANONICAL_KV_BLOCK

    def __post_init__(self) -> None:
        _coerce(self, merge=AttentionMerge, acc_dtype=AttentionDType, order=ReductionOrder, downcast_at=DowncastPoint,
                engine=ReductionEngine)
        if self.acc_dtype is not AttentionDType.FP32:
            raise AttentionContractError(f"CP attention accumulation must be fp32; got {self.acc_dtype.value}")
        _positive_int(self.kv_block, "kv_block")


# ------------------------------------------------------------------------------------ split-KV
@dataclass(frozen=True)
class SplitKVExecutionPlan:
    """The key-axis schedule one backend invocation actually ran.  ``boundaries`` are the logical KV
    ranges reduced separately; CP may move the resulting states between ranks but never changes the
    fp32 merge recorded here."""
    requested_mode: SplitKVMode
    requested_split_size: int | None
    actual_mode: SplitKVMode | None
    actual_split_size: int | None
    boundaries: tuple[tuple[int, int], ...]
    merge_order: ReductionOrder = ReductionOrder.GLOBAL_BLOCK_INDEX
    acc_dtype: AttentionDType = AttentionDType.FP32
    downcast_at: DowncastPoint = DowncastPoint.FINAL_WRITE
    backend: str = "reference"
    source: str = "contract_exact"
    fallback: bool = False
    fallback_reason: str | None = None

    def __post_init__(self) -> None:
        _coerce(self, requested_mode=SplitKVMode)
        if self.actual_mode is not None:
            _coerce(self, actual_mode=SplitKVMode)
        for name in ("requested_split_size", "actual_split_size"):
            if getattr(self, name) is not None:
                _positive_int(getattr(self, name), name)
        if self.requested_mode is SplitKVMode.FIXED:
            if self.requested_split_size is None:
                raise AttentionContractError("requested fixed Split-KV mode requires requested_split_size")
        elif self.requested_split_size is not None:
            raise AttentionContractError("requested_split_size is only valid for requested fixed Split-KV mode")
        try:
            bounds = tuple(tuple(b) for b in self.boundaries)
        except TypeError as exc:
            raise AttentionContractError("Split-KV boundaries must be an iterable of (start, end) pairs") from exc
        prev = 0
        for i, b in enumerate(bounds):
            if len(b) != 2:
                raise AttentionContractError(f"Split-KV boundary {i} must contain exactly start and end")
            if not _range_ok(*b):
                raise AttentionContractError("Split-KV boundaries must satisfy 0 <= start < end")
            if i > 0 and b[0] != prev:
                raise AttentionContractError("Split-KV boundaries must be contiguous and in logical KV order")
            prev = b[1]
        if self.actual_mode is None and bounds:
            raise AttentionContractError("unknown actual Split-KV plan cannot declare boundaries")
        if self.actual_mode is not None and not bounds:
            raise AttentionContractError("actual Split-KV plan must declare logical boundaries")
        if self.actual_mode is SplitKVMode.FIXED:
            if self.actual_split_size is None:
                raise AttentionContractError("actual fixed Split-KV mode requires actual_split_size")
            widths = [e - s for s, e in bounds]
            if any(w != self.actual_split_size for w in widths[:-1]) or (widths and widths[-1] > self.actual_split_size):
                raise AttentionContractError("fixed Split-KV boundaries must use actual_split_size except for a shorter "
                                             "final split")
        elif self.actual_split_size is not None:
            raise AttentionContractError("actual_split_size is only valid for actual fixed Split-KV mode")
        if self.actual_mode is SplitKVMode.DISABLED and len(bounds) != 1:
            raise AttentionContractError("disabled Split-KV execution must contain exactly one boundary")
        object.__setattr__(self, "boundaries", bounds)
        _coerce(self, merge_order=ReductionOrder, acc_dtype=AttentionDType, downcast_at=DowncastPoint)
        if self.acc_dtype is not AttentionDType.FP32:
            raise AttentionContractError("Split-KV partial states must be merged in fp32")
        for name in ("backend", "source"):
            if not isinstance(getattr(self, name), str) or not getattr(self, name).strip():
                raise AttentionContractError(f"Split-KV {name} must be a non-empty string")
        if not isinstance(self.fallback, bool):
            raise AttentionContractError("Split-KV fallback must be a bool")
        if self.fallback and not self.fallback_reason:
            raise AttentionContractError("Split-KV fallback_reason is required for a fallback")
        if not self.fallback and self.fallback_reason is not None:
            raise AttentionContractError("Split-KV fallback_reason must be None when fallback=False")
        if not self.fallback and self.actual_mode is not None:
            if self.actual_mode is not self.requested_mode:
                raise AttentionContractError("actual Split-KV mode may differ from requested mode only for a fallback")
            if self.actual_split_size != self.requested_split_size:
                raise AttentionContractError("actual Split-KV size may differ from requested size only for a fallback")

    @property
    def actual_split_count(self) -> int | None:
        return None if self.actual_mode is None else len(self.boundaries)

    def to_dict(self) -> dict[str, Any]:
        return {"requested_split_kv_policy": self.requested_mode.value, "requested_split_kv_size": self.requested_split_size,
                "actual_split_kv_policy": None if self.actual_mode is None else self.actual_mode.value,
                "actual_split_kv_size": self.actual_split_size, "actual_split_kv_count": self.actual_split_count,
                "actual_split_boundaries": [list(b) for b in self.boundaries],
                "split_kv_merge_order": self.merge_order.value, "split_kv_accum_dtype": self.acc_dtype.value,
                "split_kv_downcast_at": self.downcast_at.value, "split_kv_backend": self.backend,
                "split_kv_plan_source": self.source, "split_kv_fallback": self.fallback,
                "split_kv_fallback_reason": self.fallback_reason}


@dataclass(frozen=True)
class SplitKVSpec:
    """Requested key-axis split policy shared by training and rollout."""
    mode: SplitKVMode = SplitKVMode.DISABLED
    fixed_split_size: int | None = None
    strict_consistency: bool = True

    @classmethod
    def disabled(cls, *, strict_consistency: bool = True) -> "SplitKVSpec":
        return cls(SplitKVMode.DISABLED, None, strict_consistency)

    @classmethod
    def fixed(cls, split_size: int, *, strict_consistency: bool = True) -> "SplitKVSpec":
        return cls(SplitKVMode.FIXED, split_size, strict_consistency)

    @classmethod
    def auto(cls, *, strict_consistency: bool = False) -> "SplitKVSpec":
        return cls(SplitKVMode.AUTO, None, strict_consistency)

    def __post_init__(self) -> None:
        object.__setattr__(self, "mode", _enum_value(SplitKVMode, self.mode, "split_kv.mode"))
        if not isinstance(self.strict_consistency, bool):
            raise AttentionContractError("split_kv.strict_consistency must be a bool")
        if self.mode is SplitKVMode.FIXED:
            if self.fixed_split_size is None:
                raise AttentionContractError("fixed Split-KV policy requires fixed_split_size")
            _positive_int(self.fixed_split_size, "split_kv.fixed_split_size")
        elif self.fixed_split_size is not None:
            raise AttentionContractError("fixed_split_size is only valid for fixed Split-KV policy")
        if self.strict_consistency and self.mode is SplitKVMode.AUTO:
            raise AttentionContractError("auto Split-KV is runtime-shape dependent and is not allowed in strict consistency")

    def resolve(self, total_kv_tokens: int, *, backend: str) -> SplitKVExecutionPlan:
        """The plan of a policy whose schedule is fully known from the contract (AUTO is not)."""
        total = _positive_int(total_kv_tokens, "total_kv_tokens")
        if self.mode is SplitKVMode.AUTO:
            return SplitKVExecutionPlan(self.mode, None, None, None, (), backend=backend, source="runtime_required")
        size = total if self.mode is SplitKVMode.DISABLED else self.fixed_split_size
        bounds = tuple((s, min(s + size, total)) for s in range(0, total, size))
        return SplitKVExecutionPlan(self.mode, self.fixed_split_size, self.mode, self.fixed_split_size, bounds,
                                    backend=backend, source="contract_exact")

    def to_dict(self) -> dict[str, Any]:
        return {"mode": self.mode.value, "fixed_split_size": self.fixed_split_size,
                "strict_consistency": self.strict_consistency}


_PLAN_ALIGNMENT_FIELDS = ("requested_mode", "requested_split_size", "actual_mode", "actual_split_size", "boundaries",
                          "merge_order", "acc_dtype", "downcast_at", "fallback")


def validate_split_kv_alignment(training: SplitKVExecutionPlan, rollout: SplitKVExecutionPlan) -> None:
    """Fail closed unless training and rollout executed the same logical plan."""
    if training.actual_mode is None or rollout.actual_mode is None:
        raise AttentionContractError("strict Split-KV alignment requires actual runtime plans from both sides")
    bad = [f for f in _PLAN_ALIGNMENT_FIELDS if getattr(training, f) != getattr(rollout, f)]
    if bad:
        raise AttentionContractError("training/rollout Split-KV execution plans differ: " + ", ".join(bad))


# What a bitwise comparison across configurations requires.  TP degree and batch size are absent on
# purpose: a head shard's result here depends on neither (one fixed per-row program), so requiring
# them to match would reject comparisons that are in fact bit-equal.
CROSS_CONFIG_BOUND_FIELDS = ("dtype", "head_dim", "causal", "export_lse")


def validate_cross_config_alignment(training: "AttentionContract", rollout: "AttentionContract") -> None:
    """Fail closed unless both sides describe one comparable invocation; names the field that diverged."""
    if not isinstance(training, AttentionContract) or not isinstance(rollout, AttentionContract):
        raise AttentionContractError("both sides must be AttentionContract instances")
    bad = [n for n in ("global_q_heads", "global_kv_heads") if getattr(training.sharding, n) != getattr(rollout.sharding, n)]
    if bad:
        raise AttentionContractError("training and rollout describe different global head layouts: " + ", ".join(bad))
    bad = [n for n in CROSS_CONFIG_BOUND_FIELDS if getattr(training, n) != getattr(rollout, n)]
    if bad:
        raise AttentionContractError("training and rollout attention contracts differ: " + ", ".join(bad))
    if training.split_kv != rollout.split_kv:
        raise AttentionContractError("training and rollout Split-KV policies differ")
    if training.reduction != rollout.reduction:
        raise AttentionContractError("training and rollout reduction specs differ")


@dataclass(frozen=True, order=True)
class SplitKVRuntimeCoordinate:
    """Identity of one (batch item, TP rank, CP consumer, CP owner) runtime plan."""
    batch_index: int
    tp_rank: int
    cp_rank: int
    owner_cp_rank: int

    def validate(self, *, batch_size: int, tp_world_size: int, cp_world_size: int) -> None:
        for name, limit, what in (("batch_index", batch_size, "batch_size"), ("tp_rank", tp_world_size, "tp_world_size"),
                                  ("cp_rank", cp_world_size, "cp_world_size"),
                                  ("owner_cp_rank", cp_world_size, "cp_world_size")):
            if _non_negative_int(getattr(self, name), name) >= limit:
                raise AttentionContractError(f"Split-KV {name} is outside {what}")

    def to_dict(self) -> dict[str, int]:
        return {"batch_index": self.batch_index, "tp_rank": self.tp_rank, "cp_rank": self.cp_rank,
                "owner_cp_rank": self.owner_cp_rank}


@dataclass(frozen=True)
class SplitKVRuntimePlanEntry:
    """The actual plan of one consumer for one owner's KV range."""
    coordinate: SplitKVRuntimeCoordinate
    expected_kv_range: tuple[int, int]
    execution: SplitKVExecutionPlan

    def validate(self, *, batch_size: int, tp_world_size: int, cp_world_size: int, total_kv_tokens: int) -> None:
        self.coordinate.validate(batch_size=batch_size, tp_world_size=tp_world_size, cp_world_size=cp_world_size)
        try:
            start, end = self.expected_kv_range
        except (TypeError, ValueError) as exc:
            raise AttentionContractError("expected_kv_range must contain exactly (start, end)") from exc
        if not _range_ok(start, end, total_kv_tokens):
            raise AttentionContractError("expected_kv_range must satisfy 0 <= start < end <= total_kv_tokens")
        if self.execution.actual_mode is None:
            raise AttentionContractError("complete Split-KV plan sets require actual runtime plans")
        b = self.execution.boundaries
        if b[0][0] != start or b[-1][1] != end:
            raise AttentionContractError("Split-KV execution boundaries must exactly cover expected_kv_range")

    def to_dict(self) -> dict[str, Any]:
        return {**self.coordinate.to_dict(), "expected_kv_range": list(self.expected_kv_range), **self.execution.to_dict()}


def _format_split_kv_coordinates(coordinates: Iterable[SplitKVRuntimeCoordinate]) -> list[dict[str, int]]:
    return [c.to_dict() for c in sorted(coordinates)]


@dataclass(frozen=True)
class SplitKVRuntimePlanSet:
    """All actual plans over batch x TP x CP consumer x CP owner.  Every consumer reports the plan it
    used for every owner's range; the duplication is what exposes a rank that silently chose another
    schedule or merge policy."""
    batch_size: int
    tp_world_size: int
    cp_world_size: int
    total_kv_tokens: tuple[int, ...]
    entries: tuple[SplitKVRuntimePlanEntry, ...]

    def __post_init__(self) -> None:
        B = _positive_int(self.batch_size, "batch_size")
        tp = _positive_int(self.tp_world_size, "tp_world_size")
        cp = _positive_int(self.cp_world_size, "cp_world_size")
        totals = _integer_tuple(self.total_kv_tokens, "total_kv_tokens")
        if len(totals) != B or any(t <= 0 for t in totals):
            raise AttentionContractError("total_kv_tokens must contain one positive length per batch item")
        entries = tuple(self.entries)
        object.__setattr__(self, "total_kv_tokens", totals)
        object.__setattr__(self, "entries", entries)
        want = {SplitKVRuntimeCoordinate(b, t, c, o) for b in range(B) for t in range(tp) for c in range(cp) for o in range(cp)}
        got = [e.coordinate for e in entries]
        if len(set(got)) != len(got):
            raise AttentionContractError("Split-KV runtime plan set contains duplicate coordinates")
        missing, extra = want.difference(got), set(got).difference(want)
        if missing or extra:
            raise AttentionContractError("Split-KV runtime plan set coordinate coverage is incomplete; "
                                         f"missing={_format_split_kv_coordinates(missing)}, "
                                         f"extra={_format_split_kv_coordinates(extra)}")
        for e in entries:
            e.validate(batch_size=B, tp_world_size=tp, cp_world_size=cp, total_kv_tokens=totals[e.coordinate.batch_index])
        by = {e.coordinate: e for e in entries}
        for b, total in enumerate(totals):                           # owners tile [0, total) in owner order
            for t in range(tp):
                prev = 0
                for o in range(cp):
                    s, e = by[SplitKVRuntimeCoordinate(b, t, 0, o)].expected_kv_range
                    if s != prev:
                        raise AttentionContractError("Split-KV owner ranges must be gap-free in CP owner order")
                    prev = e
                if prev != total:
                    raise AttentionContractError("Split-KV owner ranges do not cover total_kv_tokens")
        for b in range(B):                                           # every consumer saw the same plan per owner
            for o in range(cp):
                group = [by[SplitKVRuntimeCoordinate(b, t, c, o)] for t in range(tp) for c in range(cp)]
                for e in group[1:]:
                    if e.expected_kv_range != group[0].expected_kv_range:
                        raise AttentionContractError("Split-KV owner range differs across TP/CP consumers")
                    try:
                        validate_split_kv_alignment(group[0].execution, e.execution)
                    except AttentionContractError as exc:
                        raise AttentionContractError("Split-KV plan differs across TP/CP consumers for "
                                                     f"batch={b}, owner_cp={o}: {exc}") from exc

    def to_dict(self) -> dict[str, Any]:
        return {"batch_size": self.batch_size, "tp_world_size": self.tp_world_size, "cp_world_size": self.cp_world_size,
                "total_kv_tokens": list(self.total_kv_tokens),
                "entries": [e.to_dict() for e in sorted(self.entries, key=lambda e: e.coordinate)],
                "coverage": "complete_batch_tp_cp_owner_cartesian_product"}


def validate_split_kv_plan_set_alignment(training: SplitKVRuntimePlanSet, rollout: SplitKVRuntimePlanSet) -> None:
    """Fail closed unless the complete training and rollout plan sets align."""
    bad = [f for f in ("batch_size", "tp_world_size", "cp_world_size", "total_kv_tokens")
           if getattr(training, f) != getattr(rollout, f)]
    if bad:
        raise AttentionContractError("training/rollout Split-KV plan-set topology differs: " + ", ".join(bad))
    tr = {e.coordinate: e for e in training.entries}
    ro = {e.coordinate: e for e in rollout.entries}
    if tr.keys() != ro.keys():
        raise AttentionContractError("training/rollout Split-KV plan-set coordinates differ")
    for c in sorted(tr):
        if tr[c].expected_kv_range != ro[c].expected_kv_range:
            raise AttentionContractError(f"training/rollout expected KV range differs at {c}")
        try:
            validate_split_kv_alignment(tr[c].execution, ro[c].execution)
        except AttentionContractError as exc:
            raise AttentionContractError(f"training/rollout Split-KV plan differs at {c}: {exc}") from exc


def build_split_kv_runtime_plan_set(total_kv_tokens: Iterable[int], *, tp_world_size: int, cp_world_size: int,
                                    split_kv: SplitKVSpec, backend: str = "contract_reference") -> SplitKVRuntimePlanSet:
    """The complete owner-local plan set a contract implies (owners get near-equal contiguous ranges)."""
    totals = _integer_tuple(total_kv_tokens, "total_kv_tokens")
    tp = _positive_int(tp_world_size, "tp_world_size")
    cp = _positive_int(cp_world_size, "cp_world_size")
    if not totals or any(t < cp for t in totals):
        raise AttentionContractError("contract plan sets require at least one KV token per CP owner")
    if not isinstance(split_kv, SplitKVSpec):
        raise AttentionContractError("split_kv must be a SplitKVSpec")
    entries: list[SplitKVRuntimePlanEntry] = []
    for b, total in enumerate(totals):
        base, rem = divmod(total, cp)
        owners, s = [], 0
        for o in range(cp):
            e = s + base + (1 if o < rem else 0)
            owners.append((s, e))
            s = e
        for t in range(tp):
            for c in range(cp):
                for o, (o0, o1) in enumerate(owners):
                    loc = split_kv.resolve(o1 - o0, backend=backend)
                    plan = SplitKVExecutionPlan(loc.requested_mode, loc.requested_split_size, loc.actual_mode,
                                                loc.actual_split_size, tuple((o0 + x, o0 + y) for x, y in loc.boundaries),
                                                loc.merge_order, loc.acc_dtype, loc.downcast_at, loc.backend, loc.source,
                                                loc.fallback, loc.fallback_reason)
                    entries.append(SplitKVRuntimePlanEntry(SplitKVRuntimeCoordinate(b, t, c, o), (o0, o1), plan))
    return SplitKVRuntimePlanSet(len(totals), tp, cp, totals, tuple(entries))


# ------------------------------------------------------------------------------------ KV cache / RoPE / projections
@dataclass(frozen=True)
class KVCacheSpec:
    """Logical identity of the paged KV cache a replay reads: per sequence its length, the global
    position of every cached token, its page row, and which leading pages are a shared read-only prefix."""
    cache_positions: tuple[int, ...]
    kv_seq_lens: tuple[int, ...]
    block_table: tuple[tuple[int, ...], ...]
    global_token_positions: tuple[int, ...]
    page_size: int
    prefix_cache_enabled: bool = False
    prefix_cache_key: str | None = None
    shared_prefix_page_count: int = 0

    def __post_init__(self) -> None:
        pos = _integer_tuple(self.cache_positions, "cache_positions")
        lens = _integer_tuple(self.kv_seq_lens, "kv_seq_lens")
        page = _positive_int(self.page_size, "page_size")
        gpos = _integer_tuple(self.global_token_positions, "global_token_positions")
        if not pos or any(p < 0 for p in pos):
            raise AttentionContractError("cache_positions must contain non-negative positions")
        if not lens or any(n <= 0 for n in lens):
            raise AttentionContractError("kv_seq_lens must contain positive sequence lengths")
        if len(pos) != len(lens):
            raise AttentionContractError("cache_positions must contain one entry per kv_seq_lens entry")
        if not gpos or any(p < 0 for p in gpos):
            raise AttentionContractError("global_token_positions must contain non-negative positions")
        if len(gpos) != sum(lens):
            raise AttentionContractError("global_token_positions must describe every logical cached token; "
                                         f"expected {sum(lens)}, got {len(gpos)}")
        rows, off = [], 0
        for i, n in enumerate(lens):
            row = gpos[off:off + n]
            if not _strictly_increasing(row):
                raise AttentionContractError("global_token_positions must be strictly increasing within each sequence; "
                                             f"sequence {i} is invalid")
            if pos[i] != row[-1]:
                raise AttentionContractError("cache_positions must equal the terminal global token position for each "
                                             f"sequence; sequence {i} expected {row[-1]}, got {pos[i]}")
            rows.append(row)
            off += n
        try:
            table = tuple(tuple(r) for r in self.block_table)
        except TypeError as exc:
            raise AttentionContractError("block_table must be a two-dimensional integer table") from exc
        if len(table) != len(lens) or any(not r for r in table):
            raise AttentionContractError("block_table must contain one non-empty row per kv_seq_lens entry")
        active: list[tuple[int, ...]] = []
        for i, (row, n) in enumerate(zip(table, lens)):
            live, padded = [], False
            for j, blk in enumerate(row):
                if not is_plain_int(blk) or blk < -1:
                    raise AttentionContractError("block_table entries must be integer block ids or -1 padding; "
                                                 f"got block_table[{i}][{j}]={blk!r}")
                if blk == -1:
                    padded = True
                elif padded:
                    raise AttentionContractError(f"block_table -1 padding must be trailing; row {i} contains an active block "
                                                 "after padding")
                else:
                    live.append(blk)
            want = (n + page - 1) // page
            if len(live) != want:
                raise AttentionContractError("block_table active page count must match kv_seq_lens and page_size; "
                                             f"row {i} expected {want}, got {len(live)}")
            if len(set(live)) != len(live):
                raise AttentionContractError(f"block_table row {i} contains duplicate active page ids")
            active.append(tuple(live))
        if not isinstance(self.prefix_cache_enabled, bool):
            raise AttentionContractError("prefix_cache_enabled must be a bool")
        shared = _non_negative_int(self.shared_prefix_page_count, "shared_prefix_page_count")
        if self.prefix_cache_enabled and not self.prefix_cache_key:
            raise AttentionContractError("prefix_cache_key is required when prefix_cache_enabled=True")
        if not self.prefix_cache_enabled and self.prefix_cache_key is not None:
            raise AttentionContractError("prefix_cache_key must be None when prefix_cache_enabled=False")
        if not self.prefix_cache_enabled and shared:
            raise AttentionContractError("shared_prefix_page_count must be 0 when prefix_cache_enabled=False")
        shared_pages: tuple[int, ...] = ()
        if shared:
            if any(len(r) < shared for r in active):
                raise AttentionContractError("shared_prefix_page_count exceeds an active block-table row")
            ntok = shared * page
            if any(n < ntok for n in lens):
                raise AttentionContractError("shared prefix pages must be fully populated and read-only")
            shared_pages = active[0][:shared]
            for i in range(1, len(active)):
                if active[i][:shared] != shared_pages:
                    raise AttentionContractError(f"shared prefix page ids must match across every sequence; sequence {i} is "
                                                 "inconsistent")
                if rows[i][:ntok] != rows[0][:ntok]:
                    raise AttentionContractError("shared prefix token positions must match across every sequence; "
                                                 f"sequence {i} is inconsistent")
        owner: dict[int, int] = {}
        for i, r in enumerate(active):
            for pg in r[shared:]:
                if pg in shared_pages:
                    raise AttentionContractError("a writable suffix page cannot alias a read-only shared prefix page")
                if pg in owner:
                    raise AttentionContractError("active pages may be shared across sequences only when declared as read-only "
                                                 f"prefix pages; page {pg} is used by sequences {owner[pg]} and {i}")
                owner[pg] = i
        for name, value in (("cache_positions", pos), ("kv_seq_lens", lens), ("block_table", table),
                            ("global_token_positions", gpos)):
            object.__setattr__(self, name, value)

    @classmethod
    def contiguous(cls, kv_seq_lens, page_size: int = CANONICAL_KV_BLOCK, shared_prefix_tokens: int = 0,
                   prefix_cache_key: str | None = None) -> "KVCacheSpec":
        """Sequences at positions 0..n-1 with fresh pages; the first ``shared_prefix_tokens`` (a whole number
        of pages) of every sequence live in the same pages."""
        lens = tuple(int(n) for n in kv_seq_lens)
        if shared_prefix_tokens % page_size:
            raise AttentionContractError("a shared prefix must be a whole number of pages")
        shared = shared_prefix_tokens // page_size
        table, nxt = [], shared
        for n in lens:
            need = (n + page_size - 1) // page_size
            table.append(tuple(range(shared)) + tuple(range(nxt, nxt + need - shared)))
            nxt += need - shared
        width = max(len(r) for r in table)
        table = [r + (-1,) * (width - len(r)) for r in table]
        gpos = tuple(p for n in lens for p in range(n))
        return cls(tuple(n - 1 for n in lens), lens, tuple(table), gpos, page_size, bool(shared),
                   (prefix_cache_key or "shared-prefix") if shared else None, shared)


@dataclass(frozen=True)
class RoPESpec:
    """RoPE identity of the attention inputs and of the cached keys: pre- or post-rotation, the angle
    base, where the cast happens and whether rotation is fused into the attention boundary."""
    q_state: RoPEState = RoPEState.POST_ROPE
    k_state: RoPEState = RoPEState.POST_ROPE
    k_cache_state: RoPEState = RoPEState.POST_ROPE
    theta: float = 1.0e6
    rotary_dim: int = 128
    rope_scaling: str | None = None
    position_ids: tuple[int, ...] | None = None
    query_position_offsets: tuple[int, ...] | None = None
    key_position_offsets: tuple[int, ...] | None = None
    cast_at: RoPECastPoint = RoPECastPoint.AFTER_ROPE
    output_dtype: AttentionDType = AttentionDType.BF16
    fusion_boundary: RoPEFusionBoundary = RoPEFusionBoundary.UNFUSED_ROPE_ATTENTION

    def __post_init__(self) -> None:
        _coerce(self, q_state=RoPEState, k_state=RoPEState, k_cache_state=RoPEState)
        if isinstance(self.theta, bool) or not isinstance(self.theta, (float, int)) or float(self.theta) <= 0.0:
            raise AttentionContractError(f"theta must be a positive number; got {self.theta!r}")
        object.__setattr__(self, "theta", float(self.theta))
        _positive_int(self.rotary_dim, "rotary_dim")
        if self.rope_scaling is not None and (not isinstance(self.rope_scaling, str) or not self.rope_scaling.strip()):
            raise AttentionContractError("rope_scaling must be a non-empty string when provided")
        for name in ("position_ids", "query_position_offsets", "key_position_offsets"):
            v = getattr(self, name)
            if v is None:
                continue
            v = _integer_tuple(v, name)
            if not v or any(x < 0 for x in v):
                raise AttentionContractError(f"{name} must contain non-negative positions")
            object.__setattr__(self, name, v)
        _coerce(self, cast_at=RoPECastPoint, output_dtype=AttentionDType, fusion_boundary=RoPEFusionBoundary)


@dataclass(frozen=True)
class AttentionProjectionSpec:
    """How the QKV or output projection executes: bf16 in and out, fp32 accumulation over K in ascending
    order without a K split, and which collective follows it under TP and SP."""
    name: str
    input_dtype: AttentionDType = AttentionDType.BF16
    output_dtype: AttentionDType = AttentionDType.BF16
    acc_dtype: AttentionDType = AttentionDType.FP32
    split_kv: SplitKVMode = SplitKVMode.DISABLED
    k_order: str = "ascending"
    backend_policy: str = "native_verified_then_common_deterministic"
    deterministic_backend: str = "rlkernel.b200.det_gemm"
    tp_forward_collective: ProjectionCollective = ProjectionCollective.NONE
    tp_backward_dgrad_collective: ProjectionCollective = ProjectionCollective.NONE
    sp_forward_collective: ProjectionCollective = ProjectionCollective.NONE
    sp_backward_collective: ProjectionCollective = ProjectionCollective.NONE
    qkv_split_order: tuple[str, ...] = ()
    require_runtime_readback: bool = True
    canonical_k_chunks: int = 8            # row-parallel projections sum 8 canonical K chunks in a fixed tree

    @classmethod
    def qkv(cls) -> "AttentionProjectionSpec":
        return cls("qkv", tp_backward_dgrad_collective=ProjectionCollective.ALL_REDUCE,
                   sp_forward_collective=ProjectionCollective.ALL_GATHER,
                   sp_backward_collective=ProjectionCollective.REDUCE_SCATTER, qkv_split_order=("q", "k", "v"))

    @classmethod
    def output(cls) -> "AttentionProjectionSpec":
        return cls("o_proj", tp_forward_collective=ProjectionCollective.ALL_REDUCE,
                   sp_forward_collective=ProjectionCollective.REDUCE_SCATTER,
                   sp_backward_collective=ProjectionCollective.ALL_GATHER)

    def __post_init__(self) -> None:
        if self.name not in {"qkv", "o_proj"}:
            raise AttentionContractError("projection name must be qkv or o_proj")
        _coerce(self, input_dtype=AttentionDType, output_dtype=AttentionDType, acc_dtype=AttentionDType)
        object.__setattr__(self, "split_kv", _enum_value(SplitKVMode, self.split_kv, "projection.split_kv"))
        _coerce(self, tp_forward_collective=ProjectionCollective, tp_backward_dgrad_collective=ProjectionCollective,
                sp_forward_collective=ProjectionCollective, sp_backward_collective=ProjectionCollective)
        if self.input_dtype is not AttentionDType.BF16:
            raise AttentionContractError("Attention projections require BF16 input")
        if self.output_dtype is not AttentionDType.BF16:
            raise AttentionContractError("Attention projections require BF16 output")
        if self.acc_dtype is not AttentionDType.FP32:
            raise AttentionContractError("Attention projections require FP32 accumulation")
        if self.split_kv is not SplitKVMode.DISABLED:
            raise AttentionContractError("Attention projection GEMMs must disable Split-K")
        if self.k_order != "ascending":
            raise AttentionContractError("Attention projection GEMMs require ascending K order")
        for name in ("backend_policy", "deterministic_backend"):
            if not isinstance(getattr(self, name), str) or not getattr(self, name).strip():
                raise AttentionContractError(f"{name} must be a non-empty string")
        if not isinstance(self.require_runtime_readback, bool) or not self.require_runtime_readback:
            raise AttentionContractError("projection runtime readback must be required")
        order = tuple(self.qkv_split_order)
        if self.name == "qkv":
            if order != ("q", "k", "v"):
                raise AttentionContractError("QKV projection must split in Q, K, V order")
        elif order:
            raise AttentionContractError("o_proj must not declare a QKV split order")
        object.__setattr__(self, "qkv_split_order", order)
        _positive_int(self.canonical_k_chunks, "canonical_k_chunks")


# ------------------------------------------------------------------------------------ the contract
@dataclass(frozen=True)
class AttentionContract:
    """Complete semantic request consumed by contract-aware dispatch."""
    role: AttentionRole
    mode: AttentionMode
    dtype: AttentionDType
    batch_size: int
    query_sequence_length: int
    head_dim: int
    causal: bool
    causal_offsets: tuple[int, ...] | None
    sharding: ShardingSpec
    reduction: ReductionSpec = field(default_factory=ReductionSpec)
    split_kv: SplitKVSpec = field(default_factory=SplitKVSpec.disabled)
    kv_cache: KVCacheSpec | None = None
    rope: RoPESpec | None = None
    export_lse: bool = True
    qkv_projection: AttentionProjectionSpec = field(default_factory=AttentionProjectionSpec.qkv)
    output_projection: AttentionProjectionSpec = field(default_factory=AttentionProjectionSpec.output)

    def __post_init__(self) -> None:
        _coerce(self, role=AttentionRole, mode=AttentionMode, dtype=AttentionDType)
        B = _positive_int(self.batch_size, "batch_size")
        Sq = _positive_int(self.query_sequence_length, "query_sequence_length")
        _positive_int(self.head_dim, "head_dim")
        for name, kind in (("sharding", ShardingSpec), ("reduction", ReductionSpec), ("split_kv", SplitKVSpec),
                           ("qkv_projection", AttentionProjectionSpec), ("output_projection", AttentionProjectionSpec)):
            if not isinstance(getattr(self, name), kind):
                raise AttentionContractError(f"{name} must be a {kind.__name__}")
        if self.qkv_projection.name != "qkv":
            raise AttentionContractError("qkv_projection must use name='qkv'")
        if self.output_projection.name != "o_proj":
            raise AttentionContractError("output_projection must use name='o_proj'")
        if self.mode is AttentionMode.PREFILL and Sq != self.sharding.local_sequence_length:
            raise AttentionContractError("prefill query_sequence_length must equal sharding.local_sequence_length; "
                                         f"got {Sq} and {self.sharding.local_sequence_length}")
        packed = self.sharding.packed_sequence_offsets
        if packed is not None and len(packed) - 1 != B:
            raise AttentionContractError("packed sequence count must equal logical batch_size; "
                                         f"got {len(packed) - 1} packed sequences and batch_size={B}")
        if not isinstance(self.causal, bool):
            raise AttentionContractError("causal must be a bool")
        if self.causal and self.causal_offsets is None:
            raise AttentionContractError("causal_offsets are required for causal attention")
        if self.causal_offsets is not None:
            offs = _integer_tuple(self.causal_offsets, "causal_offsets")
            if not offs or any(o < 0 for o in offs):
                raise AttentionContractError("causal_offsets must contain non-negative offsets")
            if len(offs) != B:
                raise AttentionContractError("causal_offsets must contain one entry per "
                                             f"{'packed sequence' if packed is not None else 'batch entry'}")
            object.__setattr__(self, "causal_offsets", offs)
        if not isinstance(self.export_lse, bool) or not self.export_lse:
            raise AttentionContractError("export_lse must be True for the attention-domain LSE contract")
        if self.mode is AttentionMode.DECODE and self.kv_cache is None:
            raise AttentionContractError("kv_cache metadata is required for decode attention")
        if self.kv_cache is not None and not isinstance(self.kv_cache, KVCacheSpec):
            raise AttentionContractError("kv_cache must be a KVCacheSpec when provided")
        if self.rope is not None:
            if not isinstance(self.rope, RoPESpec):
                raise AttentionContractError("rope must be a RoPESpec when provided")
            if self.rope.rotary_dim > self.head_dim:
                raise AttentionContractError(f"rotary_dim={self.rope.rotary_dim} must not exceed head_dim={self.head_dim}")
            if self.rope.position_ids is not None and len(self.rope.position_ids) not in {Sq, self.sharding.local_sequence_length}:
                raise AttentionContractError("position_ids must describe the local query sequence or full local sequence length")
            for name in ("query_position_offsets", "key_position_offsets"):
                v = getattr(self.rope, name)
                if v is not None and len(v) != B:
                    raise AttentionContractError(f"{name} must contain one entry per logical batch entry")
        if self.mode is AttentionMode.DECODE and self.kv_cache is not None:
            if len(self.kv_cache.kv_seq_lens) != B:
                raise AttentionContractError("decode kv_seq_lens must contain one entry per batch entry")
            if len(self.kv_cache.cache_positions) != B:
                raise AttentionContractError("decode cache_positions must contain one entry per batch entry")

    def to_dict(self) -> dict[str, Any]:
        """Stable, JSON-compatible provenance of the request."""
        sh = self.sharding
        d: dict[str, Any] = {
            "semantic_operator": "attention", "contract_id": ATTENTION_CONTRACT_ID,
            "role": self.role.value, "mode": self.mode.value, "dtype": self.dtype.value, "batch_size": self.batch_size,
            "query_sequence_length": self.query_sequence_length, "head_dim": self.head_dim, "causal": self.causal,
            "causal_offsets": None if self.causal_offsets is None else list(self.causal_offsets),
            "export_lse": self.export_lse, "lse_domain": "attention",
            "sharding": {
                "tp_rank": sh.tp_rank, "tp_world_size": sh.tp_world_size, "cp_rank": sh.cp_rank,
                "cp_world_size": sh.cp_world_size, "sp_rank": sh.sp_rank, "sp_world_size": sh.sp_world_size,
                "global_q_heads": sh.global_q_heads, "global_kv_heads": sh.global_kv_heads,
                "local_q_head_start": sh.local_q_head_start, "local_q_heads": sh.local_q_heads,
                "local_kv_head_start": sh.local_kv_head_start, "local_kv_heads": sh.local_kv_heads,
                "global_sequence_length": sh.global_sequence_length, "local_sequence_length": sh.local_sequence_length,
                "global_block_indices": list(sh.global_block_indices),
                "global_block_token_starts": list(sh.global_block_token_starts),
                "local_block_offsets": list(sh.local_block_offsets),
                "packed_sequence_offsets": None if sh.packed_sequence_offsets is None else list(sh.packed_sequence_offsets)},
            "reduction": {"merge": self.reduction.merge.value, "acc_dtype": self.reduction.acc_dtype.value,
                          "order": self.reduction.order.value, "downcast_at": self.reduction.downcast_at.value,
                          "engine": self.reduction.engine.value, "kv_block": self.reduction.kv_block},
            "split_kv": self.split_kv.to_dict(),
            "kv_cache": None, "rope": None,
            "qkv_projection": _projection_dict(self.qkv_projection),
            "output_projection": _projection_dict(self.output_projection),
        }
        if self.kv_cache is not None:
            kc = self.kv_cache
            d["kv_cache"] = {"cache_positions": list(kc.cache_positions), "kv_seq_lens": list(kc.kv_seq_lens),
                             "block_table": [list(r) for r in kc.block_table],
                             "global_token_positions_sha256": stable_hash(list(kc.global_token_positions)),
                             "page_size": kc.page_size, "prefix_cache_enabled": kc.prefix_cache_enabled,
                             "prefix_cache_key": kc.prefix_cache_key, "shared_prefix_page_count": kc.shared_prefix_page_count}
        if self.rope is not None:
            r = self.rope
            d["rope"] = {"q_state": r.q_state.value, "k_state": r.k_state.value, "k_cache_state": r.k_cache_state.value,
                         "theta": r.theta, "rotary_dim": r.rotary_dim, "rope_scaling": r.rope_scaling,
                         "position_ids": None if r.position_ids is None else list(r.position_ids),
                         "query_position_offsets": None if r.query_position_offsets is None else list(r.query_position_offsets),
                         "key_position_offsets": None if r.key_position_offsets is None else list(r.key_position_offsets),
                         "cast_at": r.cast_at.value, "output_dtype": r.output_dtype.value,
                         "fusion_boundary": r.fusion_boundary.value}
        return d

    def cross_rank_fingerprint(self) -> str:
        """Rank-independent identity: the rank fields and the local head / sequence / block bounds derived
        from them are left out, so every rank of one logical invocation computes the same value."""
        payload = self.to_dict()
        drop = {"tp_rank", "cp_rank", "sp_rank", "local_q_head_start", "local_q_heads", "local_kv_head_start",
                "local_kv_heads", "local_sequence_length", "global_block_indices", "global_block_token_starts",
                "local_block_offsets"}
        payload["sharding"] = {k: v for k, v in payload["sharding"].items() if k not in drop}
        if self.mode is AttentionMode.PREFILL:
            payload.pop("query_sequence_length")            # equals the rank-local sequence length in prefill
        if payload["rope"] is not None and self.sharding.cp_world_size > 1:
            payload["rope"]["position_ids"] = None           # a rank's own positions
        return stable_hash(payload)

    def preflight(self, group=None) -> None:
        assert_same_across_ranks(self.cross_rank_fingerprint(), group, "attention contract")

    # convenience views used by the bindings and the registry
    @property
    def num_q_heads(self) -> int:
        return self.sharding.global_q_heads

    @property
    def num_kv_heads(self) -> int:
        return self.sharding.global_kv_heads

    @classmethod
    def for_layout(cls, num_q_heads: int, num_kv_heads: int, *, head_dim: int = 128, seq_len: int = 1024, batch_size: int = 1,
                   tp_rank: int = 0, tp_world_size: int = 1, cp_rank: int = 0, cp_world_size: int = 1,
                   layout: CPLayout | str = CPLayout.NONE, role: AttentionRole = AttentionRole.TRAIN,
                   mode: AttentionMode = AttentionMode.PREFILL, dtype: AttentionDType = AttentionDType.BF16,
                   causal: bool = True, rope: RoPESpec | None = None, kv_cache: KVCacheSpec | None = None,
                   engine: ReductionEngine = ReductionEngine.IN_KERNEL) -> "AttentionContract":
        """The common case: ``batch_size`` sequences of ``seq_len`` tokens in one of the CP layouts."""
        sh = ShardingSpec.for_layout(num_q_heads=num_q_heads, num_kv_heads=num_kv_heads, seq_len=seq_len, tp_rank=tp_rank,
                                     tp_world_size=tp_world_size, cp_rank=cp_rank, cp_world_size=cp_world_size, layout=layout)
        sq = sh.local_sequence_length if mode is AttentionMode.PREFILL else 1
        return cls(role, mode, dtype, batch_size, sq, head_dim, causal, (0,) * batch_size if causal else None, sh,
                   ReductionSpec(engine=engine), kv_cache=kv_cache, rope=rope)


def _projection_dict(p: AttentionProjectionSpec) -> dict[str, Any]:
    return {"name": p.name, "input_dtype": p.input_dtype.value, "output_dtype": p.output_dtype.value,
            "acc_dtype": p.acc_dtype.value, "split_kv": p.split_kv.value, "k_order": p.k_order,
            "backend_policy": p.backend_policy, "deterministic_backend": p.deterministic_backend,
            "tp_forward_collective": p.tp_forward_collective.value,
            "tp_backward_dgrad_collective": p.tp_backward_dgrad_collective.value,
            "sp_forward_collective": p.sp_forward_collective.value, "sp_backward_collective": p.sp_backward_collective.value,
            "qkv_split_order": list(p.qkv_split_order), "require_runtime_readback": p.require_runtime_readback,
            "canonical_k_chunks": p.canonical_k_chunks}


@dataclass(frozen=True)
class AttentionBackendCapability:
    """What a concrete backend declares to contract-aware dispatch."""
    backend_id: str
    roles: frozenset
    modes: frozenset
    dtypes: frozenset
    cp_world_sizes: tuple[int, ...]
    tp_world_sizes: tuple[int, ...] | None = None
    exports_attention_lse: bool = False
    deterministic_cp_merge: bool = False
    supports_packed_varlen: bool = False
    supports_kv_cache: bool = False
    supports_rope_metadata: bool = False
    supports_fused_rope_attention: bool = False
    supports_split_kv_disabled: bool = True
    supports_split_kv_fixed: bool = False
    supports_split_kv_auto: bool = False
    reports_actual_split_kv_plan: bool = False
    implementation_kind: str = "production"
    head_dims: tuple[int, ...] | None = None
    causal_only: bool = False

    def __post_init__(self) -> None:
        if not isinstance(self.backend_id, str) or not self.backend_id.strip():
            raise AttentionContractError("backend_id must be a non-empty string")
        roles = frozenset(_enum_value(AttentionRole, v, "roles") for v in self.roles)
        modes = frozenset(_enum_value(AttentionMode, v, "modes") for v in self.modes)
        dtypes = frozenset(_enum_value(AttentionDType, v, "dtypes") for v in self.dtypes)
        if not roles or not modes or not dtypes:
            raise AttentionContractError("backend roles, modes, and dtypes must not be empty")
        cps = _world_sizes(self.cp_world_sizes, "cp_world_sizes")
        if cps is None:
            raise AttentionContractError("cp_world_sizes must contain positive values")
        tps = _world_sizes(self.tp_world_sizes, "tp_world_sizes")
        for flag in ("exports_attention_lse", "deterministic_cp_merge", "supports_packed_varlen", "supports_kv_cache",
                     "supports_rope_metadata", "supports_fused_rope_attention", "supports_split_kv_disabled",
                     "supports_split_kv_fixed", "supports_split_kv_auto", "reports_actual_split_kv_plan", "causal_only"):
            if not isinstance(getattr(self, flag), bool):
                raise AttentionContractError(f"{flag} must be a bool")
        if self.implementation_kind not in {"production", "reference", "deterministic"}:
            raise AttentionContractError("implementation_kind must be production, reference, or deterministic")
        for name, value in (("roles", roles), ("modes", modes), ("dtypes", dtypes), ("cp_world_sizes", cps),
                            ("tp_world_sizes", tps)):
            object.__setattr__(self, name, value)

    def incompatibilities(self, contract: AttentionContract) -> tuple[str, ...]:
        """Every reason this backend cannot materialise ``contract``."""
        why: list[str] = []
        if contract.role not in self.roles:
            why.append(f"role={contract.role.value} is unsupported")
        if contract.mode not in self.modes:
            why.append(f"mode={contract.mode.value} is unsupported")
        if contract.dtype not in self.dtypes:
            why.append(f"dtype={contract.dtype.value} is unsupported")
        tp, cp = contract.sharding.tp_world_size, contract.sharding.cp_world_size
        if self.tp_world_sizes is not None and tp not in self.tp_world_sizes:
            why.append(f"TP={tp} is unsupported")
        if cp not in self.cp_world_sizes:
            why.append(f"CP={cp} is unsupported")
        if self.head_dims is not None and contract.head_dim not in self.head_dims:
            why.append(f"head_dim={contract.head_dim} is unsupported")
        if self.causal_only and not contract.causal:
            why.append("non-causal attention is unsupported")
        if contract.export_lse and not self.exports_attention_lse:
            why.append("attention-domain LSE export is unsupported")
        if cp > 1 and not self.deterministic_cp_merge:
            why.append("deterministic CP (out, lse) merge is unsupported")
        if contract.sharding.packed_sequence_offsets is not None and not self.supports_packed_varlen:
            why.append("packed varlen layout is unsupported")
        if contract.kv_cache is not None and not self.supports_kv_cache:
            why.append("KV-cache identity materialization is unsupported")
        if contract.rope is not None and not self.supports_rope_metadata:
            why.append("RoPE/position metadata is unsupported")
        if (contract.rope is not None and contract.rope.fusion_boundary is RoPEFusionBoundary.FUSED_ROPE_ATTENTION
                and not self.supports_fused_rope_attention):
            why.append("fused RoPE+Attention boundary is unsupported")
        ok = {SplitKVMode.DISABLED: self.supports_split_kv_disabled, SplitKVMode.FIXED: self.supports_split_kv_fixed,
              SplitKVMode.AUTO: self.supports_split_kv_auto}
        if not ok[contract.split_kv.mode]:
            why.append(f"Split-KV policy={contract.split_kv.mode.value} is unsupported")
        if contract.split_kv.strict_consistency and not self.reports_actual_split_kv_plan:
            why.append("actual Split-KV execution-plan provenance is unsupported")
        return tuple(why)

    def supports(self, contract: AttentionContract) -> bool:
        return not self.incompatibilities(contract)

    def to_dict(self) -> dict[str, Any]:
        d = {"backend_id": self.backend_id, "roles": sorted(r.value for r in self.roles),
             "modes": sorted(m.value for m in self.modes), "dtypes": sorted(t.value for t in self.dtypes),
             "tp_world_sizes": list(self.tp_world_sizes) if self.tp_world_sizes else None,
             "cp_world_sizes": list(self.cp_world_sizes), "implementation_kind": self.implementation_kind,
             "head_dims": list(self.head_dims) if self.head_dims else None, "causal_only": self.causal_only}
        for flag in ("exports_attention_lse", "deterministic_cp_merge", "supports_packed_varlen", "supports_kv_cache",
                     "supports_rope_metadata", "supports_fused_rope_attention", "supports_split_kv_disabled",
                     "supports_split_kv_fixed", "supports_split_kv_auto", "reports_actual_split_kv_plan"):
            d[flag] = getattr(self, flag)
        return d


@dataclass(frozen=True)
class AttentionDispatchResult:
    """A concrete backend plus the provenance bound to the request."""
    op: Any
    capability: AttentionBackendCapability
    provenance: dict[str, Any]


B200_ATTENTION_CAPABILITY = AttentionBackendCapability(
    backend_id="b200-tcgen05", roles=frozenset(AttentionRole), modes=frozenset(AttentionMode),
    dtypes=frozenset({AttentionDType.BF16}), cp_world_sizes=(1, 2, 4, 8), tp_world_sizes=(1, 2, 4, 8),
    exports_attention_lse=True, deterministic_cp_merge=True, supports_packed_varlen=True, supports_kv_cache=True,
    supports_rope_metadata=True, supports_fused_rope_attention=True, reports_actual_split_kv_plan=True,
    implementation_kind="production", head_dims=(128,), causal_only=True)
REFERENCE_ATTENTION_CAPABILITY = AttentionBackendCapability(
    backend_id="pytorch-blockwise-reference", roles=frozenset(AttentionRole), modes=frozenset(AttentionMode),
    dtypes=frozenset(AttentionDType), cp_world_sizes=(1, 2, 4, 8), exports_attention_lse=True, deterministic_cp_merge=True,
    supports_packed_varlen=True, supports_kv_cache=True, supports_rope_metadata=True, supports_split_kv_fixed=True,
    reports_actual_split_kv_plan=True, implementation_kind="reference")

__all__ = [
    "ATTENTION_CONTRACT_ID", "AttentionBackendCapability", "AttentionContract", "AttentionContractError", "AttentionDType",
    "AttentionDispatchResult", "AttentionMerge", "AttentionMode", "AttentionProjectionSpec", "AttentionRole",
    "B200_ATTENTION_CAPABILITY", "CANONICAL_KV_BLOCK", "CPLayout", "CROSS_CONFIG_BOUND_FIELDS", "DowncastPoint",
    "KVCacheSpec", "MergeOrder", "ProjectionCollective", "REFERENCE_ATTENTION_CAPABILITY", "ReductionEngine",
    "ReductionOrder", "ReductionSpec", "RoPECastPoint", "RoPEFusionBoundary", "RoPESpec", "RoPEState",
    "STRICT_ATTENTION_CORE_ID", "STRICT_ATTENTION_FA4_SCHEDULE_ID", "STRICT_ATTENTION_PRODUCTION_CORE_ID",
    "STRICT_ATTENTION_REFERENCE_CORE_ID", "STRICT_ATTENTION_RING_SCHEDULE_ID", "STRICT_ATTENTION_SCHEDULE_ID",
    "ShardingSpec", "SplitKVExecutionPlan", "SplitKVMode", "SplitKVRuntimeCoordinate", "SplitKVRuntimePlanEntry",
    "SplitKVRuntimePlanSet", "SplitKVSpec", "build_split_kv_runtime_plan_set", "validate_cross_config_alignment",
    "validate_split_kv_alignment", "validate_split_kv_plan_set_alignment",
]
