"""Context-parallel attention reference with an explicit ring schedule and a backward comparison (parity:
rl_engine/reference/attention/cp_attention.py:35-1942).

Two forward paths over the same sharding:

* strict (``strict_bitwise=True``): every rank attends its query rows to the whole logical K/V in ascending 128-key
  blocks -- what an all-gather of K/V, or the peer-memory kernel, computes.  Bit-equal to one rank for every CP degree
  and layout.
* ring: K/V shards travel round a ring; at step s rank r holds the shard of rank (r - s) mod cp and produces one
  partial state per held chunk.  The partial states are merged -- by ascending global block start
  (``merge_order='global_block_index'``) or in the order they arrived (``'arrival'``, the control group).  A merge of
  partial states is other arithmetic than the one-pass online softmax, so this path is tolerance-equal to the strict one;
  the schedule object says which rank sees which block when.

The backward reference differentiates the strict forward per rank; ``compare_cp_attention_backward`` reports the drift
of dq / dk / dv between a CP degree and one rank, per rank shard.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch

from rl_kernel_b200.contracts.operators.attention import SplitKVSpec
from rl_kernel_b200.reference.attention.blockwise import (BLOCK, DeterministicCPAttentionReferenceOp as _StrictCPOp,
                                                          blockwise_attention_reference, merge_two_states, zigzag_chunks)


@dataclass(frozen=True)
class AttentionPartialState:
    out: torch.Tensor            # [n, Hq, D] fp32
    lse: torch.Tensor            # [n, Hq]
    block_start: int             # first global key position covered
    block_end: int
    source_rank: int = 0
    step: int = 0

    def __post_init__(self) -> None:
        if self.block_end <= self.block_start:
            raise ValueError("a partial state covers a non-empty key range")
        if self.out.shape[:-1] != self.lse.shape:
            raise ValueError("out [n, H, D] and lse [n, H] disagree")


@dataclass(frozen=True)
class AttentionRingBlock:
    step: int
    holder_rank: int
    source_rank: int
    key_start: int
    key_end: int


@dataclass(frozen=True)
class AttentionRingSchedule:
    cp_world_size: int
    seq_len: int
    layout: str
    blocks: tuple[AttentionRingBlock, ...]

    @classmethod
    def build(cls, *, cp_world_size: int, seq_len: int, layout: str = "zigzag") -> "AttentionRingSchedule":
        if cp_world_size < 1 or seq_len < 1:
            raise ValueError("cp_world_size and seq_len must be positive")
        if layout == "zigzag":
            chunks = zigzag_chunks(seq_len, cp_world_size) if cp_world_size > 1 else [[(0, seq_len)]]
        elif layout == "contiguous":
            if seq_len % cp_world_size:
                raise ValueError("seq_len must divide by cp_world_size")
            c = seq_len // cp_world_size
            chunks = [[(r * c, (r + 1) * c)] for r in range(cp_world_size)]
        else:
            raise ValueError("layout must be zigzag or contiguous")
        blocks = []
        for step in range(cp_world_size):
            for r in range(cp_world_size):
                src = (r - step) % cp_world_size
                blocks += [AttentionRingBlock(step, r, src, a, b) for a, b in chunks[src]]
        return cls(cp_world_size, seq_len, layout, tuple(blocks))

    def owned(self, rank: int) -> list[tuple[int, int]]:
        return [(b.key_start, b.key_end) for b in self.blocks if b.step == 0 and b.holder_rank == rank]

    def arrivals(self, rank: int) -> list[AttentionRingBlock]:
        return [b for b in self.blocks if b.holder_rank == rank]

    def provenance(self) -> dict[str, object]:
        text = ";".join(f"{b.step}:{b.holder_rank}<{b.source_rank}[{b.key_start},{b.key_end})" for b in self.blocks)
        return {"cp_world_size": self.cp_world_size, "seq_len": self.seq_len, "layout": self.layout, "steps": self.cp_world_size,
                "blocks": len(self.blocks), "schedule_sha256": hashlib.sha256(text.encode()).hexdigest()[:16]}


def merge_attention_partial_states(states: Sequence[AttentionPartialState], *, order: str = "global_block_index"
                                   ) -> tuple[torch.Tensor, torch.Tensor]:
    """Merge partial states of one set of query rows over disjoint key ranges."""
    if not states:
        raise ValueError("nothing to merge")
    if order == "global_block_index":
        states = sorted(states, key=lambda s: s.block_start)
        for a, b in zip(states, states[1:]):
            if b.block_start < a.block_end:
                raise ValueError(f"partial states overlap: [{a.block_start},{a.block_end}) and [{b.block_start},{b.block_end})")
    elif order != "arrival":
        raise ValueError("order must be global_block_index or arrival")
    o, l = states[0].out.float(), states[0].lse
    for s in states[1:]:
        o, l = merge_two_states(o, l, s.out.float(), s.lse)
    return o, l


@dataclass(frozen=True)
class DeterministicAttentionCoreResult:
    out: torch.Tensor
    lse: torch.Tensor
    provenance: dict = field(default_factory=dict)


class DeterministicAttentionCore:
    """The shared core: 128-key blocks ascending, per-row products; an optional fixed split-KV with an ordered merge."""

    core_id = "rlkernel.attention.blockwise128.v1"

    def __init__(self, *, split_kv: SplitKVSpec | None = None) -> None:
        self.split_kv = split_kv

    def forward_with_lse(self, q, k, v, *, q_positions: torch.Tensor, scale: float | None = None,
                         p_dtype: torch.dtype | None = None) -> DeterministicAttentionCoreResult:
        size = self.split_kv.fixed_split_size if self.split_kv is not None and self.split_kv.fixed_split_size else None
        if not size:
            o, l = blockwise_attention_reference(q, k, v, q_positions, scale=scale, p_dtype=p_dtype, strict=True)
            return DeterministicAttentionCoreResult(o, l, {"core": self.core_id, "splits": 1})
        if size % BLOCK:
            raise ValueError(f"a fixed split must be a multiple of the {BLOCK}-key block")
        parts = []
        for a in range(0, k.shape[0], size):
            e = min(k.shape[0], a + size)
            o, l = blockwise_attention_reference(q, k[a:e], v[a:e], q_positions - a, scale=scale, p_dtype=p_dtype, strict=True)
            dead = (q_positions - a) < 0
            parts.append(AttentionPartialState(o.float().masked_fill(dead[:, None, None], 0.0), l.masked_fill(dead[:, None], float("-inf")),
                                               a, e))
        o, l = merge_attention_partial_states(parts)
        return DeterministicAttentionCoreResult(o.to(q.dtype), l, {"core": self.core_id, "splits": len(parts), "split_size": size})


class DeterministicCPAttentionReferenceOp:
    """``op(q, k, v)`` on one causal sequence (q [S, Hq, D], k / v [S, Hkv, D]) sharded over ``cp`` simulated ranks."""

    def __init__(self, cp: int = 1, layout: str = "zigzag", *, strict_bitwise: bool = True, merge_order: str = "global_block_index",
                 scale: float | None = None, p_dtype: torch.dtype | None = None) -> None:
        self.cp, self.layout, self.strict_bitwise, self.merge_order = cp, layout, strict_bitwise, merge_order
        self.scale, self.p_dtype = scale, p_dtype
        self._strict = _StrictCPOp(cp, layout, scale, p_dtype)

    def ring_schedule(self, seq_len: int) -> AttentionRingSchedule:
        return AttentionRingSchedule.build(cp_world_size=self.cp, seq_len=seq_len, layout=self.layout)

    def shard_positions(self, seq_len: int) -> list[torch.Tensor]:
        return self._strict.shard_positions(seq_len)

    def execution_provenance(self, seq_len: int) -> dict[str, object]:
        return {"path": "strict_all_gather" if self.strict_bitwise else "ring_partial_merge", "merge_order": self.merge_order,
                **self.ring_schedule(seq_len).provenance()}

    def local_partial_state(self, q_local, k_block, v_block, q_positions, block: AttentionRingBlock) -> AttentionPartialState:
        """Rank-local queries against one arrived key chunk."""
        o, l = blockwise_attention_reference(q_local, k_block, v_block, q_positions - block.key_start, scale=self.scale,
                                             p_dtype=self.p_dtype, strict=True)
        dead = (q_positions - block.key_start) < 0
        return AttentionPartialState(o.float().masked_fill(dead[:, None, None], 0.0), l.masked_fill(dead[:, None], float("-inf")),
                                     block.key_start, block.key_end, block.source_rank, block.step)

    def forward_with_lse(self, q, k, v):
        if self.strict_bitwise or self.cp == 1:
            return self._strict(q, k, v)
        S = q.shape[0]
        sched = self.ring_schedule(S)
        out, lse = torch.empty_like(q), torch.empty(S, q.shape[1])
        for r, pos in enumerate(self.shard_positions(S)):
            states = [self.local_partial_state(q[pos], k[b.key_start:b.key_end], v[b.key_start:b.key_end], pos, b)
                      for b in sched.arrivals(r)]
            o, l = merge_attention_partial_states(states, order=self.merge_order)
            out[pos], lse[pos] = o.to(q.dtype), l
        return out, lse

    def __call__(self, q, k, v):
        return self.forward_with_lse(q, k, v)

    forward = __call__

    def forward_fp32(self, q, k, v):
        return self.forward_with_lse(q.float(), k.float(), v.float())

    def backward_reference(self, q, k, v, dout) -> "AttentionBackwardGradients":
        """dq / dk / dv of sum(out * dout) through the strict forward: every rank differentiates its own query rows
        against the whole K/V; dk and dv add up over the ranks in rank order (a fixed order, hence reproducible)."""
        S = q.shape[0]
        dq = torch.zeros_like(q, dtype=torch.float32)
        dk, dv = torch.zeros_like(k, dtype=torch.float32), torch.zeros_like(v, dtype=torch.float32)
        for pos in self.shard_positions(S):
            ql = q[pos].detach().float().requires_grad_(True)
            kk, vv = k.detach().float().requires_grad_(True), v.detach().float().requires_grad_(True)
            o, _ = blockwise_attention_reference(ql, kk, vv, pos, scale=self.scale, p_dtype=None, strict=False)
            (o * dout[pos].float()).sum().backward()
            dq[pos] = ql.grad
            dk += kk.grad
            dv += vv.grad
        return AttentionBackwardGradients(dq, dk, dv)


@dataclass(frozen=True)
class AttentionBackwardGradients:
    dq: torch.Tensor
    dk: torch.Tensor
    dv: torch.Tensor


@dataclass(frozen=True)
class GradientDriftStats:
    max_abs: float
    mean_abs: float
    max_rel: float

    def to_dict(self) -> dict[str, object]:
        return {"max_abs": self.max_abs, "mean_abs": self.mean_abs, "max_rel": self.max_rel}


@dataclass(frozen=True)
class AttentionBackwardRankDrift:
    rank: int
    dq: GradientDriftStats

    def to_dict(self) -> dict[str, object]:
        return {"rank": self.rank, "dq": self.dq.to_dict()}


@dataclass(frozen=True)
class AttentionBackwardComparisonReport:
    cp_world_size: int
    layout: str
    dq: GradientDriftStats
    dk: GradientDriftStats
    dv: GradientDriftStats
    ranks: tuple[AttentionBackwardRankDrift, ...]

    def to_dict(self) -> dict[str, object]:
        return {"cp_world_size": self.cp_world_size, "layout": self.layout, "dq": self.dq.to_dict(), "dk": self.dk.to_dict(),
                "dv": self.dv.to_dict(), "ranks": [r.to_dict() for r in self.ranks]}


def _drift(c: torch.Tensor, r: torch.Tensor) -> GradientDriftStats:
    d = (c.double() - r.double()).abs()
    return GradientDriftStats(float(d.max()), float(d.mean()), float(d.max() / r.double().abs().max().clamp_min(1e-30)))


def compare_cp_attention_backward(q, k, v, dout, *, cp_world_size: int, layout: str = "zigzag", scale: Optional[float] = None
                                  ) -> AttentionBackwardComparisonReport:
    one = DeterministicCPAttentionReferenceOp(1, layout, scale=scale).backward_reference(q, k, v, dout)
    op = DeterministicCPAttentionReferenceOp(cp_world_size, layout, scale=scale)
    many = op.backward_reference(q, k, v, dout)
    ranks = tuple(AttentionBackwardRankDrift(r, _drift(many.dq[pos], one.dq[pos])) for r, pos in enumerate(op.shard_positions(q.shape[0])))
    return AttentionBackwardComparisonReport(cp_world_size, layout, _drift(many.dq, one.dq), _drift(many.dk, one.dk), _drift(many.dv, one.dv), ranks)


__all__ = ["AttentionBackwardComparisonReport", "AttentionBackwardGradients", "AttentionBackwardRankDrift", "AttentionPartialState",
           "AttentionRingBlock", "AttentionRingSchedule", "DeterministicAttentionCore", "DeterministicAttentionCoreResult",
           "DeterministicCPAttentionReferenceOp", "GradientDriftStats", "compare_cp_attention_backward",
           "merge_attention_partial_states"]
