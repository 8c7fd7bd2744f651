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

import math

from rl_kernel_b200.contracts.operators.attention import (SplitKVExecutionPlan, SplitKVMode, SplitKVRuntimeCoordinate,
                                                          SplitKVRuntimePlanEntry, SplitKVRuntimePlanSet, SplitKVSpec)
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



# ------------------------------------------------------------------------------------------------ saved forward state
STRICT_ATTENTION_CORE_ID = DeterministicAttentionCore.core_id
STRICT_ATTENTION_SCHEDULE_ID = "ascending_128_key_blocks.per_row_products.v1"


def _tensor_fingerprint(t: torch.Tensor) -> str:
    return hashlib.sha256(t.detach().contiguous().cpu().view(torch.uint8).numpy().tobytes()).hexdigest()


@dataclass(frozen=True)
class AttentionSavedForwardState:
    """What a training forward keeps for its backward: the fp32 output and log-sum-exp of every query row, the geometry
    they were computed under, and digests of the operands, so that a backward fed other tensors (a stale K/V after a
    cache write, a different sharding) is refused instead of producing plausible numbers."""
    out: torch.Tensor                       # [S, Hq, D] fp32
    lse: torch.Tensor                       # [S, Hq] fp32
    scale: float
    cp_world_size: int
    layout: str
    kv_chunk_size: Optional[int]
    query_positions: tuple[tuple[int, ...], ...]      # per rank, the logical positions of its query rows
    q_shape: tuple[int, ...]
    k_shape: tuple[int, ...]
    v_shape: tuple[int, ...]
    q_dtype: torch.dtype
    k_dtype: torch.dtype
    v_dtype: torch.dtype
    q_fingerprint: str
    k_fingerprint: str
    v_fingerprint: str
    out_fingerprint: str
    lse_fingerprint: str
    strict_bitwise: bool
    strict_schedule: Optional[str]

    def __post_init__(self) -> None:
        if self.out.dtype is not torch.float32 or self.lse.dtype is not torch.float32:
            raise ValueError("saved attention out/lse must be FP32")
        if self.out.ndim != 3 or self.lse.shape != self.out.shape[:2]:
            raise ValueError("saved attention out [S, H, D] / lse [S, H] shapes are invalid")
        if not math.isfinite(self.scale) or self.scale <= 0:
            raise ValueError("saved attention scale must be positive and finite")
        if self.strict_schedule != (STRICT_ATTENTION_SCHEDULE_ID if self.strict_bitwise else None):
            raise ValueError("saved attention strict schedule does not match strict_bitwise")
        if self.kv_chunk_size is not None and self.kv_chunk_size < 1:
            raise ValueError("kv_chunk_size must be >= 1 when provided")

    def validate_operands(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> None:
        for name, t, shape, dtype, fp in (("q", q, self.q_shape, self.q_dtype, self.q_fingerprint), ("k", k, self.k_shape, self.k_dtype, self.k_fingerprint),
                                          ("v", v, self.v_shape, self.v_dtype, self.v_fingerprint)):
            if tuple(t.shape) != shape or t.dtype != dtype:
                raise ValueError(f"backward operand {name} is {tuple(t.shape)} {t.dtype}; the forward saw {shape} {dtype}")
            if _tensor_fingerprint(t) != fp:
                raise ValueError(f"backward operand {name} differs from the tensor the forward state was saved for")
        if _tensor_fingerprint(self.out) != self.out_fingerprint or _tensor_fingerprint(self.lse) != self.lse_fingerprint:
            raise ValueError("the saved out / lse were modified after the forward")


@dataclass(frozen=True)
class AttentionBackwardPathResult:
    """One materialised backward path (a CP degree and an optional KV chunking) with the state it started from."""
    name: str
    out: torch.Tensor
    lse: torch.Tensor
    gradients: AttentionBackwardGradients
    saved_forward_state: AttentionSavedForwardState
    provenance: dict


@dataclass(frozen=True)
class AttentionBackwardPathDrift:
    candidate_name: str
    reference_name: str
    out: GradientDriftStats
    lse: GradientDriftStats
    dq: GradientDriftStats
    dk: GradientDriftStats
    dv: GradientDriftStats
    ranks: tuple[AttentionBackwardRankDrift, ...]

    def to_dict(self) -> dict[str, object]:
        return {"candidate": self.candidate_name, "reference": self.reference_name, "out": self.out.to_dict(), "lse": self.lse.to_dict(),
                "dq": self.dq.to_dict(), "dk": self.dk.to_dict(), "dv": self.dv.to_dict(), "ranks": [r.to_dict() for r in self.ranks]}


def backward_path_name(*, cp_world_size: int, kv_chunk_size: Optional[int]) -> str:
    return f"cp{cp_world_size}" + ("" if kv_chunk_size is None else f"_kvchunk{kv_chunk_size}") + "_backward_reference"


def save_forward_state(op: DeterministicCPAttentionReferenceOp, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *,
                       kv_chunk_size: Optional[int] = None) -> AttentionSavedForwardState:
    """Run ``op``'s forward in fp32 and keep what the explicit backward needs."""
    S, D = q.shape[0], q.shape[-1]
    out, lse = op.forward_with_lse(q.float(), k.float(), v.float())
    out, lse = out.float().contiguous(), lse.float().contiguous()
    scale = op.scale if op.scale is not None else 1.0 / math.sqrt(D)
    return AttentionSavedForwardState(
        out, lse, float(scale), op.cp, op.layout, kv_chunk_size, tuple(tuple(int(x) for x in p.tolist()) for p in op.shard_positions(S)),
        tuple(q.shape), tuple(k.shape), tuple(v.shape), q.dtype, k.dtype, v.dtype, _tensor_fingerprint(q), _tensor_fingerprint(k),
        _tensor_fingerprint(v), _tensor_fingerprint(out), _tensor_fingerprint(lse), op.strict_bitwise,
        STRICT_ATTENTION_SCHEDULE_ID if op.strict_bitwise else None)


def backward_from_saved_state(state: AttentionSavedForwardState, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                              dout: torch.Tensor) -> AttentionBackwardGradients:
    """The attention backward written out (no autograd), from the saved log-sum-exp:

        P = exp(scale * Q K^T - lse),  delta = rowsum(dO * O),  dV += P^T dO,  dS = P * (dO V^T - delta),
        dQ += scale * dS K,  dK += scale * dS^T Q

    evaluated rank by rank over that rank's query rows and, within a rank, over key chunks of ``kv_chunk_size`` in
    ascending order; dK / dV accumulate in (rank, chunk) order, a fixed order for every run.  Causality is by logical
    position, so any layout gives the gradients of the same function."""
    state.validate_operands(q, k, v)
    if tuple(dout.shape) != tuple(state.out.shape):
        raise ValueError(f"dout must have the output shape {tuple(state.out.shape)}, got {tuple(dout.shape)}")
    S, Hq, D = q.shape
    Hkv = k.shape[1]
    g = Hq // Hkv
    qf, do = q.float(), dout.float()
    kf = k.float().repeat_interleave(g, dim=1)                   # [S, Hq, D]
    vf = v.float().repeat_interleave(g, dim=1)
    dq = torch.zeros(S, Hq, D)
    dk_h, dv_h = torch.zeros(S, Hq, D), torch.zeros(S, Hq, D)
    delta = (do * state.out).sum(-1)                             # [S, Hq]
    chunk = state.kv_chunk_size or S
    keys = torch.arange(S)
    for pos in state.query_positions:
        rows = torch.tensor(pos, dtype=torch.long)
        if rows.numel() == 0:
            continue
        ql, dol, lsel, dl = qf[rows], do[rows], state.lse[rows], delta[rows]
        last = int(rows.max()) + 1
        for a in range(0, last, chunk):
            e = min(last, a + chunk)
            vis = keys[a:e][None, :] <= rows[:, None]                                   # [n, c]
            sc = torch.einsum("nhd,chd->hnc", ql, kf[a:e]) * state.scale
            p = torch.exp(sc - lsel.t().unsqueeze(-1))
            p = torch.where(vis[None], p, torch.zeros_like(p))
            dv_h[a:e] += torch.einsum("hnc,nhd->chd", p, dol)
            dp = torch.einsum("nhd,chd->hnc", dol, vf[a:e])
            ds = p * (dp - dl.t().unsqueeze(-1))
            dq[rows] += torch.einsum("hnc,chd->nhd", ds, kf[a:e]) * state.scale
            dk_h[a:e] += torch.einsum("hnc,nhd->chd", ds, ql) * state.scale
    dk = dk_h.view(S, Hkv, g, D).sum(2)
    dv = dv_h.view(S, Hkv, g, D).sum(2)
    return AttentionBackwardGradients(dq, dk, dv)


def backward_path(q, k, v, dout, *, cp_world_size: int = 1, layout: str = "zigzag", kv_chunk_size: Optional[int] = None,
                  scale: Optional[float] = None, strict_bitwise: bool = True, name: Optional[str] = None) -> AttentionBackwardPathResult:
    op = DeterministicCPAttentionReferenceOp(cp_world_size, layout, strict_bitwise=strict_bitwise, scale=scale)
    state = save_forward_state(op, q, k, v, kv_chunk_size=kv_chunk_size)
    grads = backward_from_saved_state(state, q, k, v, dout)
    prov = {"cp_world_size": cp_world_size, "layout": layout, "kv_chunk_size": kv_chunk_size, "core": STRICT_ATTENTION_CORE_ID,
            "schedule": state.strict_schedule, "forward": op.execution_provenance(q.shape[0]),
            "split_kv": split_kv_execution_plan_provenance(q.shape[0], cp_world_size=cp_world_size, kv_chunk_size=kv_chunk_size,
                                                           backend="deterministic_cp_reference")}
    return AttentionBackwardPathResult(name or backward_path_name(cp_world_size=cp_world_size, kv_chunk_size=kv_chunk_size), state.out,
                                       state.lse, grads, state, prov)


def compare_backward_paths(candidate: AttentionBackwardPathResult, reference: AttentionBackwardPathResult) -> AttentionBackwardPathDrift:
    ranks = tuple(AttentionBackwardRankDrift(r, _drift(candidate.gradients.dq[list(pos)], reference.gradients.dq[list(pos)]))
                  for r, pos in enumerate(candidate.saved_forward_state.query_positions) if pos)
    c, r = candidate.gradients, reference.gradients
    fin = torch.isfinite(reference.lse)
    return AttentionBackwardPathDrift(candidate.name, reference.name, _drift(candidate.out, reference.out),
                                      _drift(candidate.lse[fin], reference.lse[fin]), _drift(c.dq, r.dq), _drift(c.dk, r.dk), _drift(c.dv, r.dv), ranks)


# ------------------------------------------------------------------------------------------------ split-KV plans
def _split_bounds(length: int, parts: int) -> list[tuple[int, int]]:
    base, rem = divmod(length, parts)
    out, s = [], 0
    for i in range(parts):
        e = s + base + (1 if i < rem else 0)
        out.append((s, e))
        s = e
    return out


def _plan(owner: tuple[int, int], kv_chunk_size: Optional[int], backend: str, source: str) -> SplitKVExecutionPlan:
    a, e = owner
    if kv_chunk_size is None:
        mode, bounds = SplitKVMode.DISABLED, ((a, e),)
    else:
        mode, bounds = SplitKVMode.FIXED, tuple((x, min(x + kv_chunk_size, e)) for x in range(a, e, kv_chunk_size))
    return SplitKVExecutionPlan(mode, kv_chunk_size, mode, kv_chunk_size, bounds, backend=backend, source=source)


def split_kv_execution_plan_provenance(length: int, *, cp_world_size: int, kv_chunk_size: Optional[int], backend: str) -> list[dict]:
    """The plan every CP owner's key range was actually consumed with, as provenance records."""
    if length < 1 or cp_world_size < 1 or (kv_chunk_size is not None and kv_chunk_size < 1):
        raise ValueError("length, cp_world_size and kv_chunk_size must be >= 1")
    return [{"owner_cp_rank": o, **_plan(b, kv_chunk_size, backend, "reference_execution").to_dict()}
            for o, b in enumerate(_split_bounds(length, cp_world_size)) if b[1] > b[0]]


def build_reference_split_kv_runtime_plan_set(total_kv_tokens: Sequence[int], *, tp_world_size: int, cp_world_size: int,
                                              kv_chunk_size: Optional[int], backend: str = "deterministic_cp_reference"
                                              ) -> SplitKVRuntimePlanSet:
    """Complete batch x TP x CP consumer x CP owner plans of the reference path (what a runtime must report to be bound)."""
    totals = tuple(int(t) for t in total_kv_tokens)
    if not totals or any(t < cp_world_size for t in totals):
        raise ValueError("reference runtime plan sets require at least one KV token per CP owner")
    if tp_world_size < 1 or cp_world_size < 1 or (kv_chunk_size is not None and kv_chunk_size < 1):
        raise ValueError("world sizes and kv_chunk_size must be >= 1")
    entries = [SplitKVRuntimePlanEntry(SplitKVRuntimeCoordinate(b, t, c, o), owner, _plan(owner, kv_chunk_size, backend, "reference_execution"))
               for b, total in enumerate(totals) for t in range(tp_world_size) for c in range(cp_world_size)
               for o, owner in enumerate(_split_bounds(total, cp_world_size))]
    return SplitKVRuntimePlanSet(len(totals), tp_world_size, cp_world_size, totals, tuple(entries))


CPAttentionReferenceOp = DeterministicCPAttentionReferenceOp

__all__ = ["AttentionBackwardComparisonReport", "AttentionBackwardGradients", "AttentionBackwardPathDrift", "AttentionBackwardPathResult",
           "AttentionBackwardRankDrift", "AttentionPartialState", "AttentionRingBlock", "AttentionRingSchedule", "AttentionSavedForwardState",
           "CPAttentionReferenceOp", "DeterministicAttentionCore", "DeterministicAttentionCoreResult", "DeterministicCPAttentionReferenceOp",
           "GradientDriftStats", "STRICT_ATTENTION_CORE_ID", "STRICT_ATTENTION_SCHEDULE_ID", "backward_from_saved_state", "backward_path",
           "backward_path_name", "build_reference_split_kv_runtime_plan_set", "compare_backward_paths", "compare_cp_attention_backward",
           "merge_attention_partial_states", "save_forward_state", "split_kv_execution_plan_provenance"]
