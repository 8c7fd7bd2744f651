"""Context-parallel attention: the communication contract and its implementations
(parity: rl_engine/backends/cuda/attention/cp_comm.py:43-1759).

Three ways to run attention whose sequence is split over ``cp_world_size`` ranks share one data
model (``AttentionParallelSpec``, ``AttentionCPBlockMetadata``, ``AttentionCPPartialState``,
``AttentionCPCommunicationPlan``):

``PeerMemoryAttentionCPCommunication``  (the product path on NVLink)
    Nothing is gathered: the attention kernel reads the other ranks' K/V tiles through peer tensor
    maps while it computes (rl_kernel_b200.distributed.cp_attention.CPAttention).  Every rank
    computes only its own query rows, so the work is divided by CP instead of replicated; the
    per-row program (ascending 128-key blocks) is the single-GPU one, hence the same bits.

``CUDAAGRSAttentionCPCommunication``  (the reference's strict graph, kept for comparison and CPU tests)
    all-gather(Q, K, V, positions) in rank order -> one shared attention core on the full logical
    sequence -> "reduce-scatter" of (out, lse), which is a slice because every rank holds the same
    full result.  Differentiable; the transport is any deterministic collective
    (``all_gather(t) -> [world, ...]``), Gloo on CPU included.

``P2PNCCLAttentionCPCommunication``  (partial-state reference)
    Each rank attends to the K/V blocks it owns and produces fp32 ``(out, lse)`` partial states tagged
    with their global block index; states travel by explicit send/recv in (peer, block) order, are
    sorted by block index and merged with the fp32 online-softmax rule; the root scatters the
    merged rows to their owners.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Literal, Protocol, Sequence

import torch

CPCommunicationBackend = Literal["peer_memory", "cuda_ag_rs", "p2p_nccl_reference", "local_debug"]
CPCommunicationStatus = Literal["interface_only", "implemented"]
_BACKENDS = ("peer_memory", "cuda_ag_rs", "p2p_nccl_reference", "local_debug")


class AttentionCPCommunicationUnavailable(RuntimeError):
    """The requested CP communication backend cannot run in this process."""


def _is_int(x) -> bool:
    return isinstance(x, int) and not isinstance(x, bool)


def _positive_int(value, name: str) -> int:
    if not _is_int(value) or value <= 0:
        raise ValueError(f"{name} must be a positive integer; got {value!r}")
    return value


def _rank_in_world(rank, world: int, name: str) -> int:
    if not _is_int(rank) or not 0 <= rank < world:
        raise ValueError(f"{name}={rank!r} must lie in [0, {world})")
    return rank


def _range_ok(start, end) -> bool:
    return _is_int(start) and _is_int(end) and 0 <= start < end


@dataclass(frozen=True)
class AttentionParallelSpec:
    """TP/CP identity of the calling rank."""
    tp_world_size: int = 2
    tp_rank: int = 0
    cp_world_size: int = 2
    cp_rank: int = 0

    def validate(self) -> None:
        _positive_int(self.tp_world_size, "tp_world_size")
        _positive_int(self.cp_world_size, "cp_world_size")
        _rank_in_world(self.tp_rank, self.tp_world_size, "tp_rank")
        _rank_in_world(self.cp_rank, self.cp_world_size, "cp_rank")

    def provenance(self) -> dict[str, int]:
        self.validate()
        return {"tp_world_size": self.tp_world_size, "tp_rank": self.tp_rank,
                "cp_world_size": self.cp_world_size, "cp_rank": self.cp_rank}


@dataclass(frozen=True)
class AttentionCPBlockMetadata:
    """Logical identity of one K/V block (and of the partial state computed against it)."""
    global_block_index: int
    kv_block_start: int
    kv_block_end: int
    owner_cp_rank: int
    owner_tp_rank: int

    def validate(self, parallel: AttentionParallelSpec) -> None:
        parallel.validate()
        if not _is_int(self.global_block_index) or self.global_block_index < 0:
            raise ValueError("global_block_index must be non-negative")
        if not _range_ok(self.kv_block_start, self.kv_block_end):
            raise ValueError("KV block bounds must satisfy 0 <= start < end")
        _rank_in_world(self.owner_cp_rank, parallel.cp_world_size, "owner_cp_rank")
        _rank_in_world(self.owner_tp_rank, parallel.tp_world_size, "owner_tp_rank")

    def provenance(self) -> dict[str, int]:
        return {"global_block_index": self.global_block_index, "kv_block_start": self.kv_block_start,
                "kv_block_end": self.kv_block_end, "owner_cp_rank": self.owner_cp_rank,
                "owner_tp_rank": self.owner_tp_rank}


def _check_state(out: torch.Tensor, lse: torch.Tensor, what: str, out_dtypes) -> None:
    if out.ndim != 4 or lse.ndim != 3:
        raise ValueError(f"{what} must have out [B, Hq, Sq, D] and lse [B, Hq, Sq]")
    if out.shape[:3] != lse.shape:
        raise ValueError(f"{what} out and lse must share [B, Hq, Sq]")
    if out.device != lse.device:
        raise ValueError(f"{what} out and lse must be on the same device")
    if lse.dtype != torch.float32:
        raise ValueError(f"{what} lse must be FP32")
    if out.dtype not in out_dtypes:
        raise ValueError(f"{what} out must be one of {[str(d) for d in out_dtypes]}")


@dataclass(frozen=True)
class AttentionCPPartialState:
    """One local or received fp32 ``(out, lse)`` state before the CP merge."""
    out: torch.Tensor
    lse: torch.Tensor
    block: AttentionCPBlockMetadata

    def validate(self, parallel: AttentionParallelSpec) -> None:
        self.block.validate(parallel)
        _check_state(self.out, self.lse, "partial", (torch.float32,))


@dataclass(frozen=True)
class AttentionCPMergedState:
    """Merged fp32 state before it is scattered to the query owners."""
    out: torch.Tensor
    lse: torch.Tensor

    def validate(self) -> None:
        _check_state(self.out, self.lse, "merged", (torch.float32,))


@dataclass(frozen=True)
class AttentionCPOutputShard:
    """This rank's final rows: output in the compute dtype, LSE in fp32."""
    out: torch.Tensor
    lse: torch.Tensor

    def validate(self) -> None:
        _check_state(self.out, self.lse, "strict output", (torch.float16, torch.bfloat16))


@dataclass(frozen=True)
class AttentionCPCommunicationPlan:
    """What a CP attention call communicates and how the pieces are ordered."""
    parallel: AttentionParallelSpec
    backend: str = "peer_memory"
    status: str = "implemented"
    pattern: str = "ag_rs"
    compute_communication: str = "decoupled"
    merge_order: str = "global_block_index"
    accum_dtype: torch.dtype = torch.float32
    return_lse: bool = True
    expected_blocks: tuple[AttentionCPBlockMetadata, ...] = ()
    expected_kv_token_range: tuple[int, int] | None = None
    query_token_ranges: tuple[tuple[int, int], ...] = ()
    merge_root_cp_rank: int = 0

    def validate(self) -> None:
        self.parallel.validate()
        if self.backend not in _BACKENDS:
            raise ValueError(f"unsupported CP communication backend: {self.backend}")
        if self.status not in ("interface_only", "implemented"):
            raise ValueError(f"unsupported CP communication status: {self.status}")
        want_pattern = "in_kernel_peer_loads" if self.backend == "peer_memory" else "ag_rs"
        if self.pattern not in ("ag_rs", want_pattern):
            raise ValueError(f"backend {self.backend} communicates by {want_pattern}, not {self.pattern}")
        if self.backend != "peer_memory" and self.compute_communication != "decoupled":
            raise ValueError("gather/scatter backends keep compute and communication decoupled")
        if self.merge_order != "global_block_index":
            raise ValueError("CP partial states merge in global_block_index order")
        if self.accum_dtype is not torch.float32:
            raise ValueError("CP merge accumulation must be FP32")
        if not self.return_lse:
            raise ValueError("CP communication requires LSE-carrying states")
        _rank_in_world(self.merge_root_cp_rank, self.parallel.cp_world_size, "merge_root_cp_rank")
        _validate_expected_block_manifest(self)
        _validate_query_token_ranges(self)
        if self.backend == "p2p_nccl_reference":
            if self.status != "implemented":
                raise ValueError("P2P reference plans must use status='implemented'")
            if not self.expected_blocks or self.expected_kv_token_range is None:
                raise ValueError("P2P reference requires a complete expected block manifest")
            if not self.query_token_ranges:
                raise ValueError("P2P reference requires one query range per CP rank")

    def provenance(self) -> dict[str, object]:
        self.validate()
        peer = self.backend == "peer_memory"
        return {
            "cp_comm_backend": self.backend, "cp_comm_status": self.status,
            "cp_comm_pattern": "in_kernel_peer_loads" if peer else self.pattern,
            "cp_comm_compute_communication": "fused" if peer else self.compute_communication,
            "cp_comm_merge_order": self.merge_order, "cp_comm_accum_dtype": "fp32",
            "cp_comm_return_lse": self.return_lse,
            "cp_comm_contract": "partial_out_lse_global_block_index",
            "cp_comm_strict_contract": ("owner_rows_canonical_key_blocks_over_peer_kv" if peer
                                        else "ag_qkv_positions_shared_core_rs_out_lse"),
            "cp_comm_strict_kv_communication": "tma_peer_loads" if peer else "all_gather",
            "cp_comm_runtime": {"peer_memory": "nvlink_peer_memory", "cuda_ag_rs": "deterministic_collective",
                                "p2p_nccl_reference": "nccl", "local_debug": "local"}[self.backend],
            "cp_comm_redundant_compute_factor": 1 if peer or self.backend == "p2p_nccl_reference"
            else self.parallel.cp_world_size,
            "cp_comm_expected_kv_token_range": None if self.expected_kv_token_range is None
            else list(self.expected_kv_token_range),
            "cp_comm_expected_blocks": [b.provenance() for b in self.expected_blocks],
            "cp_comm_query_token_ranges": [list(r) for r in self.query_token_ranges],
            "cp_comm_merge_root_cp_rank": self.merge_root_cp_rank,
            **self.parallel.provenance(),
        }


def _validate_expected_block_manifest(plan: AttentionCPCommunicationPlan) -> None:
    blocks = plan.expected_blocks
    if not blocks:
        if plan.expected_kv_token_range is not None:
            raise ValueError("expected_kv_token_range requires expected_blocks")
        return
    for b in blocks:
        b.validate(plan.parallel)
        if b.owner_tp_rank != plan.parallel.tp_rank:
            raise ValueError("expected block owner_tp_rank must match the plan TP shard")
    if len(set(blocks)) != len(blocks):
        raise ValueError("expected block manifest contains duplicate metadata")
    ordered = sorted(blocks, key=lambda b: b.global_block_index)
    idx = [b.global_block_index for b in ordered]
    if len(set(idx)) != len(idx):
        raise ValueError("expected block manifest contains duplicate global_block_index values")
    if {b.owner_cp_rank for b in blocks} != set(range(plan.parallel.cp_world_size)):
        raise ValueError("expected block manifest must assign work to every CP rank")
    if plan.expected_kv_token_range is None:
        raise ValueError("expected block manifest requires expected_kv_token_range")
    try:
        start, end = plan.expected_kv_token_range
    except (TypeError, ValueError) as exc:
        raise ValueError("expected KV range must contain exactly (start, end)") from exc
    if not _range_ok(start, end):
        raise ValueError("expected KV range must satisfy 0 <= start < end")
    if ordered[0].kv_block_start != start or ordered[-1].kv_block_end != end:
        raise ValueError("expected block manifest does not cover the declared KV range")
    prev = start
    for b in ordered:
        if b.kv_block_start != prev:
            raise ValueError("expected block manifest must be gap-free and non-overlapping")
        prev = b.kv_block_end


def _validate_query_token_ranges(plan: AttentionCPCommunicationPlan) -> None:
    ranges = plan.query_token_ranges
    if not ranges:
        return
    if len(ranges) != plan.parallel.cp_world_size:
        raise ValueError("query_token_ranges must contain one range per CP rank")
    prev = 0
    for r, pair in enumerate(ranges):
        try:
            start, end = pair
        except (TypeError, ValueError) as exc:
            raise ValueError("each query token range must be (start, end)") from exc
        if not _range_ok(start, end):
            raise ValueError(f"query range of CP rank {r} must satisfy 0 <= start < end")
        if start != prev:
            raise ValueError("query token ranges must be contiguous in CP-rank order starting at 0")
        prev = end


def sort_attention_cp_partial_states(states: Sequence[AttentionCPPartialState], *,
                                     plan: AttentionCPCommunicationPlan) -> tuple[AttentionCPPartialState, ...]:
    """Validate a set of partial states and return it in ``global_block_index`` order."""
    plan.validate()
    if not states:
        raise ValueError("at least one CP attention partial state is required")
    for s in states:
        s.validate(plan.parallel)
    ordered = tuple(sorted(states, key=lambda s: s.block.global_block_index))
    idx = [s.block.global_block_index for s in ordered]
    if len(set(idx)) != len(idx):
        raise ValueError("duplicate global_block_index values are not allowed")
    if plan.expected_blocks:
        want = sorted(plan.expected_blocks, key=lambda b: b.global_block_index)
        if [s.block for s in ordered] != want:
            raise ValueError("partial states do not match the expected block manifest")
    else:
        if idx != list(range(len(ordered))):
            raise ValueError("partial states without a manifest must cover global_block_index values [0, block_count)")
        if ordered[0].block.kv_block_start != 0:
            raise ValueError("partial states without a manifest must start at KV token 0")
    if plan.expected_kv_token_range is not None:
        start, end = plan.expected_kv_token_range
        if ordered[0].block.kv_block_start != start or ordered[-1].block.kv_block_end != end:
            raise ValueError("partial states do not cover the declared expected KV token range")
    shape = ordered[0].out.shape
    prev_end = ordered[0].block.kv_block_start
    for s in ordered:
        if s.out.shape != shape:
            raise ValueError("all partial states must share the query shape [B, Hq, Sq, D]")
        if s.block.kv_block_start != prev_end:
            raise ValueError("partial states must tile the KV range without gaps or overlap")
        prev_end = s.block.kv_block_end
    return ordered


def merge_attention_cp_partial_states(states: Sequence[AttentionCPPartialState], *,
                                      plan: AttentionCPCommunicationPlan) -> AttentionCPMergedState:
    """fp32 online-softmax merge in block order: M = max(M, lse_i); out = out*e^(M_old-M) + out_i*e^(lse_i-M).
    A state whose LSE is -inf (no visible key for that row in that block) contributes nothing."""
    ordered = sort_attention_cp_partial_states(states, plan=plan)
    out = torch.zeros_like(ordered[0].out)
    lse = torch.full_like(ordered[0].lse, float("-inf"))
    for s in ordered:
        new = torch.maximum(lse, s.lse)
        safe = torch.where(torch.isinf(new), torch.zeros_like(new), new)
        w_old = torch.where(torch.isinf(lse), torch.zeros_like(lse), torch.exp(lse - safe))
        w_new = torch.where(torch.isinf(s.lse), torch.zeros_like(lse), torch.exp(s.lse - safe))
        out = out * w_old.unsqueeze(-1) + s.out * w_new.unsqueeze(-1)
        tot = w_old + w_new
        out = torch.where(tot.unsqueeze(-1) > 0, out / tot.clamp_min(1e-38).unsqueeze(-1), out)
        lse = torch.where(tot > 0, safe + torch.log(tot.clamp_min(1e-38)), new)
    return AttentionCPMergedState(out, lse)


class AttentionCPCommunication(Protocol):
    """What a CP communication backend provides."""

    def all_gather_query(self, local_q: torch.Tensor, plan: AttentionCPCommunicationPlan) -> torch.Tensor: ...

    def all_gather_kv(self, local_k: torch.Tensor, local_v: torch.Tensor,
                      plan: AttentionCPCommunicationPlan) -> tuple[torch.Tensor, torch.Tensor]: ...

    def all_gather_position_ids(self, local_query_positions: torch.Tensor, local_key_positions: torch.Tensor,
                                plan: AttentionCPCommunicationPlan) -> tuple[torch.Tensor, torch.Tensor]: ...

    def all_gather_partial_states(self, local_states: tuple[AttentionCPPartialState, ...],
                                  plan: AttentionCPCommunicationPlan) -> tuple[AttentionCPPartialState, ...]: ...

    def reduce_scatter_merged_state(self, merged_state: AttentionCPMergedState,
                                    plan: AttentionCPCommunicationPlan) -> AttentionCPMergedState: ...

    def reduce_scatter_strict_result(self, out: torch.Tensor, lse: torch.Tensor,
                                     plan: AttentionCPCommunicationPlan) -> AttentionCPOutputShard: ...


# ------------------------------------------------------------------ gather / scatter over a collective
class _AllGatherSequence(torch.autograd.Function):
    """Rank-ordered all-gather along ``sequence_dim``; the backward hands each rank the slice of
    the gradient that belongs to its rows (every rank computed the same full result, so the slices of
    the ranks' gradients are summed in the fixed tree of the collective)."""

    @staticmethod
    def forward(ctx, local, collective, sequence_dim, reduce_grad):
        ctx.collective, ctx.dim, ctx.reduce_grad = collective, int(sequence_dim), bool(reduce_grad)
        ctx.n = local.shape[ctx.dim]
        parts = collective.all_gather(local.movedim(ctx.dim, 0).contiguous())      # [world, n, ...]
        full = parts.reshape(-1, *parts.shape[2:])
        return full.movedim(0, ctx.dim).contiguous()

    @staticmethod
    def backward(ctx, grad):
        g = grad.movedim(ctx.dim, 0).contiguous()
        if ctx.reduce_grad and ctx.collective.world > 1:
            g = ctx.collective.all_reduce(g)
        r = ctx.collective.rank
        return g[r * ctx.n:(r + 1) * ctx.n].movedim(0, ctx.dim).contiguous(), None, None, None


class _ScatterSequence(torch.autograd.Function):
    """This rank's rows of a tensor that every rank holds in full; the backward gathers the ranks'
    row gradients back into the full shape."""

    @staticmethod
    def forward(ctx, full, collective, sequence_dim, start, end):
        ctx.collective, ctx.dim, ctx.bounds, ctx.total = collective, int(sequence_dim), (start, end), full.shape[sequence_dim]
        return full.narrow(ctx.dim, start, end - start).contiguous()

    @staticmethod
    def backward(ctx, grad):
        g = torch.zeros(*grad.shape[:ctx.dim], ctx.total, *grad.shape[ctx.dim + 1:], dtype=grad.dtype, device=grad.device)
        g.narrow(ctx.dim, ctx.bounds[0], ctx.bounds[1] - ctx.bounds[0]).copy_(grad)
        if ctx.collective.world > 1:                 # disjoint rows: the "sum" only fills in the other ranks' rows
            g = ctx.collective.all_reduce(g)
        return g, None, None, None, None


class CUDAAGRSAttentionCPCommunication:
    """all-gather(Q, K, V, positions) -> shared core -> slice, over a deterministic collective."""

    backend_id = "cuda_ag_rs"
    supports_autograd = True

    def __init__(self, *, process_group: Any = None, collective: Any = None) -> None:
        self._group = process_group
        self._collective = collective

    def _get_collective(self, plan: AttentionCPCommunicationPlan):
        plan.validate()
        if self._collective is None:
            from rl_kernel_b200.distributed.algorithms.collectives import TorchDistributedDeterministicCollective

            self._collective = TorchDistributedDeterministicCollective(self._group)
        c = self._collective
        if c.world != plan.parallel.cp_world_size or c.rank != plan.parallel.cp_rank:
            raise AttentionCPCommunicationUnavailable(
                f"collective is rank {c.rank} of {c.world} but the plan says CP rank {plan.parallel.cp_rank} of "
                f"{plan.parallel.cp_world_size}; pass the CP subgroup")
        return c

    def all_gather_query(self, local_q, plan, *, sequence_dim: int = 2):
        return _AllGatherSequence.apply(local_q, self._get_collective(plan), sequence_dim, False)

    def all_gather_kv(self, local_k, local_v, plan, *, sequence_dim: int = 2):
        c = self._get_collective(plan)
        # every rank's full-sequence attention uses this rank's K/V rows: their gradients add over ranks
        return (_AllGatherSequence.apply(local_k, c, sequence_dim, True),
                _AllGatherSequence.apply(local_v, c, sequence_dim, True))

    def all_gather_query_sequence_first(self, local_q, plan):
        return self.all_gather_query(local_q, plan, sequence_dim=0)

    def all_gather_kv_sequence_first(self, local_k, local_v, plan):
        return self.all_gather_kv(local_k, local_v, plan, sequence_dim=0)

    def all_gather_qkv_sequence_first(self, local_q, local_k, local_v, plan):
        k, v = self.all_gather_kv(local_k, local_v, plan, sequence_dim=0)
        return self.all_gather_query(local_q, plan, sequence_dim=0), k, v

    def all_gather_position_ids(self, local_query_positions, local_key_positions, plan):
        c = self._get_collective(plan)
        gather = lambda p: c.all_gather(p.movedim(-1, 0).contiguous()).reshape(-1, *p.shape[:-1]).movedim(0, -1)  # noqa: E731
        return gather(local_query_positions), gather(local_key_positions)

    def all_gather_partial_states(self, local_states, plan):
        c = self._get_collective(plan)
        if not plan.expected_blocks:
            raise AttentionCPCommunicationUnavailable("gathering partial states needs the expected block manifest")
        mine = sorted(local_states, key=lambda s: s.block.global_block_index)
        per_rank = {r: sorted((b for b in plan.expected_blocks if b.owner_cp_rank == r),
                              key=lambda b: b.global_block_index) for r in range(c.world)}
        if [s.block for s in mine] != per_rank[c.rank]:
            raise ValueError("local states do not match this rank's blocks in the manifest")
        counts = {len(v) for v in per_rank.values()}
        if len(counts) != 1:
            raise AttentionCPCommunicationUnavailable("the collective transport needs the same block count on every rank")
        outs = c.all_gather(torch.stack([s.out for s in mine]))          # [world, nblk, B, H, S, D]
        lses = c.all_gather(torch.stack([s.lse for s in mine]))
        got = [AttentionCPPartialState(outs[r, i], lses[r, i], b) for r in range(c.world) for i, b in enumerate(per_rank[r])]
        return sort_attention_cp_partial_states(got, plan=plan)

    def _my_rows(self, plan, total: int) -> tuple[int, int]:
        if plan.query_token_ranges:
            return plan.query_token_ranges[plan.parallel.cp_rank]
        n = total // plan.parallel.cp_world_size
        return plan.parallel.cp_rank * n, (plan.parallel.cp_rank + 1) * n

    def reduce_scatter_merged_state(self, merged_state, plan):
        merged_state.validate()
        c = self._get_collective(plan)
        s, e = self._my_rows(plan, merged_state.out.shape[2])
        return AttentionCPMergedState(_ScatterSequence.apply(merged_state.out, c, 2, s, e),
                                      _ScatterSequence.apply(merged_state.lse, c, 2, s, e))

    def reduce_scatter_strict_result(self, out, lse, plan):
        c = self._get_collective(plan)
        s, e = self._my_rows(plan, out.shape[2])
        shard = AttentionCPOutputShard(_ScatterSequence.apply(out, c, 2, s, e), _ScatterSequence.apply(lse, c, 2, s, e))
        shard.validate()
        return shard


class P2PNCCLAttentionCPCommunication:
    """Partial-state exchange by explicit send/recv in (peer, block) order; no autograd."""

    backend_id = "p2p_nccl_reference"
    supports_autograd = False

    def __init__(self, *, process_group: Any = None, dist_module: Any = None, validate_cuda_tensors: bool = True) -> None:
        if dist_module is None:
            import torch.distributed as dist_module
        self._dist = dist_module
        self._group = process_group
        self._validate_cuda_tensors = validate_cuda_tensors

    def _validate_runtime(self, plan) -> tuple[int, int]:
        plan.validate()
        if plan.backend != self.backend_id:
            raise AttentionCPCommunicationUnavailable(f"plan backend {plan.backend} is not {self.backend_id}")
        world, rank = self._dist.get_world_size(self._group), self._dist.get_rank(self._group)
        if (world, rank) != (plan.parallel.cp_world_size, plan.parallel.cp_rank):
            raise AttentionCPCommunicationUnavailable("process group does not match the plan's CP rank/world")
        return world, rank

    def _require_cuda(self, t: torch.Tensor) -> None:
        if self._validate_cuda_tensors and not t.is_cuda:
            raise AttentionCPCommunicationUnavailable("the NCCL reference transports CUDA tensors")

    def _global(self, r: int) -> int:
        return self._dist.get_global_rank(self._group, r) if self._group is not None else r

    def _exchange(self, mine: torch.Tensor, shapes: list[tuple], world: int, rank: int) -> list[torch.Tensor]:
        """Rank-ordered exchange of one tensor per rank (shapes may differ per rank)."""
        out: list[torch.Tensor] = []
        for src in range(world):
            if src == rank:
                buf = mine.contiguous()
                for dst in range(world):
                    if dst != rank:
                        self._dist.send(buf, self._global(dst), group=self._group)
            else:
                buf = torch.empty(shapes[src], dtype=mine.dtype, device=mine.device)
                self._dist.recv(buf, self._global(src), group=self._group)
            out.append(buf)
        return out

    def all_gather_query(self, local_q, plan):
        world, rank = self._validate_runtime(plan)
        self._require_cuda(local_q)
        shapes = [(*local_q.shape[:2], e - s, local_q.shape[3]) for s, e in plan.query_token_ranges]
        return torch.cat(self._exchange(local_q, shapes, world, rank), dim=2)

    def all_gather_kv(self, local_k, local_v, plan):
        world, rank = self._validate_runtime(plan)
        self._require_cuda(local_k)
        shapes = [(*local_k.shape[:2], e - s, local_k.shape[3]) for s, e in plan.query_token_ranges]
        return (torch.cat(self._exchange(local_k, shapes, world, rank), dim=2),
                torch.cat(self._exchange(local_v, shapes, world, rank), dim=2))

    def all_gather_position_ids(self, local_query_positions, local_key_positions, plan):
        world, rank = self._validate_runtime(plan)
        shapes = [(*local_query_positions.shape[:-1], e - s) for s, e in plan.query_token_ranges]
        return (torch.cat(self._exchange(local_query_positions, shapes, world, rank), dim=-1),
                torch.cat(self._exchange(local_key_positions, shapes, world, rank), dim=-1))

    def all_gather_partial_states(self, local_states, plan):
        world, rank = self._validate_runtime(plan)
        mine = sorted(local_states, key=lambda s: s.block.global_block_index)
        per_rank = {r: sorted((b for b in plan.expected_blocks if b.owner_cp_rank == r),
                              key=lambda b: b.global_block_index) for r in range(world)}
        if [s.block for s in mine] != per_rank[rank]:
            raise ValueError("local states do not match this rank's blocks in the manifest")
        for s in mine:
            self._require_cuda(s.out)
        q_shape, l_shape = mine[0].out.shape, mine[0].lse.shape
        got: list[AttentionCPPartialState] = []
        outs = self._exchange(torch.stack([s.out for s in mine]), [(len(per_rank[r]), *q_shape) for r in range(world)], world, rank)
        lses = self._exchange(torch.stack([s.lse for s in mine]), [(len(per_rank[r]), *l_shape) for r in range(world)], world, rank)
        for r in range(world):
            for i, b in enumerate(per_rank[r]):       # metadata is rebuilt from the manifest, never transported
                got.append(AttentionCPPartialState(outs[r][i], lses[r][i], b))
        return sort_attention_cp_partial_states(got, plan=plan)

    def reduce_scatter_merged_state(self, merged_state, plan):
        """The root sends every rank its query rows (explicit sends, rank order)."""
        world, rank = self._validate_runtime(plan)
        merged_state.validate()
        root = plan.merge_root_cp_rank
        s, e = plan.query_token_ranges[rank]
        if rank == root:
            for dst in range(world):
                if dst == root:
                    continue
                ds, de = plan.query_token_ranges[dst]
                self._dist.send(merged_state.out[:, :, ds:de].contiguous(), self._global(dst), group=self._group)
                self._dist.send(merged_state.lse[:, :, ds:de].contiguous(), self._global(dst), group=self._group)
            return AttentionCPMergedState(merged_state.out[:, :, s:e].contiguous(), merged_state.lse[:, :, s:e].contiguous())
        out = torch.empty(*merged_state.out.shape[:2], e - s, merged_state.out.shape[3], dtype=torch.float32,
                          device=merged_state.out.device)
        lse = torch.empty(*merged_state.lse.shape[:2], e - s, dtype=torch.float32, device=merged_state.lse.device)
        self._dist.recv(out, self._global(root), group=self._group)
        self._dist.recv(lse, self._global(root), group=self._group)
        return AttentionCPMergedState(out, lse)

    def reduce_scatter_strict_result(self, out, lse, plan):
        world, rank = self._validate_runtime(plan)
        s, e = plan.query_token_ranges[rank]
        shard = AttentionCPOutputShard(out[:, :, s:e].contiguous(), lse[:, :, s:e].contiguous())
        shard.validate()
        return shard


class PeerMemoryAttentionCPCommunication:
    """The NVLink product path: K/V stay where they are and the kernel reads them in place.

    ``attention(q, k, v, ...)`` runs ``CPAttention`` on this rank's rows; the gather / scatter methods of
    the protocol raise, because this backend has no separate communication step to call."""

    backend_id = "peer_memory"
    supports_autograd = True

    def __init__(self, *, collective: Any, device, num_q_heads: int, num_kv_heads: int, max_local_tokens: int,
                 layout: str = "zigzag") -> None:
        from rl_kernel_b200.ops.distributed import CPAttentionOp

        self.op = CPAttentionOp(collective=collective, device=device, num_q_heads=num_q_heads, num_kv_heads=num_kv_heads,
                                max_local_tokens=max_local_tokens, layout=layout)

    def plan(self, parallel: AttentionParallelSpec) -> AttentionCPCommunicationPlan:
        return AttentionCPCommunicationPlan(parallel=parallel, backend="peer_memory", pattern="in_kernel_peer_loads",
                                            compute_communication="fused")

    def attention(self, q_local, k_local, v_local, *, nseq: int, seq_len: int):
        """Packed local rows [nseq * local_len, heads * 128] in this rank's layout order -> (out, lse)."""
        return self.op(q_local, k_local, v_local, nseq=nseq, seq_len=seq_len)

    def _no(self, *_a, **_k):
        raise AttentionCPCommunicationUnavailable(
            "the peer-memory backend has no stand-alone gather/scatter: call .attention(), which reads remote K/V in the kernel")

    all_gather_query = all_gather_kv = all_gather_position_ids = all_gather_partial_states = _no
    reduce_scatter_merged_state = reduce_scatter_strict_result = _no


RCCLAGRSAttentionCPCommunication = CUDAAGRSAttentionCPCommunication      # one device family: the name is kept for imports
