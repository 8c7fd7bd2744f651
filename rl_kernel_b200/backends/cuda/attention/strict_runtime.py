"""Framework-neutral strict attention runtime (parity: StrictCUDAAttentionRuntime,
rl_engine/backends/cuda/attention/strict_runtime.py:35-544).

A framework binding hands over its local Q/K/V [B, H, S_local, D], the logical position of every
local token and the ``AttentionContract``; the runtime returns this rank's output rows and fp32
LSE plus provenance.  One arithmetic identity at every CP degree:

* CP = 1: the core runs on the local tensors.
* CP > 1 with a ``PeerMemoryAttentionCPCommunication``: the kernel reads the other ranks' K/V over
  NVLink while computing this rank's rows only (the product path; no redundant compute).
* CP > 1 with a gather/scatter communication object: all-gather(Q, K, V, positions) in rank order,
  sort by logical position, run the core on the full sequence, return the rows this rank owns.
  This is the reference's graph; it is kept because it runs on any transport (Gloo included) and
  defines the expected bits.

The core is any object with ``core_id`` / ``strict_schedule`` and ``__call__(q, k, v, causal=,
key_padding_mask=, return_lse=)`` on [B, S, H, D] tensors: ``StrictFlashAttention4Core`` on a B200,
the PyTorch ``NativeAttentionOp`` wrapped by ``ReferenceAttentionCore`` elsewhere.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from rl_kernel_b200.backends.cuda.attention.cp_comm import (AttentionCPCommunicationPlan, AttentionParallelSpec,
                                                            CUDAAGRSAttentionCPCommunication,
                                                            PeerMemoryAttentionCPCommunication)
from rl_kernel_b200.backends.cuda.attention.permutation import permute_sequence
from rl_kernel_b200.contracts.operators.attention import (STRICT_ATTENTION_PRODUCTION_CORE_ID,
                                                           STRICT_ATTENTION_SCHEDULE_ID, AttentionContract)


@dataclass(frozen=True)
class StrictCUDAAttentionResult:
    out: torch.Tensor
    lse: torch.Tensor
    provenance: dict[str, Any]


class ReferenceAttentionCore:
    """The PyTorch gold attention behind the core interface (CPU tests, non-B200 machines)."""
    core_id = STRICT_ATTENTION_PRODUCTION_CORE_ID
    strict_schedule = STRICT_ATTENTION_SCHEDULE_ID

    def __call__(self, q, k, v, *, causal=True, key_padding_mask=None, return_lse=False):
        from rl_kernel_b200.reference.attention.standard_attn import NativeAttentionOp

        return NativeAttentionOp()(q, k, v, causal=causal, key_padding_mask=key_padding_mask, return_lse=return_lse)


class StrictCUDAAttentionRuntime:
    backend_id = "rlkernel.b200.attention.canonical_blocks.v1"
    core_id = STRICT_ATTENTION_PRODUCTION_CORE_ID
    strict_schedule = STRICT_ATTENTION_SCHEDULE_ID

    def __init__(self, *, process_group: Any = None, core: Any | None = None, communication: Any | None = None) -> None:
        if core is None:
            from rl_kernel_b200.backends.cuda.attention.flash_attn import StrictFlashAttention4Core

            core = StrictFlashAttention4Core()
            core.strict_schedule = core.schedule
        self._core = core
        self._communication = communication if communication is not None else CUDAAGRSAttentionCPCommunication(
            process_group=process_group)
        if getattr(core, "core_id", None) != self.core_id:
            raise RuntimeError("the strict attention runtime requires the production core")
        if getattr(core, "strict_schedule", None) != self.strict_schedule:
            raise RuntimeError("the strict attention runtime requires the canonical fixed schedule")
        self.communication_executed = False
        self._layout_cache: dict[tuple, tuple[torch.Tensor, ...]] = {}

    @staticmethod
    def _validate_local_positions(q, k, qpos, kpos) -> None:
        if q.dim() != 4 or k.dim() != 4:
            raise ValueError("q and k must be [B, H, S, D]")
        if qpos.shape != (q.shape[0], q.shape[2]) or kpos.shape != (k.shape[0], k.shape[2]):
            raise ValueError("position ids must be [B, S_local] for queries and keys")
        if bool((qpos < 0).any()) or bool((kpos < 0).any()):
            raise ValueError("logical positions must be non-negative")

    def _position_layout(self, qpos, kpos, plan):
        key = (qpos.data_ptr(), int(qpos._version), kpos.data_ptr(), int(kpos._version), tuple(qpos.shape), tuple(kpos.shape),
               plan.parallel.cp_rank, plan.parallel.cp_world_size)
        hit = self._layout_cache.get(key)
        if hit is not None:
            return hit
        gq, gk = self._communication.all_gather_position_ids(qpos, kpos, plan)
        q_sort, k_sort = torch.argsort(gq, dim=1), torch.argsort(gk, dim=1)
        value = (torch.gather(gq, 1, q_sort), torch.gather(gk, 1, k_sort), q_sort, k_sort, torch.argsort(q_sort, dim=1))
        if len(self._layout_cache) >= 128:
            self._layout_cache.pop(next(iter(self._layout_cache)))
        self._layout_cache[key] = value
        return value

    def _run_core(self, q, k, v, causal: bool):
        """[B, H, S, D] in, ([B, H, S, D], [B, H, S]) out."""
        o, lse = self._core(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), causal=causal, return_lse=True)
        return o.transpose(1, 2), lse.transpose(1, 2)

    def forward_with_lse(self, q, k, v, *, contract: AttentionContract, causal: bool, scale: float | None, cp_world_size: int,
                         query_position_ids: torch.Tensor, key_position_ids: torch.Tensor,
                         positions_are_sorted: bool = False) -> StrictCUDAAttentionResult:
        if cp_world_size != contract.sharding.cp_world_size:
            raise RuntimeError("runtime CP world size does not match AttentionContract")
        if scale is not None and abs(scale * (q.shape[-1] ** 0.5) - 1.0) > 1e-6:
            raise ValueError("the strict core uses the 1/sqrt(head_dim) scale")
        self._validate_local_positions(q, k, query_position_ids, key_position_ids)
        prov = {"backend_id": self.backend_id, "core_id": self.core_id, "strict_schedule": self.strict_schedule,
                "cp_world_size": cp_world_size, "contract_fingerprint": contract.cross_rank_fingerprint()}
        if cp_world_size == 1:
            if not positions_are_sorted:
                order = torch.argsort(query_position_ids[0])
                if not torch.equal(order, torch.arange(order.numel(), device=order.device)):
                    raise ValueError("CP=1 inputs must be in logical position order")
            o, lse = self._run_core(q, k, v, causal)
            return StrictCUDAAttentionResult(o, lse, {**prov, "communication": "none"})
        parallel = AttentionParallelSpec(contract.sharding.tp_world_size, contract.sharding.tp_rank, cp_world_size,
                                         contract.sharding.cp_rank)
        if isinstance(self._communication, PeerMemoryAttentionCPCommunication):
            B, H, S_loc, D = q.shape
            flat = lambda t: t.transpose(1, 2).reshape(B * S_loc, -1).contiguous()           # noqa: E731
            o, lse = self._communication.attention(flat(q), flat(k), flat(v), nseq=B, seq_len=S_loc * cp_world_size)
            self.communication_executed = True
            plan = self._communication.plan(parallel)
            return StrictCUDAAttentionResult(o.view(B, S_loc, H, D).transpose(1, 2), lse.view(B, S_loc, H).transpose(1, 2),
                                             {**prov, **plan.provenance()})
        plan = AttentionCPCommunicationPlan(parallel=parallel, backend="cuda_ag_rs")
        _qs, _ks, q_sort, k_sort, inv_q = self._position_layout(query_position_ids, key_position_ids, plan)
        gq = self._communication.all_gather_query(q, plan)
        gk, gv = self._communication.all_gather_kv(k, v, plan)
        self.communication_executed = True
        if not torch.equal(q_sort, q_sort[:1].expand_as(q_sort)) or not torch.equal(k_sort, k_sort[:1].expand_as(k_sort)):
            raise ValueError("every sequence of the batch must use the same CP token layout")
        gq = permute_sequence(gq, q_sort[0], sequence_dim=2)
        gk = permute_sequence(gk, k_sort[0], sequence_dim=2)
        gv = permute_sequence(gv, k_sort[0], sequence_dim=2)
        o, lse = self._run_core(gq, gk, gv, causal)
        o = permute_sequence(o, inv_q[0], sequence_dim=2)                                  # back to gathered (rank) order
        lse = permute_sequence(lse, inv_q[0], sequence_dim=2)
        half = o.dtype in (torch.bfloat16, torch.float16)
        shard = self._communication.reduce_scatter_strict_result(o, lse, plan) if half else None
        if shard is None:                                                                  # fp32 reference core
            n = q.shape[2]
            r = parallel.cp_rank
            out, l = o[:, :, r * n:(r + 1) * n], lse[:, :, r * n:(r + 1) * n]
        else:
            out, l = shard.out, shard.lse
        return StrictCUDAAttentionResult(out, l, {**prov, **plan.provenance()})

    def __call__(self, q, k, v, **kw) -> torch.Tensor:
        return self.forward_with_lse(q, k, v, **kw).out
