"""Qwen3 SwiGLU FFN device operator with the reference's call shape (parity: qwen3_ffn / Qwen3FFNOp /
qwen3_ffn_packed_inference, rl_engine/backends/cuda/ffn/ffn.py:211-1083).

``qwen3_ffn(rmsnorm_output, gate_weight, up_weight, down_weight, *, fused_gate_up_weight, tp_group,
cp_group, sequence_parallel)``: gate / up are column-parallel, down is row-parallel.  The three GEMMs
run on the tcgen05 kernel; gate|up is one launch over the block-interleaved packed weight (packed
here when the caller holds separate tensors, cached per weight version), SwiGLU is its own kernel in
training and the GEMM's epilogue in ``packed_inference``; the down projection sums 8 canonical K
chunks in a fixed tree that the tensor-parallel all-reduce (or reduce-scatter, under sequence
parallelism) finishes, so TP = 1, 2, 4, 8 give the same bits.
"""
from __future__ import annotations

from typing import Any, Callable

import torch
from torch import Tensor

from rl_kernel_b200.ops.ffn.qwen3 import qwen3_ffn as _ffn

BACKEND_ID = "rlkernel.b200.qwen3_ffn.tcgen05.v1"
CANONICAL_TP = 8
_OBSERVERS: list[Callable[[], None]] = []
_PACK_CACHE: dict[tuple, Tensor] = {}


def register_packed_inference_observer(callback: Callable[[], None]) -> None:
    """``callback()`` runs on every packed-inference call (the rollout runtime counts them for its readback)."""
    _OBSERVERS.append(callback)


def _collective(tp_group: Any):
    if tp_group is None:
        return None, 1
    if hasattr(tp_group, "all_reduce") and hasattr(tp_group, "world"):
        return (tp_group if tp_group.world > 1 else None), tp_group.world
    import torch.distributed as dist

    from rl_kernel_b200.distributed.algorithms.collectives import collective_for_group

    world = dist.get_world_size(tp_group) if dist.is_initialized() else 1
    return (collective_for_group(tp_group) if world > 1 else None), world


def _packed_gate_up(gate: Tensor, up: Tensor, fused: Tensor | None, blk: int) -> Tensor:
    """[2I, H] with gate / up rows interleaved in blocks of ``blk`` (one block pair per canonical shard)."""
    key = (gate.data_ptr(), up.data_ptr(), gate._version, up._version, blk)
    if not (gate.requires_grad or up.requires_grad) and key in _PACK_CACHE:
        return _PACK_CACHE[key]
    I, H = gate.shape
    packed = torch.stack([gate.view(I // blk, blk, H), up.view(I // blk, blk, H)], dim=1).reshape(2 * I, H)
    if not (gate.requires_grad or up.requires_grad):
        _PACK_CACHE.clear()
        _PACK_CACHE[key] = packed
    return packed


def qwen3_ffn(rmsnorm_output: Tensor, gate_weight: Tensor, up_weight: Tensor, down_weight: Tensor, *,
              fused_gate_up_weight: Tensor | None = None, tp_group: Any = None, cp_group: Any = None,
              sequence_parallel: bool = False, deterministic: bool | None = None, disable_split_k: bool | None = None) -> Tensor:
    """Bias-free SiLU-gated FFN, differentiable in the activations and all three weights.  ``cp_group`` only has to
    be consistent (context parallelism does not touch the FFN); ``deterministic`` / ``disable_split_k`` cannot be
    turned off."""
    del cp_group
    if deterministic is False or disable_split_k is False:
        raise ValueError("the FFN kernels have one deterministic schedule without a K split; it cannot be disabled")
    if fused_gate_up_weight is not None:
        I = fused_gate_up_weight.shape[0] // 2
        gate_weight, up_weight = fused_gate_up_weight[:I], fused_gate_up_weight[I:]
    coll, world = _collective(tp_group)
    if CANONICAL_TP % world:
        raise ValueError(f"tensor-parallel degree {world} must divide the canonical {CANONICAL_TP}")
    nchunks = CANONICAL_TP // world
    if gate_weight.shape[0] % nchunks:
        raise ValueError(f"local intermediate size {gate_weight.shape[0]} must split into {nchunks} canonical shards")
    blk = gate_weight.shape[0] // nchunks
    w_gu = _packed_gate_up(gate_weight, up_weight, fused_gate_up_weight, blk)
    return _ffn(rmsnorm_output, w_gu, down_weight, canonical_tp=CANONICAL_TP, tp_size=world, collective=coll,
                sequence_parallel=sequence_parallel)


@torch.no_grad()
def qwen3_ffn_packed_inference(rmsnorm_output: Tensor, fused_gate_up_weight: Tensor, down_weight: Tensor, *,
                               tp_group: Any = None, packed_blk: int | None = None) -> Tensor:
    """Rollout form: SwiGLU runs in the gate|up GEMM's epilogue (the [T, 2I] tensor is never written).
    ``fused_gate_up_weight`` is [gate; up] stacked unless ``packed_blk`` says it is already block-interleaved."""
    from rl_kernel_b200.backends import native as nv

    for cb in _OBSERVERS:
        cb()
    coll, world = _collective(tp_group)
    nchunks = CANONICAL_TP // world
    I = fused_gate_up_weight.shape[0] // 2
    blk = packed_blk or I // nchunks
    w_gu = fused_gate_up_weight if packed_blk else _packed_gate_up(fused_gate_up_weight[:I], fused_gate_up_weight[I:], None, blk)
    x = rmsnorm_output.reshape(-1, rmsnorm_output.shape[-1]).contiguous()
    act = torch.empty(x.shape[0], I, device=x.device, dtype=x.dtype)
    nv.det_gemm_swiglu(x, w_gu.contiguous(), act, blk)
    y = torch.empty(x.shape[0], down_weight.shape[0], device=x.device, dtype=x.dtype)
    nv.det_gemm(act, down_weight.contiguous(), y, M=x.shape[0], N=down_weight.shape[0], K=I, nchunks=nchunks)
    if coll is not None:
        coll.all_reduce_(y)
    return y.reshape(*rmsnorm_output.shape[:-1], down_weight.shape[0])


class Qwen3FFNOp:
    op_class = "ffn"
    is_batch_invariant = True
    backend_id = BACKEND_ID
    backward_impl = "native"

    def __init__(self) -> None:
        self._prepared: dict[int, tuple[int, int]] = {}

    def prepare_packed_inference(self, fused_gate_up_weight: Tensor, down_weight: Tensor, *, tp_group: Any) -> tuple[int, int]:
        """Build the tensor-parallel collective before any graph capture; returns (intermediate, hidden) sizes."""
        _collective(tp_group)
        shape = (fused_gate_up_weight.shape[0] // 2, down_weight.shape[0])
        self._prepared[id(fused_gate_up_weight)] = shape
        return shape

    def packed_inference(self, rmsnorm_output: Tensor, fused_gate_up_weight: Tensor, down_weight: Tensor, *,
                         tp_group: Any = None, packed_blk: int | None = None) -> Tensor:
        return qwen3_ffn_packed_inference(rmsnorm_output, fused_gate_up_weight, down_weight, tp_group=tp_group,
                                          packed_blk=packed_blk)

    def apply(self, rmsnorm_output, gate_weight, up_weight, down_weight, **kw) -> Tensor:
        return qwen3_ffn(rmsnorm_output, gate_weight, up_weight, down_weight, **kw)

    __call__ = apply
