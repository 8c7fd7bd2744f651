"""Batch-invariant selected log-prob from materialised logits
(parity: BatchInvariantLogpSM90Op, rl_engine/backends/cuda/logprob/batch_invariant_logp.py:83-195).

bf16 logits run ``rlk_logits_tile_stats`` + ``rlk_logp_merge`` (the 128-id tile contract, one warp
per (row, tile) with a fixed in-tile order, tiles merged in ascending order), fp32 logits the same
contract evaluated with torch on the device.  Rows whose target is ``ignore_index`` return 0 and
receive no gradient.
"""
from __future__ import annotations

import torch

from rl_kernel_b200.ops.logprob import _IndexedLogpLseFn, logp_from_logits
from rl_kernel_b200.reference.logprob.tile_logp import _target_z, merge_tile_stats


def _validate_targets(logits, target_ids, ignore_index):
    vocab = logits.size(-1)
    t = target_ids.reshape(-1)
    t = t[t != ignore_index]
    if t.numel() and bool(((t < 0) | (t >= vocab)).any()):
        bad = t[(t < 0) | (t >= vocab)]
        raise ValueError(f"target_ids contains values outside [0, {vocab}): {bad.tolist()}")


def _check_shapes(logits, target_ids):
    if logits.dim() < 2:
        raise ValueError(f"logits must be at least 2-D ([*lead, V]), got shape {tuple(logits.shape)}")
    if logits.shape[:-1] != target_ids.shape:
        raise ValueError(f"logits leading shape {tuple(logits.shape[:-1])} must match target_ids shape "
                         f"{tuple(target_ids.shape)}")


class BatchInvariantLogpSM100Op:
    op_class = "reduction"
    is_batch_invariant = True
    is_fused_logp = True
    backward_impl = "native"
    backend_id = "b200"

    def __init__(self) -> None:
        pass

    def apply(self, logits, target_ids, ignore_index: int = -100, *, validate: bool = False):
        _check_shapes(logits, target_ids)
        if not logits.is_cuda:
            raise RuntimeError(f"{type(self).__name__} requires CUDA logits; a fallback to another implementation is forbidden")
        if validate:
            _validate_targets(logits, target_ids, ignore_index)
        active = target_ids != ignore_index
        safe = torch.where(active, target_ids, torch.zeros_like(target_ids))
        if logits.dtype == torch.bfloat16:
            lp = logp_from_logits(logits, safe)
        else:
            lp = self._torch_contract(logits, safe)[0]
        return torch.where(active, lp, torch.zeros_like(lp))

    __call__ = apply

    @staticmethod
    def _torch_contract(logits, targets):
        lg = logits.reshape(-1, logits.shape[-1])
        stats = _stats_on_device(lg)
        tz, _ = _target_z(lg, targets.reshape(-1), 0, 1.0)
        lp, lse = merge_tile_stats(stats, tz)
        return lp.view(targets.shape), lse.view(targets.shape)

    def forward_with_lse(self, logits, target_ids, ignore_index: int = -100, *, validate: bool = True):
        """(logp, lse), both fp32, straight from the device kernels (no gradient)."""
        _check_shapes(logits, target_ids)
        if not logits.is_cuda:
            raise RuntimeError("exact device log-prob diagnostics require CUDA logits; fallback is disabled")
        if validate:
            _validate_targets(logits, target_ids, ignore_index)
        active = target_ids != ignore_index
        safe = torch.where(active, target_ids, torch.zeros_like(target_ids))
        with torch.no_grad():
            if logits.dtype == torch.bfloat16:
                lg = logits.reshape(-1, logits.shape[-1]).contiguous()
                rows = torch.arange(lg.shape[0], device=lg.device)
                lp, lse = _IndexedLogpLseFn.apply(lg, safe.reshape(-1).contiguous(), rows, 1.0)
                lp, lse = lp.view(target_ids.shape), lse.view(target_ids.shape)
            else:
                lp, lse = self._torch_contract(logits, safe)
        return torch.where(active, lp, torch.zeros_like(lp)), lse


def _stats_on_device(lg: torch.Tensor) -> torch.Tensor:
    """The tile contract with torch ops on ``lg``'s device (fp32 / fp16 logits)."""
    from rl_kernel_b200.reference.logprob.tile_logp import tile_stats_reference

    return tile_stats_reference(lg)


BatchInvariantLogpSM90Op = BatchInvariantLogpSM100Op
