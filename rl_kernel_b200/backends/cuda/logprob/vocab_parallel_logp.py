"""Contract-driven vocabulary-parallel log-prob on the device
(parity: CudaVocabParallelLogprobOp, rl_engine/backends/cuda/logprob/vocab_parallel_logp.py:21-164).

The reference op of ``rl_engine.reference.logprob.vocab_parallel_logp`` with the per-tile
statistics and the logits gradient computed by ``rlk_logits_tile_stats`` / ``rlk_dlogits`` instead of
torch reductions.  The contract decides shard bounds, masks and the determinism scope; this
backend serves bf16 logits whose shard starts on a 128-id boundary and otherwise defers to the
PyTorch op, reporting that it did.
"""
from __future__ import annotations

import torch

from rl_kernel_b200.reference.logprob.tile_logp import TILE
from rl_kernel_b200.reference.logprob.vocab_parallel_logp import VocabParallelLogprobOp, apply_with_kernels


def native_tile_stats_available() -> bool:
    if not torch.cuda.is_available():
        return False
    from rl_kernel_b200.backends import extension

    return extension.load(required=False) is not None


class _CudaKernels:
    """The two numeric kernels the contract-driven driver needs."""

    @staticmethod
    def tile_stats(shard: torch.Tensor, vocab_start: int, real_vocab: int, num_tiles: int):
        """(tile_max, tile_sum) [rows, local tiles] of a bf16 shard whose columns at or beyond the real
        vocabulary are excluded."""
        from rl_kernel_b200.backends import native as nv

        rows, vl = shard.shape
        keep = max(0, min(vl, real_vocab - vocab_start))
        nt_local = (vl + TILE - 1) // TILE
        stats = torch.empty(rows, num_tiles, 2, device=shard.device, dtype=torch.float32)
        stats[..., 0] = float("-inf")
        stats[..., 1] = 0
        tl = torch.zeros(rows, device=shard.device, dtype=torch.float32)
        if keep:
            nv.logits_tile_stats(shard[:, :keep], None, stats, tl, vocab_start=vocab_start, inv_temp=1.0)
        t0 = vocab_start // TILE
        return stats[:, t0:t0 + nt_local, 0].contiguous(), stats[:, t0:t0 + nt_local, 1].contiguous()

    @staticmethod
    def backward(shard: torch.Tensor, targets: torch.Tensor, lse: torch.Tensor, grad_logp: torch.Tensor,
                 grad_lse: torch.Tensor | None, vocab_start: int, real_vocab: int) -> torch.Tensor:
        from rl_kernel_b200.backends import native as nv

        rows, vl = shard.shape
        keep = max(0, min(vl, real_vocab - vocab_start))
        d = torch.zeros_like(shard)
        if keep:
            d[:, :keep] = shard[:, :keep]
            view = d[:, :keep]
            nv.dlogits_(view, targets.contiguous(), lse.contiguous(), grad_logp.float().contiguous(), vocab_start=vocab_start,
                        inv_temp=1.0, g_lse=None if grad_lse is None else grad_lse.float().contiguous())
        return d


class CudaVocabParallelLogprobOp(VocabParallelLogprobOp):
    backend_id = "b200-vocab-parallel-logp"

    def apply(self, local_logits, target_ids, contract, *, tp_group=None, **kw):
        usable = (native_tile_stats_available() and local_logits.is_cuda and local_logits.dtype == torch.bfloat16
                  and contract.sharding.local_vocab_start % TILE == 0 and local_logits.shape[1] % 8 == 0)
        if not usable:
            self.last_route = "pytorch"
            return super().apply(local_logits, target_ids, contract, tp_group=tp_group, **kw)
        self.last_route = "b200"
        return apply_with_kernels(local_logits, target_ids, contract, _CudaKernels, tp_group=tp_group, **kw)
