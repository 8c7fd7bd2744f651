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
    """The two numeric kernels the contract-driven driver needs (``VocabParallelLogprobKernels``)."""

    def __init__(self, temperature: float = 1.0):
        self.inv_temp = 1.0 / temperature

    def tile_stats(self, shard: torch.Tensor, vocab_start: int, real_vocab: int, num_tiles: int):
        """(tile_max, tile_sum) [rows, num_tiles] of a bf16 shard; columns at or beyond the real vocabulary are
        excluded."""
        from rl_kernel_b200.backends import native as nv

        rows, vl = shard.shape
        keep = max(0, min(vl, real_vocab - vocab_start))
        t0 = vocab_start // TILE
        stats = torch.empty(rows, t0 + num_tiles, 2, device=shard.device, dtype=torch.float32)
        stats[..., 0] = float("-inf")
        stats[..., 1] = 0
        if keep:
            tl = torch.zeros(rows, device=shard.device, dtype=torch.float32)
            nv.logits_tile_stats(shard[:, :keep], None, stats, tl, vocab_start=vocab_start, inv_temp=self.inv_temp)
        return stats[:, t0:, 0].contiguous(), stats[:, t0:, 1].contiguous()

    def backward(self, shard: torch.Tensor, lse: torch.Tensor, coef_logp: torch.Tensor, coef_lse: torch.Tensor,
                 target_local: torch.Tensor, vocab_start: int, real_vocab: int, has_lse_grad: bool) -> torch.Tensor:
        from rl_kernel_b200.backends import native as nv

        rows, vl = shard.shape
        keep = max(0, min(vl, real_vocab - vocab_start))
        d = torch.zeros_like(shard)
        if keep:
            work = shard[:, :keep].contiguous()
            # the kernel locates the target by its GLOBAL id; rows whose target lives elsewhere get an id no column has
            tg = torch.where(target_local >= 0, target_local + vocab_start, torch.full_like(target_local, -1)).contiguous()
            nv.dlogits_(work, tg, lse.contiguous(), coef_logp.contiguous(), vocab_start=vocab_start, inv_temp=self.inv_temp,
                        g_lse=coef_lse.contiguous() if has_lse_grad else None)
            d[:, :keep] = work
        return d


class CudaVocabParallelLogprobOp(VocabParallelLogprobOp):
    backend_id = "b200-vocab-parallel-logp"
    last_route = None

    def apply(self, local_logits, target_ids, *, contract, tp_group=None, num_vocab_tiles=None, validate: bool = True,
              deterministic: bool = True):
        usable = (native_tile_stats_available() and local_logits.is_cuda and local_logits.dtype == torch.bfloat16
                  and num_vocab_tiles is None and contract.numerics.tile == TILE
                  and contract.sharding.local_vocab_start % TILE == 0 and local_logits.shape[1] % 8 == 0
                  and local_logits.is_contiguous())
        if not usable:
            self.last_route = "pytorch"
            return super().apply(local_logits, target_ids, contract=contract, tp_group=tp_group,
                                 num_vocab_tiles=num_vocab_tiles, validate=validate, deterministic=deterministic)
        self.last_route = "b200"
        return apply_with_kernels(local_logits, target_ids, contract=contract, tp_group=tp_group,
                                  num_vocab_tiles=num_vocab_tiles, validate=validate,
                                  kernels=_CudaKernels(contract.numerics.temperature))

    __call__ = apply
