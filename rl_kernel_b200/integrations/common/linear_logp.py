"""Wrapper that gives frameworks one object for "hidden states -> selected log-probs" with the
strict operator, temperature, optional vocab parallelism and top-p replay thresholds (parity:
LinearLogpWrapper, rl_engine/integrations/common/linear_logp.py:296)."""
from __future__ import annotations

import torch

from rl_kernel_b200.contracts.operators.logprob import LogprobContract, VocabShardingSpec
from rl_kernel_b200.ops.logprob import linear_logp
from rl_kernel_b200.reference.logprob.tile_logp import VocabParallelLogprobOp


class LinearLogpWrapper:
    backend_id = "b200-tcgen05"

    def __init__(self, temperature: float = 1.0, real_vocab: int | None = None, tp_group=None, vocab_start: int = 0,
                 padded_vocab: int | None = None):
        self.temperature, self.real_vocab = temperature, real_vocab
        self.tp_group, self.vocab_start, self.padded_vocab = tp_group, vocab_start, padded_vocab
        tp = 1
        if tp_group is not None:
            import torch.distributed as dist

            tp = dist.get_world_size(tp_group)
        self.vocab = VocabShardingSpec(
            tp_size=tp, real_vocab=real_vocab or (padded_vocab or 128), padded_vocab=padded_vocab or
            ((real_vocab or 128) + 128 * tp - 1) // (128 * tp) * (128 * tp))
        self.tp_rank = vocab_start // (self.vocab.padded_vocab // tp) if tp > 1 else 0
        self.contract = None          # built for the first batch (the token count is part of the contract)
        self._checked = False

    def contract_for(self, num_tokens: int, mask=None) -> LogprobContract:
        return LogprobContract.for_tokens(num_tokens, real_vocab_size=self.vocab.real_vocab,
                                          padded_vocab_size=self.vocab.padded_vocab, tp_rank=self.tp_rank,
                                          tp_world_size=self.vocab.tp_size, temperature=self.temperature, active_mask=mask)

    def __call__(self, hidden: torch.Tensor, lm_head_weight: torch.Tensor, token_ids: torch.Tensor,
                 mask: torch.Tensor | None = None) -> torch.Tensor:
        if not self._checked:
            self.contract = self.contract_for(token_ids.numel(), mask)
            self.contract.preflight(self.tp_group)
            self._checked = True
        w = lm_head_weight if self.real_vocab is None or self.tp_group is not None else lm_head_weight[: self.real_vocab]
        if self.tp_group is None:
            lp = linear_logp(hidden, w, token_ids, self.temperature)
        else:
            op = VocabParallelLogprobOp(self.temperature, self.tp_group)
            real_local = max(0, min(w.shape[0], (self.real_vocab or 10 ** 12) - self.vocab_start))
            lp = op(hidden.reshape(-1, hidden.shape[-1]), w[:real_local], token_ids.reshape(-1),
                    vocab_start=self.vocab_start, n_tiles_total=self.vocab.num_tiles).view(token_ids.shape)
        return lp if mask is None else lp.masked_fill(~mask.bool(), 0.0)
