"""Stateless forward executor: scores sequences with a frozen policy (reference / reward scoring)
without any KV cache, in micro-batches, and reports metrics (parity: StatelessForwardExecutor,
rl_engine/runtime/executor.py:95-272)."""
from __future__ import annotations

import time
from dataclasses import dataclass, field

import torch


@dataclass
class ScoreMetrics:
    sequences: int = 0
    tokens: int = 0
    seconds: float = 0.0
    micro_batches: int = 0
    backend: str = ""
    extra: dict = field(default_factory=dict)

    @property
    def tokens_per_s(self) -> float:
        return self.tokens / self.seconds if self.seconds > 0 else 0.0


class StatelessForwardExecutor:
    """``model`` is anything with ``forward(input_ids, target_ids=...) -> {"selected_logp": ...}``
    (the reference model) or a ``score(tokens) -> logp`` callable (the sm_100a trainer)."""

    def __init__(self, model, micro_batch: int = 8, reject_kv_cache: bool = True):
        self.model, self.micro_batch, self.reject_kv_cache = model, micro_batch, reject_kv_cache
        self.metrics = ScoreMetrics(backend=type(model).__name__)

    @torch.no_grad()
    def score(self, input_ids: torch.Tensor, loss_mask: torch.Tensor | None = None, **kwargs) -> torch.Tensor:
        if self.reject_kv_cache and kwargs.get("kv_cache") is not None:
            raise ValueError("the stateless executor scores without a KV cache")
        t0 = time.perf_counter()
        outs = []
        for b0 in range(0, input_ids.shape[0], self.micro_batch):
            ids = input_ids[b0:b0 + self.micro_batch]
            if callable(getattr(self.model, "score", None)):
                lp = self.model.score(ids)
            else:
                lp = self.model.forward(ids, target_ids=ids, return_logits=False)["selected_logp"]
            outs.append(lp)
            self.metrics.micro_batches += 1
        out = torch.cat(outs)
        if loss_mask is not None:
            out = out.masked_fill(~loss_mask[:, -out.shape[1]:].bool(), 0.0)
        if out.is_cuda:
            torch.cuda.synchronize(out.device)
        self.metrics.sequences += input_ids.shape[0]
        self.metrics.tokens += input_ids.numel()
        self.metrics.seconds += time.perf_counter() - t0
        return out


def score_reference_logprobs(model, input_ids, loss_mask=None, micro_batch: int = 8) -> torch.Tensor:
    return StatelessForwardExecutor(model, micro_batch).score(input_ids, loss_mask)
