"""Operator bridge: one call that resolves the selected-log-prob operator for an integration and
records the execution (parity: OperatorBridge / selected_logprobs_with_operator,
rl_engine/runtime/operators.py:105-307)."""
from __future__ import annotations

import torch

from rl_kernel_b200.runtime.registry import kernel_registry
from rl_kernel_b200.runtime.semantic_registry import OperatorSession, semantic_catalog


class OperatorBridge:
    def __init__(self, session: OperatorSession | None = None, temperature: float = 1.0):
        self.session = session or semantic_catalog.session("bridge")
        self.temperature = temperature

    def selected_logprobs(self, *, logits: torch.Tensor | None = None, hidden: torch.Tensor | None = None,
                          lm_head_weight: torch.Tensor | None = None, token_ids: torch.Tensor,
                          mask: torch.Tensor | None = None, module: str = "") -> torch.Tensor:
        if (logits is None) == (hidden is None):
            raise ValueError("give exactly one of logits / hidden")
        if hidden is not None:
            if lm_head_weight is None:
                raise ValueError("hidden input needs lm_head_weight")
            op = kernel_registry.get_op("linear_logp", temperature=self.temperature)
            lp = op(hidden, lm_head_weight, token_ids)
        else:
            op = kernel_registry.get_op("batch_invariant_logp", temperature=self.temperature)
            lp = op(logits, token_ids)
        res = kernel_registry.last_resolution
        backend = "reference" if res.actual.name.startswith("REF") else "b200-tcgen05"
        self.session.observe("selected_logprob", backend, module, res.fallback)
        return lp if mask is None else lp.masked_fill(~mask.bool(), 0.0)


def selected_logprobs_with_operator(logits, token_ids, mask=None, temperature: float = 1.0):
    return OperatorBridge(temperature=temperature).selected_logprobs(logits=logits, token_ids=token_ids, mask=mask)
