"""Providers the vime orchestrator loads by import path (parity: rl_engine/integrations/orchestrators/vime/providers/
__init__.py).  Each submodule exposes ``provider(request)`` over structural request / result objects; the factory helpers
below return the strict operator objects for workers that bind them once instead of per request."""
from __future__ import annotations

from rl_kernel_b200.integrations.orchestrators.vime.providers import attention, linear_logp_provider, logp  # noqa: F401
from rl_kernel_b200.integrations.orchestrators.vime.providers.attention import (AttentionProviderResult,  # noqa: F401
                                                                                AttentionProviderUnavailable, attention_provider)
from rl_kernel_b200.integrations.orchestrators.vime.providers.linear_logp_provider import (LinearLogpProviderUnavailable,  # noqa: F401
                                                                                           LinearLogpResult)
from rl_kernel_b200.integrations.orchestrators.vime.providers.logp import ProviderResult, SelectedLogprobProviderUnavailable  # noqa: F401


def linear_logp_operator(temperature: float = 1.0, real_vocab: int | None = None, tp_group=None, vocab_start: int = 0,
                         padded_vocab: int | None = None):
    from rl_kernel_b200.integrations.common.linear_logp import LinearLogpWrapper

    return LinearLogpWrapper(temperature, real_vocab, tp_group, vocab_start, padded_vocab)


def logp_operator(backend: str = "batch_invariant", temperature: float = 1.0):
    from rl_kernel_b200.runtime.registry import kernel_registry

    return kernel_registry.get_logprob_op(backend, temperature=temperature)


def attention_operator(contract=None):
    from rl_kernel_b200.runtime.registry import kernel_registry

    return kernel_registry.get_attention_op("b200" if contract is not None and contract.sharding.cp_world_size > 1 else "auto",
                                            contract=contract)


def ffn_operator(canonical_tp: int = 8, tp_size: int = 1, collective=None):
    from rl_kernel_b200.runtime.registry import kernel_registry

    return kernel_registry.get_op("ffn", canonical_tp=canonical_tp, tp_size=tp_size, collective=collective)


__all__ = ["AttentionProviderResult", "AttentionProviderUnavailable", "LinearLogpProviderUnavailable", "LinearLogpResult", "ProviderResult",
           "SelectedLogprobProviderUnavailable", "attention", "attention_operator", "attention_provider", "ffn_operator",
           "linear_logp_operator", "linear_logp_provider", "logp", "logp_operator"]
