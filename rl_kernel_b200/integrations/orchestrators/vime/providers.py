"""Provider functions in the shape the vime orchestrator loads (parity:
rl_engine/integrations/orchestrators/vime/providers/{attention,linear_logp_provider,logp}.py): each
returns the strict operator for its module, bound to the parallel layout of the calling worker."""
from __future__ import annotations

from rl_kernel_b200.integrations.common.linear_logp import LinearLogpWrapper
from rl_kernel_b200.runtime.registry import kernel_registry


def linear_logp_provider(temperature: float = 1.0, real_vocab: int | None = None, tp_group=None, vocab_start: int = 0,
                         padded_vocab: int | None = None) -> LinearLogpWrapper:
    return LinearLogpWrapper(temperature, real_vocab, tp_group, vocab_start, padded_vocab)


def logp_provider(backend: str = "batch_invariant", temperature: float = 1.0):
    return kernel_registry.get_logprob_op(backend, temperature=temperature)


def attention_provider(contract=None):
    return kernel_registry.get_attention_op("b200" if contract is not None and contract.sharding.cp_size > 1 else "auto",
                                            contract=contract)


def ffn_provider(canonical_tp: int = 8, tp_size: int = 1, collective=None):
    return kernel_registry.get_op("ffn", canonical_tp=canonical_tp, tp_size=tp_size, collective=collective)
