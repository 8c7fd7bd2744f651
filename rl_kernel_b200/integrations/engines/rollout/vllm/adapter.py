"""vLLM-side integration object (parity: VllmIntegration, rl_engine/integrations/engines/rollout/vllm/adapter.py:15-39)."""
from __future__ import annotations

from rl_kernel_b200.integrations.common.runtime import FrameworkOperatorIntegration


class VllmIntegration(FrameworkOperatorIntegration):
    def __init__(self, plan=None, *, rl_kernel_operators=None):
        super().__init__("vllm", "rollout", plan)
        for module, op in (rl_kernel_operators or {}).items():
            self.install(module, op)

    def attention(self, *args, **kwargs):
        return self.execute("attention", *args, **kwargs)

    def ffn(self, *args, **kwargs):
        return self.execute("ffn", *args, **kwargs)

    def logp(self, *args, **kwargs):
        return self.execute("logp", *args, **kwargs)


__all__ = ["VllmIntegration"]
