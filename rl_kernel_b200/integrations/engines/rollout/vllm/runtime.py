"""vLLM-style rollout binding (parity: rl_engine/integrations/engines/rollout/vllm/runtime.py:
587-1966).  ``install_vllm_integration`` patches the given model classes — passed in explicitly so
that stand-in classes work — to route RMSNorm, the QKV/O projections, the FFN, attention and
``compute_logits`` + sampling through the deterministic operators, according to the plan.
``register_vllm_plugin`` is the entry point vLLM's plugin loader calls."""
from __future__ import annotations

import os

import torch

from rl_kernel_b200.integrations.common.runtime import FrameworkOperatorIntegration
from rl_kernel_b200.integrations.engines.rollout.vllm.operators import (VllmAttentionOperator, VllmFFNOperator,
                                                                         VllmLogpOperator)
from rl_kernel_b200.runtime.plan import IntegrationPlan

_STATE: dict = {}


def _patch_method(cls, name, fn):
    orig = getattr(cls, name, None)
    setattr(cls, f"_rlk_orig_{name}", orig)
    setattr(cls, name, fn)
    return orig


def install_vllm_integration(*, decoder_layer_cls=None, attention_cls=None, mlp_cls=None, rmsnorm_cls=None,
                             model_cls=None, sampler_cls=None, plan: IntegrationPlan | None = None,
                             tp_size: int = 1, collective=None, temperature: float | None = None,
                             real_vocab: int | None = None) -> FrameworkOperatorIntegration:
    plan = plan or IntegrationPlan.from_env()
    integ = FrameworkOperatorIntegration("vllm", "rollout", plan)
    want = plan.side("rollout")
    temperature = temperature if temperature is not None else float(os.environ.get("RL_KERNEL_VLLM_TEMPERATURE", "1.0"))
    real_vocab = real_vocab or (int(os.environ["RL_KERNEL_VLLM_REAL_VOCAB_SIZE"])
                                if "RL_KERNEL_VLLM_REAL_VOCAB_SIZE" in os.environ else None)
    if want["attention"] and attention_cls is not None:
        op = VllmAttentionOperator()
        integ.install("attention", op)

        def attn_forward(self, q, k, v, kv_cache=None, positions=None, **kw):
            return integ.execute("attention", self, q, k, v, kv_cache=kv_cache, positions=positions, **kw)

        _patch_method(attention_cls, "forward", attn_forward)
    if want["ffn"] and mlp_cls is not None:
        op = VllmFFNOperator(tp_size=tp_size, collective=collective)
        integ.install("ffn", op)

        def mlp_forward(self, x):
            return integ.execute("ffn", self, x)

        _patch_method(mlp_cls, "forward", mlp_forward)
    if want["logp"] and model_cls is not None:
        op = VllmLogpOperator(temperature=temperature, real_vocab=real_vocab)
        integ.install("logp", op)

        def compute_logits(self, hidden_states, *a, **kw):
            # publish what the sampler needs to recompute the sampled token's log-prob with the same
            # strict operator as the trainer (parity: publish_rollout_linear_logp_context)
            _STATE["linear_logp_context"] = {"hidden": hidden_states, "lm_head": self.lm_head.weight,
                                             "real_vocab": real_vocab}
            orig = getattr(type(self), "_rlk_orig_compute_logits")
            return orig(self, hidden_states, *a, **kw)

        _patch_method(model_cls, "compute_logits", compute_logits)
        if sampler_cls is not None:
            def sampler_forward(self, logits, sampling_metadata=None, **kw):
                orig = getattr(type(self), "_rlk_orig_forward")
                out = orig(self, logits, sampling_metadata, **kw)
                ctx = _STATE.get("linear_logp_context")
                ids = getattr(out, "sampled_token_ids", out)
                if ctx is not None and isinstance(ids, torch.Tensor):
                    lp = integ.execute("logp", ctx["hidden"], ctx["lm_head"], ids.reshape(-1))
                    try:
                        out.rl_kernel_logprobs = lp
                    except AttributeError:
                        _STATE["last_logprobs"] = lp
                return out

            _patch_method(sampler_cls, "forward", sampler_forward)
    if rmsnorm_cls is not None and (want["attention"] or want["ffn"]):
        from rl_kernel_b200.ops.norm import rms_norm

        def norm_forward(self, x, residual=None):
            eps = getattr(self, "variance_epsilon", getattr(self, "eps", 1e-6))
            if residual is not None:
                x = (x.float() + residual.float()).to(x.dtype)
                return rms_norm(x, self.weight, eps), x
            return rms_norm(x, self.weight, eps)

        _patch_method(rmsnorm_cls, "forward", norm_forward)
        _patch_method(rmsnorm_cls, "forward_native", norm_forward)
    _STATE["integration"] = integ
    return integ


def last_rollout_logprobs():
    return _STATE.get("last_logprobs")


def register_vllm_plugin() -> None:
    """Entry point for ``vllm.general_plugins``: installs on the real Qwen3 classes when
    RL_KERNEL_VLLM_INTEGRATION=1 (parity: runtime.py:1961-1966)."""
    if os.environ.get("RL_KERNEL_VLLM_INTEGRATION", "0") not in ("1", "true", "True"):
        return
    from vllm.model_executor.layers.layernorm import RMSNorm  # noqa: PLC0415
    from vllm.model_executor.models import qwen3 as q3  # noqa: PLC0415

    install_vllm_integration(decoder_layer_cls=q3.Qwen3DecoderLayer, attention_cls=q3.Qwen3Attention,
                             mlp_cls=getattr(q3, "Qwen3MLP", None), rmsnorm_cls=RMSNorm, model_cls=q3.Qwen3ForCausalLM)
