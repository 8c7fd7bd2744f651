"""vLLM-style rollout binding (parity: rl_engine/integrations/engines/rollout/vllm/runtime.py:587-1974).

``install_vllm_integration`` patches the given classes -- passed in explicitly, so stand-in classes
work as well as vLLM's -- to route RMSNorm (with the fused residual add), the FFN, attention over the
block KV cache, and ``compute_logits`` + sampling through the deterministic operators, according to
the integration plan.  ``patch_lm_head_padding`` gives the LM head the trainer's padded vocabulary
layout (one contiguous padded range split evenly over TP, padding rows zero) so that vocabulary
shards line up with the trainer's at every TP degree.  ``register_vllm_plugin`` is the entry point
vLLM's plugin loader calls: it files the attention backend and installs the patches on the real
Qwen3 classes when ``RL_KERNEL_VLLM_INTEGRATION=1``.
"""
from __future__ import annotations

import os
from typing import Any

import torch

from rl_kernel_b200.integrations.common.runtime import FrameworkOperatorIntegration
from rl_kernel_b200.integrations.engines.rollout.vllm.operators import (VllmAttentionOperator, VllmFFNOperator,
                                                                         VllmLogpOperator)
from rl_kernel_b200.integrations.engines.rollout.vllm.sampling_support import capture_support, support_to_threshold
from rl_kernel_b200.runtime.plan import IntegrationPlan

_STATE: dict = {}
_PATCH_MARKER = "__rl_kernel_original_init__"


def _patch_method(cls, name, fn):
    orig = getattr(cls, name, None)
    if not hasattr(cls, f"_rlk_orig_{name}"):                 # a second install keeps the true original
        setattr(cls, f"_rlk_orig_{name}", orig)
    setattr(cls, name, fn)
    return orig


def fused_add_rms_norm(x: torch.Tensor, residual: torch.Tensor | None, weight: torch.Tensor, eps: float):
    """``(rmsnorm(x + residual) * weight, x + residual)`` in one kernel pass: the sum is rounded to bf16 once, written
    as the new residual and normalised from registers.  Without a residual only the norm runs."""
    if x.is_cuda and x.dtype == torch.bfloat16:
        from rl_kernel_b200.backends import native as nv

        lead = x.shape
        x2 = x.reshape(-1, lead[-1]).contiguous()
        y = torch.empty_like(x2)
        if residual is None:
            nv.rmsnorm_fwd(x2, weight.contiguous(), y, eps)
            return y.view(lead)
        r2 = residual.reshape(-1, lead[-1]).contiguous()
        new_res = torch.empty_like(x2)
        nv.rmsnorm_fwd(x2, weight.contiguous(), y, eps, res=r2, res_out=new_res)
        return y.view(lead), new_res.view(lead)
    from rl_kernel_b200.ops.norm import rms_norm

    if residual is None:
        return rms_norm(x, weight, eps)
    s = (x.float() + residual.float()).to(x.dtype)
    return rms_norm(s, weight, eps), s


def patch_lm_head_padding(parallel_lm_head_cls, vocab_embedding_cls, *, real_vocab: int, padded_vocab: int) -> None:
    """Make the engine's tensor-parallel LM-head partition the trainer's padded layout.

    The head is built over ``padded_vocab`` rows as ONE contiguous range (no separate "added vocabulary" segment), so
    rank r of TP owns rows [r * padded / tp, (r + 1) * padded / tp) -- the shards the vocabulary-parallel log-prob
    kernels expect.  A checkpoint tensor with ``real_vocab`` rows is copied into the rows a shard owns and the padding
    rows are zeroed."""
    if hasattr(parallel_lm_head_cls, _PATCH_MARKER):
        return
    if padded_vocab < real_vocab or padded_vocab % (8 * 128):
        raise RuntimeError(f"invalid strict rollout vocab contract: real={real_vocab}, padded={padded_vocab} "
                           "(the padded size must be a multiple of 8 x 128 so that tiles never straddle a shard)")
    original_init = parallel_lm_head_cls.__init__
    original_loader = vocab_embedding_cls.weight_loader

    def strict_weight_loader(instance: Any, param: Any, loaded_weight: torch.Tensor) -> None:
        strict_real = getattr(instance, "_rl_kernel_real_vocab_size", None)
        out_dim = getattr(param, "output_dim", 0)
        if strict_real is not None and getattr(param, "packed_dim", None) is None and \
                loaded_weight.shape[out_dim] == int(strict_real):
            idx = instance.shard_indices
            start = int(idx.org_vocab_start_index)
            size = int(idx.org_vocab_end_index) - start
            have = max(0, min(size, int(strict_real) - start))
            data = param.data
            if have:
                data[:have].copy_(loaded_weight.narrow(out_dim, start, have))
            data[have:].zero_()                              # padding rows of the shard and any alignment tail
            instance._rl_kernel_lm_head_version = getattr(instance, "_rl_kernel_lm_head_version", 0) + 1
            return
        original_loader(instance, param, loaded_weight)

    def strict_init(instance: Any, *args: Any, **kwargs: Any) -> None:
        if args:
            args = (padded_vocab, *args[1:])
        else:
            kwargs["num_embeddings"] = padded_vocab
        kwargs["org_num_embeddings"] = padded_vocab
        kwargs["padding_size"] = padded_vocab               # the engine rounds UP to a multiple: keeps the size as is
        original_init(instance, *args, **kwargs)
        instance._rl_kernel_real_vocab_size = real_vocab
        got = (int(getattr(instance, "org_vocab_size", padded_vocab)), int(getattr(instance, "num_embeddings_padded", padded_vocab)))
        if got != (padded_vocab, padded_vocab):
            raise RuntimeError(f"strict rollout LM-head padding did not produce the padded vocabulary layout {padded_vocab}: {got}")

    setattr(parallel_lm_head_cls, _PATCH_MARKER, original_init)
    parallel_lm_head_cls.__init__ = strict_init
    if not hasattr(vocab_embedding_cls, "__rl_kernel_original_weight_loader__"):
        setattr(vocab_embedding_cls, "__rl_kernel_original_weight_loader__", original_loader)
        vocab_embedding_cls.weight_loader = strict_weight_loader


def install_vllm_integration(*, decoder_layer_cls=None, attention_cls=None, mlp_cls=None, rmsnorm_cls=None,
                             model_cls=None, sampler_cls=None, attention_impl_cls=None, plan: IntegrationPlan | None = None,
                             tp_size: int = 1, collective=None, temperature: float | None = None,
                             real_vocab: int | None = None, top_k: int = 0, top_p: float = 1.0
                             ) -> FrameworkOperatorIntegration:
    """``attention_cls``: a module whose ``forward(q, k, v, kv_cache=..., ...)`` is replaced (model-level attention).
    ``attention_impl_cls``: a backend implementation class with vLLM's
    ``forward(layer, query, key, value, kv_cache, attn_metadata, output)`` (used when the backend cannot be chosen
    through the engine's own selector)."""
    plan = plan or IntegrationPlan.from_env()
    integ = FrameworkOperatorIntegration("vllm", "rollout", plan)
    want = plan.side("rollout")
    temperature = temperature if temperature is not None else float(os.environ.get("RL_KERNEL_VLLM_TEMPERATURE", "1.0"))
    real_vocab = real_vocab or (int(os.environ["RL_KERNEL_VLLM_REAL_VOCAB_SIZE"])
                                if "RL_KERNEL_VLLM_REAL_VOCAB_SIZE" in os.environ else None)
    if want["attention"] and (attention_cls is not None or attention_impl_cls is not None):
        op = VllmAttentionOperator()
        integ.install("attention", op)
        if attention_cls is not None:
            def attn_forward(self, q, k, v, kv_cache=None, positions=None, **kw):
                return integ.execute("attention", self, q, k, v, kv_cache=kv_cache, positions=positions, **kw)

            _patch_method(attention_cls, "forward", attn_forward)
        if attention_impl_cls is not None:
            def impl_forward(self, layer, query, key, value, kv_cache, attn_metadata, output=None, *a, **kw):
                if attn_metadata is None:                     # the engine's profiling run
                    return output.fill_(0) if output is not None else torch.zeros_like(query)
                who = self if hasattr(self, "num_kv_heads") else layer
                return integ.execute("attention", who, query, key, value, kv_cache=kv_cache, attn_metadata=attn_metadata,
                                     output=output)

            _patch_method(attention_impl_cls, "forward", impl_forward)
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
            # publish what the sampler needs to recompute the sampled token's log-prob with the same strict operator
            # as the trainer (parity: publish_rollout_linear_logp_context)
            _STATE["linear_logp_context"] = {"hidden": hidden_states, "lm_head": self.lm_head.weight,
                                             "real_vocab": real_vocab}
            orig = getattr(type(self), "_rlk_orig_compute_logits")
            return orig(self, hidden_states, *a, **kw)

        _patch_method(model_cls, "compute_logits", compute_logits)
        if sampler_cls is not None:
            restricted = (top_k and top_k > 0) or top_p < 1.0

            def sampler_forward(self, logits, sampling_metadata=None, **kw):
                orig = getattr(type(self), "_rlk_orig_forward")
                with capture_support(bool(restricted)) as cap:
                    out = orig(self, logits, sampling_metadata, **kw)
                ctx = _STATE.get("linear_logp_context")
                ids = getattr(out, "sampled_token_ids", out)
                if ctx is not None and isinstance(ids, torch.Tensor):
                    min_keep = None
                    if restricted:
                        if "mask" in cap:                     # the support the engine's own filter kept
                            min_keep = support_to_threshold(logits, cap["mask"], temperature)
                        else:
                            from rl_kernel_b200.ops.sampling.policy import keep_threshold

                            min_keep = keep_threshold(logits, temperature=temperature, top_k=top_k, top_p=top_p,
                                                      real_vocab=real_vocab)
                    lp = integ.execute("logp", ctx["hidden"], ctx["lm_head"], ids.reshape(-1), min_keep=min_keep)
                    _STATE["last_min_keep"] = min_keep
                    try:
                        out.rl_kernel_logprobs = lp
                    except AttributeError:
                        _STATE["last_logprobs"] = lp
                return out

            _patch_method(sampler_cls, "forward", sampler_forward)
    if rmsnorm_cls is not None and (want["attention"] or want["ffn"]):
        def norm_forward(self, x, residual=None):
            eps = getattr(self, "variance_epsilon", getattr(self, "eps", 1e-6))
            return fused_add_rms_norm(x, residual, self.weight, eps)

        _patch_method(rmsnorm_cls, "forward", norm_forward)
        _patch_method(rmsnorm_cls, "forward_native", norm_forward)
        _patch_method(rmsnorm_cls, "forward_cuda", norm_forward)
    _STATE["integration"] = integ
    return integ


def last_rollout_logprobs():
    return _STATE.get("last_logprobs")


def last_rollout_support_threshold():
    """Per-token scaled-logit thresholds of the last sampling step (None when nothing was cut): what the trainer passes
    as ``min_keep`` to score the same support."""
    return _STATE.get("last_min_keep")


def register_vllm_plugin() -> None:
    """Entry point for ``vllm.general_plugins`` (parity: runtime.py:1961-1966).  Does nothing unless
    RL_KERNEL_VLLM_INTEGRATION is set, so having the package installed never changes a plain vLLM."""
    if os.environ.get("RL_KERNEL_VLLM_INTEGRATION", "0") not in ("1", "true", "True"):
        return
    from vllm.model_executor.layers.layernorm import RMSNorm  # noqa: PLC0415
    from vllm.model_executor.models import qwen3 as q3  # noqa: PLC0415

    from rl_kernel_b200.integrations.engines.rollout.vllm import sampling_support
    from rl_kernel_b200.integrations.engines.rollout.vllm.backend import register_attention_backend

    register_attention_backend()
    sampling_support.install_capture()
    if "RL_KERNEL_VLLM_PADDED_VOCAB_SIZE" in os.environ:
        from vllm.model_executor.layers.vocab_parallel_embedding import ParallelLMHead, VocabParallelEmbedding  # noqa: PLC0415

        patch_lm_head_padding(ParallelLMHead, VocabParallelEmbedding,
                              real_vocab=int(os.environ["RL_KERNEL_VLLM_REAL_VOCAB_SIZE"]),
                              padded_vocab=int(os.environ["RL_KERNEL_VLLM_PADDED_VOCAB_SIZE"]))
    install_vllm_integration(decoder_layer_cls=q3.Qwen3DecoderLayer, mlp_cls=getattr(q3, "Qwen3MLP", None),
                             rmsnorm_cls=RMSNorm, model_cls=q3.Qwen3ForCausalLM,
                             top_k=int(os.environ.get("RL_KERNEL_VLLM_TOP_K", "0")),
                             top_p=float(os.environ.get("RL_KERNEL_VLLM_TOP_P", "1.0")))
