"""Attention backend object for a vLLM-style engine (parity: the backend registration of
rl_engine/integrations/engines/rollout/vllm/runtime.py:1693-1890).

``RLKernelAttentionBackend`` answers the questions an engine asks a backend (name, implementation
class, metadata builder, KV-cache shape and the block sizes the kernel supports) and
``RLKernelAttentionImpl.forward`` is the per-layer entry with vLLM's v1 signature
``(layer, query, key, value, kv_cache, attn_metadata, output)``.  With vLLM importable the classes
derive from its abstract bases and ``register_attention_backend`` files the backend under
``AttentionBackendEnum.CUSTOM``; without it they stand alone, which is how the tests drive them.
"""
from __future__ import annotations

from typing import Any

import torch

from rl_kernel_b200.integrations.engines.rollout.vllm.operators import PAGE, VllmAttentionOperator

try:                                                                  # the real abstract bases, when present
    from vllm.v1.attention.backend import AttentionBackend as _BackendBase  # type: ignore
    from vllm.v1.attention.backend import AttentionImpl as _ImplBase  # type: ignore
    _HAVE_VLLM = True
except Exception:  # noqa: BLE001 - any import problem means "stand alone"
    _BackendBase, _ImplBase, _HAVE_VLLM = object, object, False

BACKEND_NAME = "RLKERNEL_B200"
BACKEND_CLASS_PATH = "rl_kernel_b200.integrations.engines.rollout.vllm.backend.RLKernelAttentionBackend"


class RLKernelAttentionImpl(_ImplBase):                               # type: ignore[misc]
    can_return_lse_for_decode = True

    def __init__(self, num_heads: int, head_size: int, scale: float, num_kv_heads: int | None = None,
                 alibi_slopes=None, sliding_window=None, kv_cache_dtype: str = "auto", logits_soft_cap=None,
                 attn_type: str = "decoder", kv_sharing_target_layer_name=None, **_ignored) -> None:
        if alibi_slopes is not None or sliding_window is not None or logits_soft_cap:
            raise NotImplementedError("ALiBi, sliding windows and logit soft caps are outside the deterministic contract")
        if kv_cache_dtype not in ("auto", "bfloat16"):
            raise NotImplementedError("the deterministic kernels keep the KV cache in bf16")
        if head_size != 128:
            raise NotImplementedError("head_size must be 128")
        if attn_type != "decoder":
            raise NotImplementedError("only causal decoder self-attention is implemented")
        self.num_heads, self.head_size, self.head_dim = num_heads, head_size, head_size
        self.num_kv_heads = num_kv_heads or num_heads
        self.scale = float(scale)
        self.op = VllmAttentionOperator()

    def forward(self, layer: torch.nn.Module, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                kv_cache: torch.Tensor, attn_metadata: Any, output: torch.Tensor | None = None, output_scale=None,
                output_block_scale=None) -> torch.Tensor:
        if output_scale is not None or output_block_scale is not None:
            raise NotImplementedError("fused output quantisation is not part of the deterministic contract")
        if attn_metadata is None:                                     # the engine's memory-profiling run
            return output.fill_(0) if output is not None else torch.zeros_like(query)
        if not getattr(attn_metadata, "causal", True):
            raise NotImplementedError("only causal attention is implemented")
        if getattr(attn_metadata, "use_cascade", False):
            raise NotImplementedError("cascade attention splits the key axis; shared prefixes are served by page sharing")
        return self.op.forward_paged(self, query, key, value, kv_cache, attn_metadata, output)


class RLKernelAttentionBackend(_BackendBase):                         # type: ignore[misc]
    accept_output_buffer = True
    forward_includes_kv_cache_update = True
    supported_dtypes = [torch.bfloat16]
    supported_kv_cache_dtypes = ["auto", "bfloat16"]

    @staticmethod
    def get_name() -> str:
        return BACKEND_NAME

    @staticmethod
    def get_supported_kernel_block_sizes() -> list[int]:
        return [PAGE]

    @staticmethod
    def get_supported_head_sizes() -> list[int]:
        return [128]

    @staticmethod
    def get_impl_cls():
        return RLKernelAttentionImpl

    @staticmethod
    def get_builder_cls():
        """The step metadata this backend reads (slot mapping, block table, sequence lengths, query starts) is what
        vLLM's FlashAttention builder produces, so that builder is reused."""
        if not _HAVE_VLLM:
            raise RuntimeError("the metadata builder comes from vLLM, which is not importable here")
        from vllm.v1.attention.backends.flash_attn import FlashAttentionMetadataBuilder  # type: ignore

        return FlashAttentionMetadataBuilder

    @staticmethod
    def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int,
                           cache_dtype_str: str = "auto") -> tuple[int, ...]:
        if block_size != PAGE:
            raise ValueError(f"block_size must be {PAGE}")
        return (2, num_blocks, block_size, num_kv_heads, head_size)

    @staticmethod
    def use_cascade_attention(*_a, **_k) -> bool:
        return False


def register_attention_backend() -> str:
    """File the backend under vLLM's CUSTOM slot; returns the class path that was registered."""
    if not _HAVE_VLLM:
        raise RuntimeError("vLLM is not importable: nothing to register with")
    from vllm.v1.attention.backends.registry import AttentionBackendEnum, register_backend  # type: ignore

    register_backend(AttentionBackendEnum.CUSTOM, BACKEND_CLASS_PATH)
    return BACKEND_CLASS_PATH
