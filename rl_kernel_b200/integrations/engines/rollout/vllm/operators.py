"""Operator objects the vLLM binding installs (parity: VllmAttentionOperator / VllmFFNOperator /
VllmLogpOperator, rl_engine/integrations/engines/rollout/vllm/operators.py:209-1455).

``VllmAttentionOperator`` consumes what a serving engine hands an attention layer: the new tokens'
Q/K/V, the layer's block KV cache ``[2, num_blocks, block_size, Hkv, D]``, and per-step metadata
(``slot_mapping``, ``block_table``, ``seq_lens``, ``query_start_loc``).  It stores the new K/V rows at
their slots and runs the paged kernel, whose producer walks the block table; the cache block must
be the canonical 128-key block (``--block-size 128``) because a page is the unit the per-row
program is defined on.  A legacy dense call (``kv_cache=(k, v)`` as [B, S_max, Hkv, D] tensors, or
packed prefill with ``cu_seqlens``) is still accepted.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from rl_kernel_b200.ops.attention.attention import causal_attention, decode_attention
from rl_kernel_b200.ops.attention.paged import PAGE, paged_attention_block_table, write_kv_slots
from rl_kernel_b200.ops.ffn.qwen3 import qwen3_ffn
from rl_kernel_b200.ops.logprob import linear_logp


@dataclass
class VllmKVCacheView:
    """One layer's block cache as the two row pools the kernels address."""
    k_pool: torch.Tensor            # [num_blocks * 128, Hkv * D]
    v_pool: torch.Tensor
    num_blocks: int
    num_kv_heads: int
    head_dim: int

    @classmethod
    def from_tensor(cls, kv_cache: torch.Tensor) -> "VllmKVCacheView":
        if kv_cache.dim() != 5 or kv_cache.shape[0] != 2:
            raise ValueError(f"expected a [2, num_blocks, block_size, Hkv, D] cache, got {tuple(kv_cache.shape)}")
        _, nb, bs, hkv, d = kv_cache.shape
        if bs != PAGE:
            raise ValueError(f"the deterministic paged kernel needs a KV block of {PAGE} tokens (got {bs}); start the "
                             f"engine with --block-size {PAGE}")
        if not kv_cache[0].is_contiguous():
            raise ValueError("the K and V halves of the cache must be contiguous")
        return cls(kv_cache[0].view(nb * bs, hkv * d), kv_cache[1].view(nb * bs, hkv * d), nb, hkv, d)


def _host_list(x) -> list[int]:
    return [int(v) for v in (x.tolist() if isinstance(x, torch.Tensor) else x)]


class VllmAttentionOperator:
    backend_id = "b200-tcgen05"
    schedule = "canonical_128_key_blocks_no_splitkv"

    def __init__(self, peer_pools=None, *, validate_pages: bool = True):
        self.peer_pools = peer_pools            # (k_pools, v_pools) of every PCP rank when pages live on other GPUs
        self.calls = {"paged": 0, "dense_decode": 0, "packed_prefill": 0}
        self.validate_pages = validate_pages
        self._validated_shapes: set[tuple] = set()
        self._last: dict[str, Any] = {}

    @property
    def provenance(self) -> dict[str, Any]:
        """What the operator ran last (the read-back of the rollout side of an attention binding)."""
        return {"actual_backend": self.backend_id, "schedule": self.schedule, "runtime_platform": self._last.get("platform"),
                "fallback": False, "split_kv": "disabled", "kv_block": PAGE, "calls": dict(self.calls), **self._last}

    def _validate_page_bounds_once(self, block_table: torch.Tensor, lens: list[int], num_blocks: int, slot_mapping, n: int) -> None:
        """The first time a (batch, table width, pool size) geometry is seen: every page a sequence needs is inside the
        pool and every slot of the new tokens is too.  A table that points outside the pool would make the kernel read
        another layer's memory; this costs one device-to-host read per geometry, not per step."""
        key = (len(lens), tuple(block_table.shape), num_blocks)
        if not self.validate_pages or key in self._validated_shapes:
            return
        if block_table.is_cuda and torch.cuda.is_current_stream_capturing():
            return                              # a graph capture must not read the device; the eager warm-up run validated
        need = [(L + PAGE - 1) // PAGE for L in lens]
        if need and max(need) > block_table.shape[1]:
            raise ValueError(f"a sequence of {max(lens)} tokens needs {max(need)} pages but the block table has {block_table.shape[1]} columns")
        used = torch.cat([block_table[i, :k].reshape(-1) for i, k in enumerate(need) if k]) if any(need) else block_table.new_zeros(0)
        if used.numel() and (int(used.min()) < 0 or int(used.max()) >= num_blocks):
            raise ValueError(f"block table names page {int(used.max())} / {int(used.min())} outside the pool of {num_blocks} pages")
        if slot_mapping is not None and n:
            sm = slot_mapping[:n]
            live = sm[sm >= 0]                  # a negative slot marks a padded token the engine does not store
            if live.numel() and int(live.max()) >= num_blocks * PAGE:
                raise ValueError(f"slot {int(live.max())} lies outside the pool of {num_blocks * PAGE} token slots")
        self._validated_shapes.add(key)

    def forward_paged(self, layer, query, key, value, kv_cache: torch.Tensor, attn_metadata: Any,
                      output: torch.Tensor | None = None) -> torch.Tensor:
        """query [T, Hq * D] (or [T, Hq, D]); returns [T, Hq * D].  ``attn_metadata`` needs ``slot_mapping``,
        ``block_table``, ``seq_lens`` (``seq_lens_cpu`` is preferred when present) and ``query_start_loc``
        (``query_start_loc_cpu``), ``num_actual_tokens``."""
        hq, hkv, d = layer.num_heads, layer.num_kv_heads, getattr(layer, "head_dim", None) or layer.head_size
        view = VllmKVCacheView.from_tensor(kv_cache)
        n = int(getattr(attn_metadata, "num_actual_tokens", query.shape[0]))
        q = query[:n].reshape(n, hq, d)
        lens = _host_list(getattr(attn_metadata, "seq_lens_cpu", None) if getattr(attn_metadata, "seq_lens_cpu", None)
                          is not None else attn_metadata.seq_lens)
        qsl = _host_list(getattr(attn_metadata, "query_start_loc_cpu", None)
                         if getattr(attn_metadata, "query_start_loc_cpu", None) is not None else attn_metadata.query_start_loc)
        self._validate_page_bounds_once(attn_metadata.block_table[: len(lens)], lens, view.num_blocks,
                                        getattr(attn_metadata, "slot_mapping", None) if key is not None else None, n)
        if key is not None:                                   # forward_includes_kv_cache_update
            write_kv_slots(view.k_pool, view.v_pool, key[:n].reshape(n, hkv * d), value[:n].reshape(n, hkv * d),
                           attn_metadata.slot_mapping[:n])
        self._last = {"phase": "decode" if all(qsl[i + 1] - qsl[i] == 1 for i in range(len(lens))) else "prefill_or_mixed",
                      "platform": "cuda" if query.is_cuda else "cpu-reference", "num_tokens": n, "num_sequences": len(lens),
                      "peer_pages": self.peer_pools is not None}
        out3 = None if output is None else output[:n].view(n, hq, d)
        o = paged_attention_block_table(q, view.k_pool, view.v_pool, attn_metadata.block_table[: len(lens)], lens, qsl,
                                        num_kv_heads=hkv, scale=getattr(layer, "scale", None), out=out3,
                                        peer_pools=self.peer_pools)
        self.calls["paged"] += 1
        if output is not None:
            return output
        return o.reshape(n, hq * d)

    def __call__(self, layer, q, k, v, kv_cache=None, positions=None, cu_seqlens=None, attn_metadata=None, output=None,
                 **kw):
        if attn_metadata is not None and isinstance(kv_cache, torch.Tensor) and kv_cache.dim() == 5:
            return self.forward_paged(layer, q, k, v, kv_cache, attn_metadata, output)
        hq, hkv, d = layer.num_heads, layer.num_kv_heads, layer.head_dim
        if kv_cache is not None and cu_seqlens is None:
            kc, vc = kv_cache                                  # dense [B, S_max, Hkv, D] caches already holding the token
            self.calls["dense_decode"] += 1
            return decode_attention(q.view(-1, hq, d), kc, vc, positions).reshape(q.shape[0], hq * d)
        T = q.shape[0]
        cu = cu_seqlens if cu_seqlens is not None else [0, T]
        self.calls["packed_prefill"] += 1
        return causal_attention(q.view(T, hq, d), k.view(T, hkv, d), v.view(T, hkv, d), cu).reshape(T, hq * d)


class VllmFFNOperator:
    backend_id = "b200-tcgen05"

    def __init__(self, canonical_tp: int = 8, tp_size: int = 1, collective=None):
        self.canonical_tp, self.tp_size, self.collective = canonical_tp, tp_size, collective
        self.calls = 0

    @property
    def provenance(self) -> dict[str, Any]:
        return {"actual_backend": self.backend_id, "fallback": False, "canonical_k_chunks": self.canonical_tp,
                "local_k_chunks": self.canonical_tp // self.tp_size, "tp_world_size": self.tp_size, "calls": self.calls,
                "runtime_platform": getattr(self, "_platform", None)}

    def bind_packed_inference(self, module: Any, *, tp_rank: int = 0) -> tuple[int, int]:
        """Read this rank's weights out of a serving engine's MLP module (``gate_up_proj.weight`` as [2 * I_local, H] with
        the gate rows first, ``down_proj.weight`` as [H, I_local]) and keep them on the module in the layout the FFN
        kernels use: gate and up interleaved in blocks of one canonical shard (I / canonical_tp columns).  Returns
        (hidden size, local intermediate size).  Call again after every weight update."""
        gu = module.gate_up_proj.weight.detach()
        down = module.down_proj.weight.detach()
        two_i, h = gu.shape
        i_local = two_i // 2
        if two_i % 2 or down.shape != (h, i_local):
            raise ValueError(f"unexpected MLP shapes: gate_up {tuple(gu.shape)}, down {tuple(down.shape)}")
        shards = self.canonical_tp // self.tp_size
        if i_local % shards:
            raise ValueError(f"the local intermediate size {i_local} does not split into {shards} canonical shards")
        blk = i_local // shards
        gate, up = gu[:i_local].view(shards, blk, h), gu[i_local:].view(shards, blk, h)
        module.rlk_w_gu = torch.stack([gate, up], dim=1).reshape(two_i, h).contiguous()        # [g_0 | u_0 | g_1 | u_1 | ...]
        module.rlk_w_down = down.contiguous()
        module.rlk_ffn_version = getattr(module, "rlk_ffn_version", 0) + 1
        return h, i_local

    def __call__(self, layer, x):
        """``layer`` carries ``rlk_w_gu`` / ``rlk_w_down`` in the engine layout (set at weight load)."""
        if not hasattr(layer, "rlk_w_gu"):
            self.bind_packed_inference(layer)
        self.calls += 1
        self._platform = "cuda" if x.is_cuda else "cpu-reference"
        return qwen3_ffn(x, layer.rlk_w_gu, layer.rlk_w_down, canonical_tp=self.canonical_tp, tp_size=self.tp_size,
                         collective=self.collective)


class VllmLogpOperator:
    """Sampled-token log-prob with the trainer's operator; ``min_keep`` replays the sampler's top-k / top-p support."""
    backend_id = "b200-tcgen05"

    def __init__(self, temperature: float = 1.0, real_vocab: int | None = None):
        self.temperature, self.real_vocab = temperature, real_vocab
        self.calls = 0

    @property
    def provenance(self) -> dict[str, Any]:
        return {"actual_backend": self.backend_id, "fallback": False, "temperature": self.temperature, "real_vocab_size": self.real_vocab,
                "logits_materialized": False, "calls": self.calls, "runtime_platform": getattr(self, "_platform", None)}

    def __call__(self, hidden: torch.Tensor, lm_head_weight: torch.Tensor, token_ids: torch.Tensor,
                 min_keep: torch.Tensor | None = None) -> torch.Tensor:
        w = lm_head_weight if self.real_vocab is None else lm_head_weight[: self.real_vocab]
        self.calls += 1
        self._platform = "cuda" if hidden.is_cuda else "cpu-reference"
        return linear_logp(hidden, w, token_ids, self.temperature, min_keep=min_keep)
