"""Qwen3 dense on the PyTorch reference operators: the executable definition of the model chain.

Runs on CPU in fp32 (or any dtype) and is built so that its selected-token log-probs are bitwise
invariant to batch size, padding, chunked prefill vs decode, and the tensor-parallel degree:
every GEMM is the row-wise batch-invariant reference GEMM, row-parallel projections use the
canonical K-chunk tree, attention uses the canonical 128-key block schedule, and log-probs use
the 128-id vocab-tile contract.  Tensor parallelism runs either simulated in one process
(``tp`` > 1 with ``collective=None``) or over a real process group through a fixed-order
collective (Gloo works).  Parity: Qwen3DenseBIModel, rl_engine/models/qwen3/reference.py:466-1240.
"""
from __future__ import annotations

import math

import torch

from rl_kernel_b200.models.qwen3.spec import Qwen3DenseSpec
from rl_kernel_b200.models.qwen3.weights import Qwen3DenseWeights, pad_vocab
from rl_kernel_b200.reference.activation.swiglu import swiglu_reference
from rl_kernel_b200.reference.attention.blockwise import blockwise_attention_reference
from rl_kernel_b200.reference.attention.kv_cache import StatefulKVCache
from rl_kernel_b200.reference.gemm.det_gemm import det_gemm_reference, tree_reduce
from rl_kernel_b200.reference.logprob.tile_logp import (TILE, _target_z, merge_tile_stats,
                                                         tile_stats_reference)
from rl_kernel_b200.reference.norm.rms_norm import rms_norm_reference
from rl_kernel_b200.reference.rope.rope import qk_norm_rope_reference, rope_tables


class Qwen3DenseBIModel:
    """``tp_rank``/``tp_size`` select a physical shard; ``collective`` (fixed-order) combines shards.
    With ``tp_size > 1`` and no collective the model loops over the shards itself (simulated TP)."""

    def __init__(self, spec: Qwen3DenseSpec, weights: Qwen3DenseWeights, *, execution_dtype=torch.float32,
                 tp_size: int = 1, tp_rank: int | None = None, collective=None, max_positions: int = 4096,
                 temperature: float = 1.0):
        if spec.canonical_tp % tp_size:
            raise ValueError("tp_size must divide canonical_tp")
        self.spec, self.weights, self.dtype = spec, weights, execution_dtype
        self.tp_size, self.tp_rank, self.collective = tp_size, tp_rank, collective
        if collective is not None and tp_rank is None:
            raise ValueError("a real collective needs tp_rank")
        self.cos, self.sin = rope_tables(spec.head_dim, spec.rope_theta, max_positions)
        self.inv_temp = 1.0 / temperature
        self.scale = 1.0 / math.sqrt(spec.head_dim)
        self._last_node_outputs: dict[str, torch.Tensor] = {}
        self._capture = False

    # ------------------------------------------------------------------ plumbing
    def node_names(self):
        return self.spec.node_names()

    def captured_node_outputs(self) -> dict[str, torch.Tensor]:
        return dict(self._last_node_outputs)

    def _record(self, name: str, value: torch.Tensor) -> torch.Tensor:
        if self._capture:
            self._last_node_outputs[name] = value.detach().clone()
        return value

    def _w(self, key: str) -> torch.Tensor:
        return self.weights[key].to(self.dtype)

    def _ranks(self):
        if self.collective is not None or self.tp_size == 1:
            return [self.tp_rank or 0]
        return list(range(self.tp_size))

    def _combine(self, partials: list[torch.Tensor]) -> torch.Tensor:
        """Finish the canonical tree across TP ranks."""
        if self.collective is not None:
            return self.collective.all_reduce(partials[0])
        return partials[0] if len(partials) == 1 else tree_reduce(partials, self.dtype)

    def allocate_cache(self, batch: int, max_seq_len: int, device="cpu") -> StatefulKVCache:
        return StatefulKVCache.allocate(self.spec.num_hidden_layers, batch, self.spec.num_key_value_heads,
                                        max_seq_len, self.spec.head_dim, self.dtype, device)

    # ------------------------------------------------------------------ layer
    def _attention_block(self, layer: int, h: torch.Tensor, pos: torch.Tensor, kv_cache, batch: int, seq: int):
        spec, p = self.spec, f"layers.{layer}.self_attn"
        tp = self.tp_size
        hq, hkv, d = spec.num_attention_heads // tp, spec.num_key_value_heads // tp, spec.head_dim
        eps = spec.rms_norm_eps
        chunks_per_rank = spec.canonical_tp // tp
        partials = []
        for r in self._ranks():
            qs, ks = slice(r * hq * d, (r + 1) * hq * d), slice(r * hkv * d, (r + 1) * hkv * d)
            q = det_gemm_reference(h, self._w(f"{p}.q_proj.weight")[qs]).view(-1, hq, d)
            k = det_gemm_reference(h, self._w(f"{p}.k_proj.weight")[ks]).view(-1, hkv, d)
            v = det_gemm_reference(h, self._w(f"{p}.v_proj.weight")[ks]).view(-1, hkv, d)
            flat_pos = pos.reshape(-1)
            q = qk_norm_rope_reference(q, self._w(f"{p}.q_norm.weight"), flat_pos, self.cos, self.sin, eps)
            k = qk_norm_rope_reference(k, self._w(f"{p}.k_norm.weight"), flat_pos, self.cos, self.sin, eps)
            q, k, v = (t.view(batch, seq, -1, d) for t in (q, k, v))
            outs = []
            for b in range(batch):
                if kv_cache is not None:
                    s0 = int(pos[b, 0])
                    ck, cv = kv_cache.k[layer, b], kv_cache.v[layer, b]
                    ck[s0:s0 + seq, r * hkv:(r + 1) * hkv] = k[b]
                    cv[s0:s0 + seq, r * hkv:(r + 1) * hkv] = v[b]
                    kk, vv = ck[:s0 + seq, r * hkv:(r + 1) * hkv], cv[:s0 + seq, r * hkv:(r + 1) * hkv]
                else:
                    kk, vv = k[b], v[b]
                o, _ = blockwise_attention_reference(q[b], kk, vv, pos[b], scale=self.scale)
                outs.append(o.reshape(seq, hq * d))
            attn = torch.cat(outs)
            self._record(f"layers.{layer}.attn", attn)
            wo = self._w(f"{p}.o_proj.weight")[:, qs]
            partials.append(det_gemm_reference(attn, wo, nchunks=chunks_per_rank))
        return self._combine(partials)

    def _mlp_block(self, layer: int, h: torch.Tensor) -> torch.Tensor:
        spec, p = self.spec, f"layers.{layer}.mlp"
        per = spec.intermediate_size // self.tp_size
        chunks_per_rank = spec.canonical_tp // self.tp_size
        partials = []
        for r in self._ranks():
            sl = slice(r * per, (r + 1) * per)
            act = swiglu_reference(det_gemm_reference(h, self._w(f"{p}.gate_proj.weight")[sl]),
                                   det_gemm_reference(h, self._w(f"{p}.up_proj.weight")[sl]))
            partials.append(det_gemm_reference(act, self._w(f"{p}.down_proj.weight")[:, sl],
                                               nchunks=chunks_per_rank))
        return self._combine(partials)

    # ------------------------------------------------------------------ forward
    def forward(self, input_ids: torch.Tensor, *, position_ids: torch.Tensor | None = None,
                target_ids: torch.Tensor | None = None, loss_mask: torch.Tensor | None = None,
                kv_cache: StatefulKVCache | None = None, capture_nodes: bool = False,
                return_logits: bool = True) -> dict[str, torch.Tensor]:
        """Teacher-forced prefill, or a decode step when ``kv_cache`` is given and positions continue
        it. ``target_ids`` with the shape of ``input_ids`` are shifted (position t scores token t+1)."""
        self._capture, self._last_node_outputs = capture_nodes, {}
        if input_ids.dim() != 2:
            raise ValueError(f"input_ids must be [B, S], got {tuple(input_ids.shape)}")
        batch, seq = input_ids.shape
        spec, eps = self.spec, self.spec.rms_norm_eps
        if position_ids is None:
            position_ids = torch.arange(seq).unsqueeze(0).expand(batch, seq)
        emb = self._w("embed_tokens.weight")
        s = self._record("embedding", emb[input_ids.reshape(-1)])
        for layer in range(spec.num_hidden_layers):
            h = rms_norm_reference(s, self._w(f"layers.{layer}.input_layernorm.weight"), eps)
            o = self._attention_block(layer, h, position_ids, kv_cache, batch, seq)
            h2, s = rms_norm_reference(o, self._w(f"layers.{layer}.post_attention_layernorm.weight"), eps,
                                       residual=s)
            down = self._mlp_block(layer, h2)
            s = (down.float() + s.float()).to(self.dtype)
            self._record(f"layers.{layer}.residual_mlp", s)
        hidden = self._record("final_layernorm", rms_norm_reference(s, self._w("norm.weight"), eps))
        result: dict[str, torch.Tensor] = {"hidden": hidden.view(batch, seq, -1)}
        if return_logits:
            result["logits"] = self.lm_head_logits(hidden).view(batch, seq, -1)
        if target_ids is not None:
            if target_ids.shape == input_ids.shape:
                rows = hidden.view(batch, seq, -1)[:, :-1].reshape(-1, hidden.shape[-1])
                tg = target_ids[:, 1:].reshape(-1)
                shape = (batch, seq - 1)
                mask = None if loss_mask is None else loss_mask[:, 1:]
            else:
                rows, tg, shape, mask = hidden, target_ids.reshape(-1), target_ids.shape, loss_mask
            logp = self.selected_logprobs(rows, tg).view(shape)
            result["selected_logp"] = self._record("logprob", logp)
            if mask is not None:
                m = mask.to(logp.dtype)
                result["loss"] = -(logp * m).sum() / m.sum().clamp_min(1.0)
        return result

    __call__ = forward

    def decode_step(self, token_ids: torch.Tensor, positions: torch.Tensor, kv_cache: StatefulKVCache, **kw):
        """token_ids [B], positions [B] -> same dictionary as ``forward`` for one new token per row."""
        return self.forward(token_ids.view(-1, 1), position_ids=positions.view(-1, 1), kv_cache=kv_cache, **kw)

    # ------------------------------------------------------------------ LM head / log-probs
    def _vocab_shards(self):
        spec = self.spec
        w = pad_vocab(spec, self._w("lm_head.weight"))
        per = spec.padded_vocab_size // self.tp_size
        for r in self._ranks():
            start = r * per
            real = max(0, min(per, spec.vocab_size - start))
            yield start, w[start:start + real]

    def lm_head_logits(self, hidden: torch.Tensor) -> torch.Tensor:
        """Full real-vocab logits (gathered over TP ranks when a collective is present)."""
        parts = [det_gemm_reference(hidden, w) for _, w in self._vocab_shards()]
        if self.collective is not None:
            per = self.spec.padded_vocab_size // self.tp_size
            mine = torch.zeros(hidden.shape[0], per, dtype=parts[0].dtype)
            mine[:, : parts[0].shape[1]] = parts[0]
            full = self.collective.all_gather(mine).permute(1, 0, 2).reshape(hidden.shape[0], -1)
            return full[:, : self.spec.vocab_size]
        return torch.cat(parts, dim=1)

    def selected_logprobs(self, hidden: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        nt = self.spec.num_vocab_tiles
        stats, tz = None, torch.zeros(hidden.shape[0])
        for start, w in self._vocab_shards():
            if w.shape[0] == 0:
                continue
            logits = det_gemm_reference(hidden, w)
            st = tile_stats_reference(logits, vocab_start=start, inv_temp=self.inv_temp, n_tiles_total=nt)
            z, _ = _target_z(logits, targets, start, self.inv_temp)
            t0, t1 = start // TILE, (start + w.shape[0] + TILE - 1) // TILE
            if stats is None:
                stats = st
            else:
                stats[:, t0:t1] = st[:, t0:t1]
            tz = tz + z
        if self.collective is not None:
            per_tiles = nt // self.tp_size
            r = self.tp_rank
            mine = stats[:, r * per_tiles:(r + 1) * per_tiles].contiguous()
            stats = self.collective.all_gather(mine).permute(1, 0, 2, 3).reshape(hidden.shape[0], nt, 2)
            tz = self.collective.all_gather(tz).sum(0)
        return merge_tile_stats(stats, tz)[0]


def iter_parameter_tensors(weights: Qwen3DenseWeights):
    yield from weights.items()
