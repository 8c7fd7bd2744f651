"""Pinned Qwen3 dense topology (parity: rl_engine/models/qwen3/spec.py:9-143).

``Qwen3DenseSpec.official()`` is the Qwen3-8B fingerprint; ``scaled()`` builds smaller members of
the same family for tests (the official spec itself cannot be shrunk).  ``canonical_tp`` is the
virtual tensor-parallel degree that fixes every reduction tree: weights are laid out in
``canonical_tp`` shards and a physical TP rank owns ``canonical_tp / tp`` consecutive shards, so
TP = 1, 2, 4, 8 execute the same arithmetic (the reference's "canonical virtual TP=8",
rl_engine/backends/cuda/ffn/ffn.py:338-368).
"""
from __future__ import annotations

from dataclasses import dataclass, replace

OFFICIAL_FINGERPRINT = {
    "num_hidden_layers": 36,
    "hidden_size": 4096,
    "intermediate_size": 12288,
    "num_attention_heads": 32,
    "num_key_value_heads": 8,
    "head_dim": 128,
    "vocab_size": 151936,
    "max_position_embeddings": 40960,
    "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-06,
    "hidden_act": "silu",
    "swiglu": True,
    "tie_word_embeddings": False,
    "attention_bias": False,
    "qk_norm": True,
}

NODE_KINDS = ("embedding", "rms_norm", "det_gemm", "qk_norm", "rope", "attention", "swiglu",
              "lm_head", "logprob")

VOCAB_TILE = 128


@dataclass(frozen=True)
class Qwen3DenseSpec:
    num_hidden_layers: int
    hidden_size: int
    intermediate_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int = 40960
    rope_theta: float = 1000000.0
    rms_norm_eps: float = 1e-6
    hidden_act: str = "silu"
    swiglu: bool = True
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    qk_norm: bool = True
    canonical_tp: int = 8
    model_id: str = "Qwen/Qwen3-8B"

    def __post_init__(self) -> None:
        if self.num_attention_heads % self.num_key_value_heads:
            raise ValueError("q heads must be a multiple of kv heads")
        if self.tie_word_embeddings or self.attention_bias or not self.qk_norm or not self.swiglu:
            raise ValueError("only the Qwen3 dense family (QK-norm, SwiGLU, untied head, no bias) is modelled")
        c = self.canonical_tp
        if c not in (1, 2, 4, 8) or self.num_key_value_heads % c or self.intermediate_size % c:
            raise ValueError(f"canonical_tp={c} must divide kv heads and intermediate size")

    # ----- constructors
    @classmethod
    def official(cls) -> "Qwen3DenseSpec":
        return cls(**{k: v for k, v in OFFICIAL_FINGERPRINT.items()})

    @classmethod
    def from_fingerprint(cls, fp: dict) -> "Qwen3DenseSpec":
        """Strict: every official field must match (architecture drift is an error)."""
        for key, expected in OFFICIAL_FINGERPRINT.items():
            if fp.get(key) != expected:
                raise ValueError(f"fingerprint {key}={fp.get(key)!r} != official {expected!r}")
        return cls.official()

    @classmethod
    def scaled(cls, *, layers: int, hidden: int, ffn: int, q_heads: int, kv_heads: int,
               head_dim: int = 128, vocab: int = 4096, canonical_tp: int | None = None,
               rope_theta: float = 1e6) -> "Qwen3DenseSpec":
        c = canonical_tp if canonical_tp is not None else min(8, kv_heads)
        return cls(num_hidden_layers=layers, hidden_size=hidden, intermediate_size=ffn,
                   num_attention_heads=q_heads, num_key_value_heads=kv_heads, head_dim=head_dim,
                   vocab_size=vocab, rope_theta=rope_theta, canonical_tp=c,
                   model_id=f"qwen3-scaled-{layers}x{hidden}")

    def with_layers(self, n: int) -> "Qwen3DenseSpec":
        return replace(self, num_hidden_layers=n)

    # ----- derived sizes
    @property
    def group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def qkv_dim(self) -> int:
        return self.q_dim + 2 * self.kv_dim

    @property
    def padded_vocab_size(self) -> int:
        """Vocab rounded up so that every canonical shard is a whole number of 128-id tiles
        (151936 -> 152576 = 8 * 149 * 128, the reference's canonical padded size)."""
        unit = VOCAB_TILE * self.canonical_tp
        return (self.vocab_size + unit - 1) // unit * unit

    @property
    def num_vocab_tiles(self) -> int:
        return self.padded_vocab_size // VOCAB_TILE

    def param_count(self) -> int:
        h, i = self.hidden_size, self.intermediate_size
        per_layer = h * self.qkv_dim + self.q_dim * h + 3 * h * i + 2 * h + 2 * self.head_dim
        return self.num_hidden_layers * per_layer + 2 * self.vocab_size * h + h

    def fingerprint(self) -> dict:
        return {k: getattr(self, k) for k in OFFICIAL_FINGERPRINT}

    # ----- operator graph (17 nodes per layer)
    def node_names(self) -> tuple[str, ...]:
        names = ["embedding"]
        for index in range(self.num_hidden_layers):
            p = f"layers.{index}"
            names += [f"{p}.input_layernorm", f"{p}.q_proj", f"{p}.k_proj", f"{p}.v_proj",
                      f"{p}.q_norm", f"{p}.k_norm", f"{p}.rope_q", f"{p}.rope_k", f"{p}.attn",
                      f"{p}.o_proj", f"{p}.residual_attn", f"{p}.post_attention_layernorm",
                      f"{p}.gate_proj", f"{p}.up_proj", f"{p}.swiglu", f"{p}.down_proj",
                      f"{p}.residual_mlp"]
        names += ["final_layernorm", "lm_head", "logprob", "loss"]
        return tuple(names)

    def node_kind(self, node_name: str) -> str:
        if node_name == "embedding":
            return "embedding"
        if node_name.endswith("layernorm"):
            return "rms_norm"
        if node_name.endswith((".q_norm", ".k_norm")):
            return "qk_norm"
        if node_name.endswith((".rope_q", ".rope_k")):
            return "rope"
        if node_name.endswith(".attn"):
            return "attention"
        if node_name.endswith(".swiglu"):
            return "swiglu"
        if node_name == "lm_head":
            return "lm_head"
        if node_name in ("logprob", "loss"):
            return "logprob"
        if node_name.endswith(("_proj",)):
            return "det_gemm"
        if node_name.endswith(("residual_attn", "residual_mlp")):
            return "residual"
        raise KeyError(node_name)
