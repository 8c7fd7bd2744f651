"""The trainable parameters whose gradients the chain gate compares after a real backward (parity:
rl_engine/validation/models/chain_gradients.py:18-79): embedding, final norm, LM head and, for every decoder layer,
q/k/v/o projections, q/k norm gains, the three MLP matrices and the two RMSNorm gains."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable, Sequence

_LAYER_LEAVES = (("input_layernorm.weight", "gain", "reduction"), ("self_attn.q_proj.weight", "matrix", "reduction"),
                 ("self_attn.k_proj.weight", "matrix", "reduction"), ("self_attn.v_proj.weight", "matrix", "reduction"),
                 ("self_attn.o_proj.weight", "matrix", "reduction"), ("self_attn.q_norm.weight", "gain", "reduction"),
                 ("self_attn.k_norm.weight", "gain", "reduction"), ("post_attention_layernorm.weight", "gain", "reduction"),
                 ("mlp.gate_proj.weight", "matrix", "reduction"), ("mlp.up_proj.weight", "matrix", "reduction"),
                 ("mlp.down_proj.weight", "matrix", "reduction"))
_TOP = (("embed_tokens.weight", "embedding", "gather"), ("norm.weight", "gain", "reduction"), ("lm_head.weight", "matrix", "reduction"))


@dataclass(frozen=True)
class GradParamSpec:
    name: str
    kind: str          # matrix | gain | embedding
    op_class: str      # reduction | gather


def required_grad_names(*, num_hidden_layers: int = 36) -> tuple[str, ...]:
    names = [n for n, _, _ in _TOP]
    for i in range(int(num_hidden_layers)):
        names += [f"layers.{i}.{leaf}" for leaf, _, _ in _LAYER_LEAVES]
    return tuple(names)


def grad_param_specs(*, num_hidden_layers: int = 36) -> tuple[GradParamSpec, ...]:
    specs = [GradParamSpec(n, k, c) for n, k, c in _TOP]
    for i in range(int(num_hidden_layers)):
        specs += [GradParamSpec(f"layers.{i}.{leaf}", k, c) for leaf, k, c in _LAYER_LEAVES]
    return tuple(specs)


def missing_required_grads(present: Iterable[str], *, num_hidden_layers: int = 36, tied_lm_head: bool = False) -> tuple[str, ...]:
    """Required names absent from ``present`` (names may carry a ``model.`` prefix).  With tied embeddings the LM head
    has no leaf of its own."""
    have = {n.removeprefix("model.") for n in present}
    need = [n for n in required_grad_names(num_hidden_layers=num_hidden_layers) if not (tied_lm_head and n == "lm_head.weight")]
    return tuple(n for n in need if n not in have)


def group_by_kind(names: Sequence[str]) -> dict[str, tuple[str, ...]]:
    kinds = {leaf: k for leaf, k, _ in _LAYER_LEAVES} | {n: k for n, k, _ in _TOP}
    out: dict[str, list[str]] = {}
    for n in names:
        bare = n.removeprefix("model.")
        leaf = bare.split(".", 2)[2] if bare.startswith("layers.") else bare
        out.setdefault(kinds.get(leaf, "other"), []).append(n)
    return {k: tuple(v) for k, v in out.items()}


__all__ = ["GradParamSpec", "grad_param_specs", "group_by_kind", "missing_required_grads", "required_grad_names"]
