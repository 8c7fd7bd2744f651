"""Qwen3 dense parameters in the Hugging Face key layout (minus the ``model.`` prefix) and their
packing into the engine's canonical, tensor-parallel-invariant layout.

Key layout (parity: rl_engine/models/qwen3/reference.py:431-463): ``embed_tokens.weight``,
``layers.{i}.{input_layernorm,post_attention_layernorm}.weight``,
``layers.{i}.self_attn.{q,k,v,o}_proj.weight``, ``layers.{i}.self_attn.{q,k}_norm.weight``,
``layers.{i}.mlp.{gate,up,down}_proj.weight``, ``norm.weight``, ``lm_head.weight``.

Engine layout (what the sm_100a kernels consume):
  * ``wqkv``  [(Hq+2Hkv)*D, H]: GQA-group-major rows — for KV head g: its G query heads, key head g,
    value head g.  A TP rank owns whole groups.
  * ``wgu``   [2*I, H]: ``canonical_tp`` blocks, block c = gate rows [c*I/c_tp, (c+1)*I/c_tp) then the
    same rows of up.
  * ``wo`` [H, Hq*D] and ``wd`` [H, I]: natural; a TP rank owns a column range, and the GEMM's
    canonical K chunks are the canonical shards.
  * ``embed`` / ``lm_head`` [V_pad, H]: rows beyond the real vocab are zero; a TP rank owns a row range.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Iterator, Mapping

import torch

from rl_kernel_b200.models.qwen3.spec import Qwen3DenseSpec


def required_weight_keys(spec: Qwen3DenseSpec) -> list[str]:
    keys = ["embed_tokens.weight"]
    for i in range(spec.num_hidden_layers):
        p = f"layers.{i}"
        keys += [f"{p}.input_layernorm.weight", f"{p}.self_attn.q_proj.weight",
                 f"{p}.self_attn.k_proj.weight", f"{p}.self_attn.v_proj.weight",
                 f"{p}.self_attn.o_proj.weight", f"{p}.self_attn.q_norm.weight",
                 f"{p}.self_attn.k_norm.weight", f"{p}.post_attention_layernorm.weight",
                 f"{p}.mlp.gate_proj.weight", f"{p}.mlp.up_proj.weight", f"{p}.mlp.down_proj.weight"]
    keys += ["norm.weight", "lm_head.weight"]
    return keys


def weight_shapes(spec: Qwen3DenseSpec) -> dict[str, tuple[int, ...]]:
    h, i, d = spec.hidden_size, spec.intermediate_size, spec.head_dim
    out: dict[str, tuple[int, ...]] = {"embed_tokens.weight": (spec.vocab_size, h)}
    for l in range(spec.num_hidden_layers):
        p = f"layers.{l}"
        out[f"{p}.input_layernorm.weight"] = (h,)
        out[f"{p}.self_attn.q_proj.weight"] = (spec.q_dim, h)
        out[f"{p}.self_attn.k_proj.weight"] = (spec.kv_dim, h)
        out[f"{p}.self_attn.v_proj.weight"] = (spec.kv_dim, h)
        out[f"{p}.self_attn.o_proj.weight"] = (h, spec.q_dim)
        out[f"{p}.self_attn.q_norm.weight"] = (d,)
        out[f"{p}.self_attn.k_norm.weight"] = (d,)
        out[f"{p}.post_attention_layernorm.weight"] = (h,)
        out[f"{p}.mlp.gate_proj.weight"] = (i, h)
        out[f"{p}.mlp.up_proj.weight"] = (i, h)
        out[f"{p}.mlp.down_proj.weight"] = (h, i)
    out["norm.weight"] = (h,)
    out["lm_head.weight"] = (spec.vocab_size, h)
    return out


def _sha256_file(path: Path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 22), b""):
            h.update(chunk)
    return h.hexdigest()


class Qwen3DenseWeights:
    """Parameter bag keyed by HF names."""

    def __init__(self, tensors: dict[str, torch.Tensor], source: str, content_hash: str = ""):
        self.tensors = tensors
        self.source = source
        self.content_hash = content_hash

    def __getitem__(self, key: str) -> torch.Tensor:
        return self.tensors[key]

    def __contains__(self, key: str) -> bool:
        return key in self.tensors

    def keys(self):
        return self.tensors.keys()

    def items(self) -> Iterator[tuple[str, torch.Tensor]]:
        return iter(self.tensors.items())

    @classmethod
    def synthetic(cls, spec: Qwen3DenseSpec, *, device: torch.device | str = "cpu",
                  dtype: torch.dtype = torch.bfloat16, seed: int = 0, std: float = 0.02
                  ) -> "Qwen3DenseWeights":
        """Seeded N(0, std) matrices and unit norm gains with the spec's shapes
        (rl_engine/models/qwen3/reference.py:272-318 uses N(0,1); 0.02 keeps bf16 activations tame)."""
        gen = torch.Generator(device="cpu").manual_seed(int(seed))
        tensors: dict[str, torch.Tensor] = {}
        for name, shape in weight_shapes(spec).items():
            if len(shape) == 1:
                t = torch.ones(shape, dtype=torch.float32)
            else:
                t = torch.randn(shape, generator=gen, dtype=torch.float32) * std
            tensors[name] = t.to(device=device, dtype=dtype)
        return cls(tensors, source="synthetic", content_hash=f"synthetic-seed{seed}")

    @classmethod
    def from_hf(cls, spec: Qwen3DenseSpec, source: str | Path, *, device: torch.device | str = "cpu",
                dtype: torch.dtype = torch.bfloat16, expected_sha256: Mapping[str, str] | None = None
                ) -> "Qwen3DenseWeights":
        """Load a local safetensors snapshot; shard hashes are verified when ``expected_sha256``
        (filename -> sha256) is given (parity: verify_hf_weight_snapshot, reference.py:384-428)."""
        from safetensors.torch import load_file  # local import: optional dependency

        root = Path(source)
        index = root / "model.safetensors.index.json"
        files = sorted({*json.loads(index.read_text())["weight_map"].values()}) if index.exists() \
            else [p.name for p in sorted(root.glob("*.safetensors"))]
        if not files:
            raise FileNotFoundError(f"no safetensors files under {root}")
        digest = hashlib.sha256()
        raw: dict[str, torch.Tensor] = {}
        for name in files:
            path = root / name
            sha = _sha256_file(path)
            if expected_sha256 is not None and expected_sha256.get(name) != sha:
                raise ValueError(f"checksum mismatch for {name}: {sha} != {expected_sha256.get(name)}")
            digest.update(sha.encode())
            raw.update(load_file(str(path)))
        tensors = {}
        for key, value in raw.items():
            k = key[len("model."):] if key.startswith("model.") else key
            tensors[k] = value.to(device=device, dtype=dtype)
        missing = [k for k in required_weight_keys(spec) if k not in tensors]
        if missing:
            raise KeyError(f"snapshot is missing {len(missing)} tensors, first: {missing[:3]}")
        for k, shape in weight_shapes(spec).items():
            if tuple(tensors[k].shape) != shape:
                raise ValueError(f"{k}: shape {tuple(tensors[k].shape)} != expected {shape}")
        return cls(tensors, source=str(root), content_hash=digest.hexdigest())

    def sha256_by_tensor(self) -> dict[str, str]:
        """Per-tensor content hashes (the weight audit of the reference's vime runs)."""
        out = {}
        for k, t in self.tensors.items():
            b = t.detach().contiguous().cpu()
            out[k] = hashlib.sha256(b.view(torch.uint8).numpy().tobytes()).hexdigest()
        return out


# --------------------------------------------------------------------------- engine packing
def pack_qkv(spec: Qwen3DenseSpec, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """[q_dim,H], [kv_dim,H], [kv_dim,H] -> GQA-group-major [(Hq+2Hkv)*D, H]."""
    g, d, h = spec.group_size, spec.head_dim, q.shape[1]
    qg = q.reshape(spec.num_key_value_heads, g * d, h)
    kg = k.reshape(spec.num_key_value_heads, d, h)
    vg = v.reshape(spec.num_key_value_heads, d, h)
    return torch.cat([qg, kg, vg], dim=1).reshape(spec.qkv_dim, h).contiguous()


def unpack_qkv(spec: Qwen3DenseSpec, wqkv: torch.Tensor):
    g, d, h = spec.group_size, spec.head_dim, wqkv.shape[1]
    n = wqkv.shape[0] // ((g + 2) * d)
    w = wqkv.reshape(n, (g + 2) * d, h)
    return (w[:, : g * d].reshape(n * g * d, h), w[:, g * d:(g + 1) * d].reshape(n * d, h),
            w[:, (g + 1) * d:].reshape(n * d, h))


def pack_gate_up(spec: Qwen3DenseSpec, gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    c, h = spec.canonical_tp, gate.shape[1]
    blk = spec.intermediate_size // c
    return torch.cat([gate.reshape(c, blk, h), up.reshape(c, blk, h)], dim=1).reshape(-1, h).contiguous()


def unpack_gate_up(spec: Qwen3DenseSpec, wgu: torch.Tensor):
    blk, h = spec.intermediate_size // spec.canonical_tp, wgu.shape[1]
    n = wgu.shape[0] // (2 * blk)
    w = wgu.reshape(n, 2 * blk, h)
    return w[:, :blk].reshape(n * blk, h), w[:, blk:].reshape(n * blk, h)


def pad_vocab(spec: Qwen3DenseSpec, w: torch.Tensor) -> torch.Tensor:
    pad = spec.padded_vocab_size - w.shape[0]
    if pad == 0:
        return w
    return torch.cat([w, w.new_zeros(pad, w.shape[1])], dim=0)
