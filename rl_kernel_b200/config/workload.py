"""Workload manifest: model identity, backend profiles and representative cases, plus the logical
batch transforms (chunk / pack / pad / permute) the validation cells are built from (parity:
WS1Manifest and transforms, rl_engine/config/workload.py:209-1010)."""
from __future__ import annotations

import json
from dataclasses import dataclass
from functools import lru_cache
from pathlib import Path

import torch

_DIR = Path(__file__).resolve().parent / "workloads"


@dataclass(frozen=True)
class WS1Manifest:
    workload_id: str
    seed: int
    model_identity: dict
    backend_profiles: dict
    cases: tuple

    def case(self, case_id: str) -> dict:
        for c in self.cases:
            if c["case_id"] == case_id:
                return dict(c)
        raise KeyError(case_id)


@lru_cache(maxsize=4)
def load_manifest(name: str = "qwen3_8b") -> WS1Manifest:
    d = json.loads((_DIR / f"{name}.json").read_text())
    for k in ("workload_id", "seed", "model_identity", "backend_profiles", "cases"):
        if k not in d:
            raise ValueError(f"manifest {name} lacks {k!r}")
    return WS1Manifest(d["workload_id"], int(d["seed"]), d["model_identity"], d["backend_profiles"], tuple(d["cases"]))


# ---- logical batch transforms: each returns (transformed ids, function that maps results back)
def chunk_batch(ids: torch.Tensor, size: int):
    return [ids[i:i + size] for i in range(0, ids.shape[0], size)], lambda outs: torch.cat(outs)


def permute_batch(ids: torch.Tensor, seed: int = 0):
    perm = torch.randperm(ids.shape[0], generator=torch.Generator().manual_seed(seed))
    inv = torch.argsort(perm)
    return ids[perm], lambda out: out[inv]


def pad_batch(ids: torch.Tensor, pad_to: int, side: str = "right", pad_id: int = 0):
    B, S = ids.shape
    if pad_to < S:
        raise ValueError("pad_to must be at least the sequence length")
    out = ids.new_full((B, pad_to), pad_id)
    mask = torch.zeros(B, pad_to, dtype=torch.bool)
    if side == "right":
        out[:, :S], mask[:, :S] = ids, True
        return out, mask, lambda r: r[:, :r.shape[1] - (pad_to - S)]
    out[:, pad_to - S:], mask[:, pad_to - S:] = ids, True
    return out, mask, lambda r: r[:, pad_to - S:]


def pack_batch(ids: torch.Tensor, lengths: torch.Tensor):
    flat = torch.cat([ids[b, : int(lengths[b])] for b in range(ids.shape[0])])
    cu = torch.cat([lengths.new_zeros(1), lengths.cumsum(0)])
    return flat, cu
