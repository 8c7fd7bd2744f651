"""Stateful KV cache with an explicit write cursor (parity: rl_engine/reference/attention/stateful_kv.py:20-186).

``reference.attention.kv_cache.StatefulKVCache`` is the slab the reference model writes by position; this class is the
cursor-driven form used by cache-consistency checks: appends go to the cursor, reads return the written prefix (never a
caller-side concatenation), and ``identity()`` fingerprints the logical content so that two caches can be compared
without comparing layouts."""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field

import torch


@dataclass
class StatefulKVCache:
    k: torch.Tensor                     # [layers, B, Hkv, max_len, D]
    v: torch.Tensor
    cursor: list[int] = field(default_factory=list)      # written length per layer
    writes: int = 0

    @classmethod
    def allocate(cls, *, batch: int, kv_heads: int, max_len: int, head_dim: int, layers: int = 1, dtype: torch.dtype = torch.float32,
                 device: str | torch.device = "cpu") -> "StatefulKVCache":
        for name, v in (("batch", batch), ("kv_heads", kv_heads), ("max_len", max_len), ("head_dim", head_dim), ("layers", layers)):
            if v <= 0:
                raise ValueError(f"{name} must be positive")
        shape = (layers, batch, kv_heads, max_len, head_dim)
        return cls(torch.zeros(shape, dtype=dtype, device=device), torch.zeros(shape, dtype=dtype, device=device), [0] * layers)

    @property
    def max_len(self) -> int:
        return int(self.k.shape[3])

    def reset(self) -> None:
        self.cursor = [0] * len(self.cursor)
        self.k.zero_()
        self.v.zero_()
        self.writes = 0

    def _check_layer(self, layer: int) -> None:
        if not 0 <= layer < len(self.cursor):
            raise IndexError(f"layer {layer} outside [0, {len(self.cursor)})")

    def write(self, k_new: torch.Tensor, v_new: torch.Tensor, *, layer: int = 0, position: int | None = None) -> int:
        """Append ``k_new`` / ``v_new`` [B, Hkv, S_new, D] at the cursor.  ``position`` (if given) must equal the cursor:
        a cache never has holes and never rewrites history.  Returns the new length."""
        self._check_layer(layer)
        if k_new.shape != v_new.shape or k_new.dim() != 4:
            raise ValueError("k_new and v_new must both be [B, Hkv, S_new, D]")
        B, H, n, D = k_new.shape
        if (B, H, D) != (self.k.shape[1], self.k.shape[2], self.k.shape[4]):
            raise ValueError(f"write of {(B, H, D)} into a cache of {(self.k.shape[1], self.k.shape[2], self.k.shape[4])}")
        at = self.cursor[layer]
        if position is not None and position != at:
            raise ValueError(f"write at position {position} but the cursor of layer {layer} is {at}")
        if at + n > self.max_len:
            raise ValueError(f"cache overflow: {at} + {n} > {self.max_len}")
        self.k[layer, :, :, at:at + n] = k_new.to(self.k.dtype)
        self.v[layer, :, :, at:at + n] = v_new.to(self.v.dtype)
        self.cursor[layer] = at + n
        self.writes += 1
        return at + n

    def read(self, *, layer: int = 0) -> tuple[torch.Tensor, torch.Tensor, int]:
        """(k, v, length): views of the written prefix [B, Hkv, length, D]."""
        self._check_layer(layer)
        n = self.cursor[layer]
        return self.k[layer, :, :, :n], self.v[layer, :, :, :n], n

    def read_valid_mask(self, *, layer: int = 0) -> torch.Tensor:
        self._check_layer(layer)
        return torch.arange(self.max_len, device=self.k.device) < self.cursor[layer]

    def identity(self) -> dict[str, str]:
        h = hashlib.sha256()
        for layer, n in enumerate(self.cursor):
            for t in (self.k, self.v):
                h.update(t[layer, :, :, :n].contiguous().cpu().view(torch.uint8).numpy().tobytes())
        return {"content_sha256": h.hexdigest(), "lengths": ",".join(map(str, self.cursor)), "dtype": str(self.k.dtype).removeprefix("torch."),
                "shape": "x".join(map(str, self.k.shape))}


__all__ = ["StatefulKVCache"]
