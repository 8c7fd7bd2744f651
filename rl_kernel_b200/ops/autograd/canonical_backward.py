"""Canonical parameter-gradient session: per-token VJP contributions are collected with their
logical (sample, token) keys and reduced in key order, so the parameter gradient does not depend on
packing, chunking or the CP/DP split of the tokens (parity: CanonicalBackwardSession,
rl_engine/ops/autograd/canonical_backward.py:26-127)."""
from __future__ import annotations

import contextlib
import threading

import torch

_TLS = threading.local()


def active_session():
    return getattr(_TLS, "session", None)


class CanonicalBackwardSession:
    def __init__(self):
        self._parts: dict[str, list[tuple[torch.Tensor, torch.Tensor, torch.Tensor]]] = {}

    def contribute(self, name: str, keys: torch.Tensor, x: torch.Tensor, dy: torch.Tensor) -> None:
        """keys [T, 2] (sample, token); x [T, in]; dy [T, out]: dW = sum_t dy_t^T x_t in key order."""
        self._parts.setdefault(name, []).append((keys.detach().cpu(), x.detach(), dy.detach()))

    def finalize(self) -> dict[str, torch.Tensor]:
        out = {}
        for name, parts in self._parts.items():
            keys = torch.cat([p[0] for p in parts])
            x = torch.cat([p[1] for p in parts]).float()
            dy = torch.cat([p[2] for p in parts]).float()
            order = torch.argsort(keys[:, 0] * (1 << 32) + keys[:, 1], stable=True)
            acc = torch.zeros(dy.shape[1], x.shape[1], dtype=torch.float32, device=x.device)
            for t in order.tolist():       # ascending logical key: fixed reduction order
                acc += torch.outer(dy[t], x[t])
            out[name] = acc
        return out

    @contextlib.contextmanager
    def activate(self):
        prev = active_session()
        _TLS.session = self
        try:
            yield self
        finally:
            _TLS.session = prev
