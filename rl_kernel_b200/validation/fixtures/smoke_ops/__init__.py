"""Smoke-only operators used to prove that the harness detects a mismatch: ``logp_offset`` adds a
deliberate offset to the scores (parity: rl_engine/validation/fixtures/smoke_ops/
smoke_only_logp_offset.py).  Host-side fault injection only."""
from __future__ import annotations

import torch


def apply_operator_override(name: str | None, score: torch.Tensor) -> torch.Tensor:
    if name in (None, "", "none"):
        return score
    if name == "smoke_only.logp_offset":
        return score + torch.finfo(score.dtype).eps * 4
    if name == "smoke_only.flip_last_bit":
        v = score.clone().view(torch.int32 if score.dtype == torch.float32 else torch.int16)
        v[..., 0] ^= 1
        return v.view(score.dtype)
    raise ValueError(f"unknown operator override {name!r}")


SMOKE_OPERATORS = {"smoke_only.logp_reference": "rl_kernel_b200.validation.fixtures.smoke_ops.smoke_only_logp_reference.SmokeOnlyLogpReference",
                   "smoke_only.logp_offset": "rl_kernel_b200.validation.fixtures.smoke_ops.smoke_only_logp_offset.SmokeOnlyLogpOffset"}


def smoke_operator_descriptors() -> tuple[dict, ...]:
    """Descriptors of the smoke-only operators: id, import path, and the flag that keeps them out of production plans."""
    return tuple({"backend_id": k, "path": v, "semantic_operator": "selected_logprob", "smoke_only": True, "device_types": ("cpu", "cuda")}
                 for k, v in SMOKE_OPERATORS.items())


def load_smoke_operator(backend_id: str, **kwargs):
    import importlib

    try:
        path = SMOKE_OPERATORS[backend_id]
    except KeyError:
        raise ValueError(f"unknown smoke operator {backend_id!r}; known: {sorted(SMOKE_OPERATORS)}") from None
    mod, name = path.rsplit(".", 1)
    return getattr(importlib.import_module(mod), name)(**kwargs)


def register_smoke_operators(registry: dict | None = None, *, allow: bool = False) -> dict:
    """Add the smoke operators to a backend table.  ``allow`` must be set explicitly: smoke operators never enter a table
    by default."""
    if not allow:
        raise RuntimeError("smoke-only operators are registered only on explicit request (allow=True)")
    table = registry if registry is not None else {}
    table.update(SMOKE_OPERATORS)
    return table
