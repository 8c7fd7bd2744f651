"""Captures the sampling support (which ids top-k / top-p kept) while the engine's own sampler computes it, so that
the strict log-prob can be evaluated over exactly that support without filtering the vocabulary a second time
(parity: rl_engine/integrations/engines/rollout/vllm/sampling_support.py:1-48).

Only the support is reused; the log-prob itself is recomputed from the strict logits.  ``support_to_threshold``
turns a captured mask into the per-row scaled-logit threshold the sm_100a log-prob kernels take.
"""
from __future__ import annotations

from contextlib import contextmanager
from contextvars import ContextVar
from functools import wraps

import torch

_CAPTURE: ContextVar = ContextVar("rl_kernel_sampling_support", default=None)
_MARKER = "_rl_kernel_complete_support_capture"


def wrap_top_k_top_p(original):
    """A version of ``apply_top_k_top_p(logits, k, p)`` that also records ``isfinite(result)`` while a capture is open."""
    if getattr(original, _MARKER, False):
        return original

    @wraps(original)
    def wrapped(*args, **kwargs):
        result = original(*args, **kwargs)
        capture = _CAPTURE.get()
        if capture is not None:
            capture["mask"] = torch.isfinite(result)
        return result

    setattr(wrapped, _MARKER, True)
    return wrapped


def install_capture(module=None):
    """Patch ``apply_top_k_top_p`` of vLLM's sampler module (or of ``module``, for tests)."""
    if module is None:
        from vllm.v1.sample.ops import topk_topp_sampler as module  # type: ignore
    module.apply_top_k_top_p = wrap_top_k_top_p(module.apply_top_k_top_p)
    return module.apply_top_k_top_p


def supports_capture(sampler) -> bool:
    op = getattr(getattr(sampler, "topk_topp_sampler", None), "apply_top_k_top_p", None)
    return bool(getattr(op, _MARKER, False))


@contextmanager
def capture_support(enabled: bool):
    result: dict = {}
    token = _CAPTURE.set(result if enabled else None)
    try:
        yield result
    finally:
        _CAPTURE.reset(token)


def support_to_threshold(logits: torch.Tensor, mask: torch.Tensor, temperature: float = 1.0) -> torch.Tensor:
    """Per-row smallest kept scaled logit.  Exact whenever the support is an upper set of the row's logits, which
    top-k and top-p produce (ties at the boundary are kept or dropped together by both filters)."""
    z = logits.float() / max(temperature, 1e-6)
    return z.masked_fill(~mask, float("inf")).min(dim=-1).values
