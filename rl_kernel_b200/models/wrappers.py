"""Policy / reference model adapters for RL losses (parity: rl_engine/models/wrappers.py:14-160).

A wrapped model may be any ``nn.Module`` whose output is a logits tensor, an object with ``.logits``, a mapping with
``"logits"`` or a tuple whose first element is one (the Hugging Face conventions).  ``selected_logprobs`` goes through this
framework's log-prob operator (the 128-id tile contract: fused kernels on CUDA, the reference on CPU), so a policy and a
frozen reference scored through these wrappers are scored with the same arithmetic."""
from __future__ import annotations

from typing import Any, Mapping, Optional

import torch


def extract_logits(model_output: Any) -> torch.Tensor:
    out = model_output
    if isinstance(out, torch.Tensor):
        logits = out
    elif hasattr(out, "logits"):
        logits = out.logits
    elif isinstance(out, Mapping) and "logits" in out:
        logits = out["logits"]
    elif isinstance(out, (tuple, list)) and out:
        logits = out[0]
    else:
        raise TypeError(f"cannot find logits in a model output of type {type(out)!r}")
    if not isinstance(logits, torch.Tensor):
        raise TypeError(f"logits must be a torch.Tensor, got {type(logits)!r}")
    if logits.ndim < 2:
        raise ValueError("logits must be at least [tokens, vocab]")
    return logits


def _slice_positions(logits: torch.Tensor, start: Optional[int], end: Optional[int]) -> torch.Tensor:
    if start is None and end is None:
        return logits
    idx = [slice(None)] * logits.ndim
    idx[-2] = slice(start, end)
    return logits[tuple(idx)]


class PolicyModelWrapper(torch.nn.Module):
    """The trainable policy."""

    def __init__(self, model: torch.nn.Module):
        super().__init__()
        self.model = model

    def forward(self, input_ids: torch.Tensor, **model_kwargs: Any) -> Any:
        return self.model(input_ids, **model_kwargs)

    def forward_logits(self, input_ids: torch.Tensor, **model_kwargs: Any) -> torch.Tensor:
        return extract_logits(self.forward(input_ids, **model_kwargs))

    def selected_logprobs(self, input_ids: torch.Tensor, token_ids: torch.Tensor, *, mask: Optional[torch.Tensor] = None,
                          logits_start: Optional[int] = None, logits_end: Optional[int] = None, temperature: float = 1.0,
                          output_dtype: torch.dtype = torch.float32, **model_kwargs: Any) -> torch.Tensor:
        """log p(token_ids[..., t] | ...) from the logits at positions ``logits_start:logits_end``; masked-out entries are 0."""
        from rl_kernel_b200.ops.logprob import logp_from_logits

        logits = _slice_positions(self.forward_logits(input_ids, **model_kwargs), logits_start, logits_end)
        if logits.shape[:-1] != token_ids.shape:
            raise ValueError(f"token_ids {tuple(token_ids.shape)} do not match the logits' positions {tuple(logits.shape[:-1])}")
        lp = logp_from_logits(logits.reshape(-1, logits.shape[-1]), token_ids.reshape(-1), temperature=temperature).view(token_ids.shape)
        if mask is not None:
            lp = lp.masked_fill(~mask.bool(), 0.0)
        return lp.to(output_dtype)


class ReferenceModelWrapper(PolicyModelWrapper):
    """The frozen reference of the KL penalty: parameters without gradients, eval mode, no autograd graph."""

    def __init__(self, model: torch.nn.Module, *, freeze: bool = True, eval_mode: bool = True):
        super().__init__(model)
        if freeze:
            self.freeze()
        if eval_mode:
            self.eval()

    def freeze(self) -> "ReferenceModelWrapper":
        for p in self.model.parameters():
            p.requires_grad_(False)
        return self

    def forward_logits(self, input_ids: torch.Tensor, **model_kwargs: Any) -> torch.Tensor:
        with torch.no_grad():
            return super().forward_logits(input_ids, **model_kwargs)

    def selected_logprobs(self, input_ids: torch.Tensor, token_ids: torch.Tensor, **kw: Any) -> torch.Tensor:
        with torch.no_grad():
            return super().selected_logprobs(input_ids, token_ids, **kw)


__all__ = ["PolicyModelWrapper", "ReferenceModelWrapper", "extract_logits"]
