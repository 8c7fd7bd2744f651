"""Sampler front end (parity: SamplerBackend, rl_engine/ops/sampling/api.py:12-79; FlashInfer is
replaced by the Gumbel-max kernel of csrc/sampling/sampling.cu)."""
from __future__ import annotations

import enum

import torch

from rl_kernel_b200.ops._dispatch import use_native
from rl_kernel_b200.ops.sampling.policy import keep_threshold
from rl_kernel_b200.reference.sampling.policy import sample_from_logits


class SamplerBackend(str, enum.Enum):
    B200 = "b200"
    TORCH = "torch"


def sample(logits: torch.Tensor, *, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0, seed: int = 0,
           step: int = 0, row_keys: torch.Tensor | None = None, greedy: bool = False, real_vocab: int | None = None,
           generator=None) -> torch.Tensor:
    """One id per row of ``logits`` [rows, V]."""
    if not use_native(logits):
        if greedy:
            return logits[:, :real_vocab].argmax(-1) if real_vocab else logits.argmax(-1)
        return sample_from_logits(logits, temperature=temperature, top_k=top_k, top_p=top_p, generator=generator,
                                  real_vocab=real_vocab)
    from rl_kernel_b200.backends import native as nv

    lg = logits if real_vocab is None else logits[:, :real_vocab]
    if lg.shape[1] % 8:
        raise ValueError("the sampler needs a vocab size that is a multiple of 8")
    thr = keep_threshold(lg, temperature=temperature, top_k=top_k, top_p=top_p)
    ids = torch.empty(lg.shape[0], device=lg.device, dtype=torch.int64)
    nv.sample_gumbel(lg, ids, None, vocab_start=0, inv_temp=1.0 / max(temperature, 1e-6), seed=seed, step=step,
                     greedy=greedy, min_keep=thr, row_keys=row_keys)
    return ids
