"""Policy ratio and k3 reference-KL per token from logits
(parity: NativeRatioKLOp, rl_engine/reference/loss/ratio_kl.py:12-75)."""
from __future__ import annotations

import torch

from rl_kernel_b200.reference.logprob.logp import NativeLogpOp


def ratio_kl_from_logps(logp, old_logp, ref_logp, mask):
    m = mask.bool()
    delta = (logp - old_logp.float()).masked_fill(~m, 0.0)
    ratio = torch.exp(delta)
    if ref_logp is None:
        return ratio, torch.zeros_like(ratio)
    diff = (ref_logp.float() - logp).masked_fill(~m, 0.0)
    return ratio, torch.exp(diff) - diff - 1.0


class NativeRatioKLOp:
    def __init__(self):
        self._logp = NativeLogpOp()

    def __call__(self, policy_logits, ref_logits, action_ids, attention_mask, old_logps):
        mask = attention_mask.bool()
        vocab = policy_logits.size(-1)
        bad = mask & ((action_ids < 0) | (action_ids >= vocab))
        if bad.any():
            raise ValueError(f"action_ids at active positions must be in [0, {vocab})")
        ids = action_ids.masked_fill(~mask, 0)
        off = ~mask.unsqueeze(-1)
        lp = self._logp.apply_fp32(policy_logits.masked_fill(off, 0.0), ids)
        with torch.no_grad():
            lr = self._logp.apply_fp32(ref_logits.masked_fill(off, 0.0), ids)
        return ratio_kl_from_logps(lp, old_logps, lr, mask)

    forward = __call__
