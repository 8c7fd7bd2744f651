"""Plain softmax attention with GQA, causal and key-padding masks (the fp32 gold;
parity: NativeAttentionOp, rl_engine/reference/attention/standard_attn.py:13)."""
from __future__ import annotations

import math

import torch


class NativeAttentionOp:
    def __call__(self, q, k, v, *, causal: bool = True, key_padding_mask=None, scale: float | None = None,
                 q_pos0: int | None = None, return_lse: bool = False):
        """q [B, Sq, Hq, D]; k, v [B, Skv, Hkv, D]. Query i sits at key position q_pos0 + i
        (default Skv - Sq, i.e. the queries are the last Sq positions)."""
        B, Sq, Hq, D = q.shape
        Skv, Hkv = k.shape[1], k.shape[2]
        g = Hq // Hkv
        scale = scale if scale is not None else 1.0 / math.sqrt(D)
        qf = q.float().permute(0, 2, 1, 3)
        kf = k.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
        vf = v.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
        s = qf @ kf.transpose(-1, -2) * scale
        if causal:
            p0 = Skv - Sq if q_pos0 is None else q_pos0
            qpos = torch.arange(Sq, device=q.device)[:, None] + p0
            kpos = torch.arange(Skv, device=q.device)[None, :]
            s = s.masked_fill(kpos > qpos, float("-inf"))
        if key_padding_mask is not None:
            s = s.masked_fill(~key_padding_mask.bool()[:, None, None, :], float("-inf"))
        lse = torch.logsumexp(s, dim=-1)
        p = torch.exp(s - lse.unsqueeze(-1))
        p = torch.nan_to_num(p, nan=0.0)
        o = (p @ vf).permute(0, 2, 1, 3).to(q.dtype)
        return (o, lse.permute(0, 2, 1)) if return_lse else o

    forward = __call__
