"""Row-local fp32 VJPs used by validation to check native backward kernels
(parity: rl_engine/ops/autograd/vjp_fp32.py:22-131)."""
from __future__ import annotations

import torch


def rms_norm_vjp_fp32(x: torch.Tensor, w: torch.Tensor, dy: torch.Tensor, eps: float = 1e-6):
    xf, wf, g = x.float(), w.float(), dy.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    xh = xf * rstd
    wg = wf * g
    dx = rstd * (wg - xh * (wg * xh).mean(-1, keepdim=True))
    return dx, (g * xh).reshape(-1, x.shape[-1]).sum(0)


def swiglu_vjp_fp32(gate: torch.Tensor, up: torch.Tensor, dout: torch.Tensor):
    g, u, d = gate.float(), up.float(), dout.float()
    sig = torch.sigmoid(g)
    return d * u * sig * (1 + g * (1 - sig)), d * g * sig
