"""Operator specs for validation: how to build inputs, the fp32 gold, the candidate, and which
invariance transformations apply (parity: OP_SPECS of tools/validation/operators/check_operator.py)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch


@dataclass(frozen=True)
class OpSpec:
    name: str
    make_inputs: Callable[[int, torch.device, torch.dtype, int], dict]   # (rows, device, dtype, seed) -> inputs
    gold: Callable[[dict], torch.Tensor]
    candidate: Callable[[dict], torch.Tensor]
    row_inputs: tuple[str, ...]          # inputs whose first dim is the batch/token dim
    grad_inputs: tuple[str, ...] = ()    # inputs that receive gradients
    out_dtype: str = "bfloat16"


def _mk(shape, gen, device, dtype, scale=1.0):
    return (torch.randn(shape, generator=gen) * scale).to(device=device, dtype=dtype)


def _gemm_inputs(rows, device, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    return {"x": _mk((rows, 256), g, device, dtype), "w": _mk((128, 256), g, device, dtype, 0.05)}


def _norm_inputs(rows, device, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    return {"x": _mk((rows, 256), g, device, dtype), "w": (1 + 0.1 * torch.randn(256, generator=g)).to(device=device, dtype=dtype)}


def _swiglu_inputs(rows, device, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    return {"gu": _mk((rows, 512), g, device, dtype)}


def _logp_inputs(rows, device, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    return {"hidden": _mk((rows, 128), g, device, dtype), "w": _mk((512, 128), g, device, dtype, 0.1),
            "targets": torch.randint(0, 512, (rows,), generator=g).to(device)}


def build_specs() -> dict[str, OpSpec]:
    from rl_kernel_b200.ops.activation import swiglu_packed
    from rl_kernel_b200.ops.gemm.det_gemm import det_gemm_linear
    from rl_kernel_b200.ops.logprob import linear_logp
    from rl_kernel_b200.ops.norm import rms_norm

    def rms_gold(i):
        x, w = i["x"].float(), i["w"].float()
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w

    def swiglu_gold(i):
        g, u = i["gu"].float().chunk(2, -1)
        return torch.nn.functional.silu(g) * u

    def logp_gold(i):
        return torch.log_softmax(i["hidden"].float() @ i["w"].float().t(), -1).gather(1, i["targets"][:, None])[:, 0]

    return {
        "det_gemm": OpSpec("det_gemm", _gemm_inputs, lambda i: i["x"].float() @ i["w"].float().t(),
                           lambda i: det_gemm_linear(i["x"], i["w"]), ("x",), ("x", "w")),
        "rms_norm": OpSpec("rms_norm", _norm_inputs, rms_gold, lambda i: rms_norm(i["x"], i["w"]), ("x",), ("x", "w")),
        "swiglu": OpSpec("swiglu", _swiglu_inputs, swiglu_gold, lambda i: swiglu_packed(i["gu"]), ("gu",), ("gu",)),
        "linear_logp": OpSpec("linear_logp", _logp_inputs, logp_gold,
                              lambda i: linear_logp(i["hidden"], i["w"], i["targets"]), ("hidden", "targets"),
                              ("hidden", "w"), "float32"),
    }
