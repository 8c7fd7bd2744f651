"""Megatron-style training binding (parity: rl_engine/integrations/engines/train/megatron/
runtime.py:384-1170): deterministic TP reduce / copy autograd functions, canonical column and
row projections, RMSNorm replacement and the log-prob output layer.  Classes to patch are passed in,
so stand-ins work without Megatron-LM."""
from __future__ import annotations

import torch

from rl_kernel_b200.integrations.common.runtime import FrameworkOperatorIntegration
from rl_kernel_b200.integrations.engines.train.megatron.operators import (MegatronAttentionOperator,
                                                                           MegatronFFNOperator, MegatronLogpOperator)
from rl_kernel_b200.ops.attention.projection import _TPAllReduce, _TPCopy
from rl_kernel_b200.ops.gemm.det_gemm import det_gemm_linear
from rl_kernel_b200.runtime.plan import IntegrationPlan

DeterministicTPReduce = _TPAllReduce
DeterministicTPCopy = _TPCopy


class CanonicalColumnProjection(torch.nn.Module):
    """y_local = x @ W_local^T; backward all-reduces dX with the fixed tree."""

    def __init__(self, weight: torch.Tensor, collective=None):
        super().__init__()
        self.weight = torch.nn.Parameter(weight)
        self.collective = collective

    def forward(self, x):
        return det_gemm_linear(_TPCopy.apply(x, self.collective), self.weight)


class DeterministicTPOutputProjection(torch.nn.Module):
    """y = all_reduce_tree(x_local @ W_local^T) with canonical K chunks."""

    def __init__(self, weight: torch.Tensor, canonical_tp: int = 8, tp_size: int = 1, collective=None):
        super().__init__()
        self.weight = torch.nn.Parameter(weight)
        self.nchunks, self.collective = canonical_tp // tp_size, collective

    def forward(self, x):
        return _TPAllReduce.apply(det_gemm_linear(x, self.weight, self.nchunks), self.collective)


def install_megatron_integration(*, attention_cls=None, mlp_cls=None, norm_cls=None, output_layer_cls=None,
                                 plan: IntegrationPlan | None = None, tp_size: int = 1, cp_size: int = 1,
                                 collective=None, temperature: float = 1.0) -> FrameworkOperatorIntegration:
    plan = plan or IntegrationPlan.from_env()
    integ = FrameworkOperatorIntegration("megatron", "train", plan)
    want = plan.side("train")
    if want["attention"] and attention_cls is not None:
        integ.install("attention", MegatronAttentionOperator(cp_size=cp_size))
        setattr(attention_cls, "_rlk_orig_core", getattr(attention_cls, "core_attention", None))
        attention_cls.core_attention = lambda self, q, k, v, **kw: integ.execute("attention", self, q, k, v, **kw)
    if want["ffn"] and mlp_cls is not None:
        integ.install("ffn", MegatronFFNOperator(tp_size=tp_size, collective=collective))
        setattr(mlp_cls, "_rlk_orig_forward", getattr(mlp_cls, "forward", None))
        mlp_cls.forward = lambda self, x: integ.execute("ffn", self, x)
    if want["logp"] and output_layer_cls is not None:
        integ.install("logp", MegatronLogpOperator(temperature=temperature))
        output_layer_cls.selected_logprobs = lambda self, hidden, targets: integ.execute("logp", self, hidden, targets)
    if norm_cls is not None:
        from rl_kernel_b200.ops.norm import rms_norm

        norm_cls.forward = lambda self, x: rms_norm(x, self.weight, getattr(self, "eps", 1e-6))
    return integ


def initialize_from_environment(**classes):
    import os

    if os.environ.get("RL_KERNEL_MEGATRON_INTEGRATION", "0") in ("1", "true", "True"):
        return install_megatron_integration(**classes)
    return None
