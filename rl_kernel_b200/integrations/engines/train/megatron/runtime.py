"""Megatron-style training binding (parity: rl_engine/integrations/engines/train/megatron/
runtime.py:384-1170): deterministic TP reduce / copy autograd functions, canonical column and
row projections, RMSNorm replacement and the log-prob output layer.  Classes to patch are passed in,
so stand-ins work without Megatron-LM."""
from __future__ import annotations

import torch

from rl_kernel_b200.integrations.common.runtime import FrameworkOperatorIntegration
from rl_kernel_b200.integrations.engines.train.megatron.operators import (MegatronAttentionOperator,
                                                                           MegatronFFNOperator, MegatronLogpOperator)
from rl_kernel_b200.ops.attention.projection import _SPAllGather, _SPReduceScatter, _TPAllReduce, _TPCopy
from rl_kernel_b200.ops.gemm.det_gemm import det_gemm_linear
from rl_kernel_b200.runtime.plan import IntegrationPlan

DeterministicTPReduce = _TPAllReduce
DeterministicTPCopy = _TPCopy


class CanonicalColumnProjection(torch.nn.Module):
    """y_local = x @ W_local^T; backward all-reduces dX with the fixed tree."""

    def __init__(self, weight: torch.Tensor, collective=None, sequence_parallel: bool = False):
        super().__init__()
        self.weight = torch.nn.Parameter(weight)
        self.collective = collective
        self.sequence_parallel = sequence_parallel       # x holds this rank's token rows: all-gather before the GEMM

    def forward(self, x):
        enter = _SPAllGather if self.sequence_parallel else _TPCopy
        return det_gemm_linear(enter.apply(x, self.collective), self.weight)


class DeterministicTPOutputProjection(torch.nn.Module):
    """y = all_reduce_tree(x_local @ W_local^T) with canonical K chunks."""

    def __init__(self, weight: torch.Tensor, canonical_tp: int = 8, tp_size: int = 1, collective=None,
                 sequence_parallel: bool = False):
        super().__init__()
        self.weight = torch.nn.Parameter(weight)
        self.nchunks, self.collective = canonical_tp // tp_size, collective
        self.sequence_parallel = sequence_parallel       # the sum is reduce-scattered back to token rows

    def forward(self, x):
        leave = _SPReduceScatter if self.sequence_parallel else _TPAllReduce
        return leave.apply(det_gemm_linear(x, self.weight, self.nchunks), self.collective)


def install_megatron_integration(*, attention_cls=None, mlp_cls=None, norm_cls=None, output_layer_cls=None,
                                 plan: IntegrationPlan | None = None, tp_size: int = 1, cp_size: int = 1,
                                 collective=None, temperature: float = 1.0, cp_rank: int = 0, tp_rank: int = 0,
                                 cp_collective=None, cp_communication=None, cp_core=None, sequence_parallel: bool = False,
                                 canonical_cp_classes: dict | None = None) -> FrameworkOperatorIntegration:
    """``cp_collective`` (+ ``cp_rank``): context-parallel attention through the native peer-memory operator, or
    through ``cp_communication`` (a gather/scatter object) on transports without peer memory.
    ``canonical_cp_classes``: keyword arguments for ``canonical_cp.install`` (model / embedding / checkpoint classes,
    loss module, parallel state) to make parameter gradients layout-invariant under CP."""
    plan = plan or IntegrationPlan.from_env()
    integ = FrameworkOperatorIntegration("megatron", "train", plan)
    want = plan.side("train")
    if canonical_cp_classes:
        from rl_kernel_b200.distributed.algorithms import canonical_cp

        canonical_cp.install(**canonical_cp_classes)
    if want["attention"] and attention_cls is not None:
        integ.install("attention", MegatronAttentionOperator(cp_size=cp_size, cp_rank=cp_rank, cp_collective=cp_collective,
                                                             communication=cp_communication, core=cp_core,
                                                             tp_size=tp_size, tp_rank=tp_rank))
        setattr(attention_cls, "_rlk_orig_core", getattr(attention_cls, "core_attention", None))
        attention_cls.core_attention = lambda self, q, k, v, **kw: integ.execute("attention", self, q, k, v, **kw)
    if want["ffn"] and mlp_cls is not None:
        integ.install("ffn", MegatronFFNOperator(tp_size=tp_size, collective=collective, sequence_parallel=sequence_parallel))
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
