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


class MegatronUnavailable(RuntimeError):
    """Megatron-LM (``megatron.core``) cannot be imported here."""


_ORIGINALS = "__rl_kernel_originals__"


def _patch(cls, name: str, new) -> None:
    """Replace ``cls.name`` once, remembering the original (absent attributes are remembered as absent) so that
    ``uninstall_megatron_integration`` can put the class back."""
    saved = cls.__dict__.get(_ORIGINALS)
    if saved is None:
        saved = {}
        setattr(cls, _ORIGINALS, saved)
    if name not in saved:
        saved[name] = cls.__dict__.get(name, _ABSENT)
    setattr(cls, name, new)


_ABSENT = object()


def _hook_id(cls, name: str) -> str:
    return f"{cls.__module__}.{cls.__qualname__}.{name}"


def resolve_megatron_classes() -> dict:
    """The Megatron-LM classes this binding patches, by their import paths in ``megatron.core``."""
    try:
        from megatron.core.tensor_parallel.layers import ColumnParallelLinear, RowParallelLinear  # type: ignore
        from megatron.core.transformer.dot_product_attention import DotProductAttention  # type: ignore
        from megatron.core.transformer.mlp import MLP  # type: ignore
    except Exception as exc:  # noqa: BLE001
        raise MegatronUnavailable("megatron.core is not importable; pass the classes to patch explicitly") from exc
    return {"attention_cls": DotProductAttention, "mlp_cls": MLP, "column_linear_cls": ColumnParallelLinear,
            "row_linear_cls": RowParallelLinear}


def install_megatron_integration(*, attention_cls=None, mlp_cls=None, norm_cls=None, output_layer_cls=None,
                                 column_linear_cls=None, row_linear_cls=None,
                                 plan: IntegrationPlan | None = None, tp_size: int = 1, cp_size: int = 1,
                                 collective=None, temperature: float = 1.0, cp_rank: int = 0, tp_rank: int = 0,
                                 cp_collective=None, cp_communication=None, cp_core=None, sequence_parallel: bool = False,
                                 canonical_tp: int = 8, canonical_cp_classes: dict | None = None) -> FrameworkOperatorIntegration:
    """Patch the given Megatron classes so that the modules the plan gives to RL-Kernel on the training side run this
    package's operators.  Every patched method is recorded as an installed hook; ``uninstall_megatron_integration``
    restores the classes.

    ``cp_collective`` (+ ``cp_rank``): context-parallel attention through the native peer-memory operator, or through
    ``cp_communication`` (a gather / scatter object) on transports without peer memory.  ``column_linear_cls`` /
    ``row_linear_cls``: the tensor-parallel linear layers (QKV / gate-up and output / down projections); their forward
    becomes the deterministic GEMM with the fixed-tree collectives and returns Megatron's ``(output, bias)`` pair.
    ``canonical_cp_classes``: keyword arguments for ``canonical_cp.install`` to make parameter gradients
    layout-invariant under CP."""
    plan = plan or IntegrationPlan.from_env()
    integ = FrameworkOperatorIntegration("megatron", "train", plan)
    want = plan.side("train")
    patched: list[tuple[type, str]] = []

    def hook(module: str, cls, name: str, fn) -> None:
        _patch(cls, name, fn)
        patched.append((cls, name))
        integ.record_installed_hook(module, _hook_id(cls, name))

    if canonical_cp_classes:
        from rl_kernel_b200.distributed.algorithms import canonical_cp

        canonical_cp.install(**canonical_cp_classes)
    if want["attention"] and attention_cls is not None:
        integ.install("attention", MegatronAttentionOperator(cp_size=cp_size, cp_rank=cp_rank, cp_collective=cp_collective,
                                                             communication=cp_communication, core=cp_core,
                                                             tp_size=tp_size, tp_rank=tp_rank))
        if not hasattr(attention_cls, "_rlk_orig_core"):
            setattr(attention_cls, "_rlk_orig_core", getattr(attention_cls, "core_attention", None))
        hook("attention", attention_cls, "core_attention", lambda self, q, k, v, **kw: integ.execute("attention", self, q, k, v, **kw))
    if want["ffn"] and mlp_cls is not None:
        integ.install("ffn", MegatronFFNOperator(canonical_tp=canonical_tp, tp_size=tp_size, collective=collective,
                                                 sequence_parallel=sequence_parallel))
        if not hasattr(mlp_cls, "_rlk_orig_forward"):
            setattr(mlp_cls, "_rlk_orig_forward", getattr(mlp_cls, "forward", None))
        hook("ffn", mlp_cls, "forward", lambda self, x: integ.execute("ffn", self, x))
    if want["logp"] and output_layer_cls is not None:
        integ.install("logp", MegatronLogpOperator(temperature=temperature))
        hook("logp", output_layer_cls, "selected_logprobs", lambda self, hidden, targets: integ.execute("logp", self, hidden, targets))
    if (want["attention"] or want["ffn"]) and column_linear_cls is not None:
        def column_forward(self, x, *_a, **_k):
            enter = _SPAllGather if sequence_parallel else _TPCopy
            y = det_gemm_linear(enter.apply(x.reshape(-1, x.shape[-1]), collective if tp_size > 1 else None), self.weight)
            y = y.reshape(*x.shape[:-1], -1) if not sequence_parallel else y
            bias = getattr(self, "bias", None)
            return (y, bias) if getattr(self, "skip_bias_add", False) or bias is None else (y + bias, None)

        hook("attention" if want["attention"] else "ffn", column_linear_cls, "forward", column_forward)
    if (want["attention"] or want["ffn"]) and row_linear_cls is not None:
        nchunks = canonical_tp // tp_size

        def row_forward(self, x, *_a, **_k):
            leave = _SPReduceScatter if sequence_parallel else _TPAllReduce
            y = leave.apply(det_gemm_linear(x.reshape(-1, x.shape[-1]), self.weight, nchunks), collective if tp_size > 1 else None)
            y = y.reshape(*x.shape[:-1], -1) if not sequence_parallel else y
            bias = getattr(self, "bias", None)
            return (y, bias) if getattr(self, "skip_bias_add", False) or bias is None else (y + bias, None)

        hook("attention" if want["attention"] else "ffn", row_linear_cls, "forward", row_forward)
    if norm_cls is not None:
        from rl_kernel_b200.ops.norm import rms_norm

        _patch(norm_cls, "forward", lambda self, x: rms_norm(x, self.weight, getattr(self, "eps", 1e-6)))
        patched.append((norm_cls, "forward"))
    integ.patched = patched
    return integ


def uninstall_megatron_integration(integ: FrameworkOperatorIntegration) -> int:
    """Put back every attribute ``install_megatron_integration`` replaced; returns how many were restored."""
    n = 0
    for cls, name in getattr(integ, "patched", []):
        saved = cls.__dict__.get(_ORIGINALS, {})
        if name in saved:
            orig = saved.pop(name)
            if orig is _ABSENT:
                if name in cls.__dict__:
                    delattr(cls, name)
            else:
                setattr(cls, name, orig)
            n += 1
    integ.patched = []
    return n


def initialize_from_environment(**classes):
    import os

    if os.environ.get("RL_KERNEL_MEGATRON_INTEGRATION", "0") in ("1", "true", "True"):
        if not classes:
            classes = resolve_megatron_classes()
        return install_megatron_integration(**classes)
    return None
