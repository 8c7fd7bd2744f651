"""Gradient adapters of the operator harness (parity: rl_engine/validation/operators/gradient_adapters.py:1-1354).

An adapter knows how to (a) lay an operator's differentiable inputs out for one batch configuration, (b) run forward and
backward with an upstream gradient that is a fixed value per logical token and exactly zero on padding, and (c) hand the
gradients back keyed by logical token (token inputs) or as whole tensors (parameters).  The adapters live with the forward
adapters in ``operator_specs`` -- one object per operator kind does both directions -- and this module exposes the
gradient side: which inputs of which operator are differentiated, how parameter gradients are judged, and a one-call
runner."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from rl_kernel_b200.config.workload import build_logical_batch, load_manifest
from rl_kernel_b200.validation.operators.forward_invariance import ConfigSpec, _run_config, build_config_matrix
from rl_kernel_b200.validation.operators.operator_specs import ADAPTERS, OP_SPECS, make_candidate, make_operator_case

TOKEN_INPUTS = {"x", "gate", "up", "q", "k", "v", "logp"}
"""Inputs that carry one row per logical token: their gradients are keyed by token and must keep their bits under every
batch configuration."""
PARAMETER_INPUTS = {"weight"}
"""Inputs shared by all tokens: their gradient is a sum over tokens in physical order, so its bits follow the order; it
is bit-compared where the order is the same and bounded relatively elsewhere."""


@dataclass(frozen=True)
class GradientAdapterInfo:
    op_name: str
    adapter: str
    token_inputs: tuple[str, ...]
    parameter_inputs: tuple[str, ...]


def gradient_adapter_info(op_name: str) -> GradientAdapterInfo:
    spec = OP_SPECS[op_name]
    return GradientAdapterInfo(op_name, spec.adapter, tuple(n for n in spec.grad_input_names if n in TOKEN_INPUTS),
                               tuple(n for n in spec.grad_input_names if n in PARAMETER_INPUTS))


GRADIENT_ADAPTERS = {name: gradient_adapter_info(name) for name, spec in OP_SPECS.items() if spec.grad_input_names}


def run_gradient_case(op_name: str, config: ConfigSpec | str = "BN/full", *, candidate: str = "auto", device: str = "cpu",
                      dtype: torch.dtype | None = None, seed: int = 0, manifest=None) -> dict:
    """Forward + backward of ``op_name`` under one configuration -> {"out": {token: tensor}, "grads": {input: ...}}."""
    if op_name not in GRADIENT_ADAPTERS:
        raise KeyError(f"operator {op_name!r} has no differentiable inputs")
    m = manifest or load_manifest()
    if isinstance(config, str):
        config = next(c for c in build_config_matrix(m) if c.config_id == config)
    batch = build_logical_batch(m)
    cand = make_candidate(op_name=op_name, candidate=candidate, device=device, dtype=dtype)
    spec, adapter, st = make_operator_case(op_name, batch=batch, device=cand.device, dtype=cand.dtype, seed=seed)
    with torch.enable_grad():
        out, grads = _run_config(spec, adapter, cand, st, config, batch, m, True)
    return {"out": out, "grads": grads, "adapter": type(ADAPTERS[spec.adapter]).__name__}


__all__ = ["GRADIENT_ADAPTERS", "GradientAdapterInfo", "PARAMETER_INPUTS", "TOKEN_INPUTS", "gradient_adapter_info", "run_gradient_case"]
