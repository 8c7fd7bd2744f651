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


# ------------------------------------------------------------------------------------------------ registry view
# Which adapter serves which node of the model chain, what the backend profiles of the manifest expect there, and
# whether that is covered (parity: GradientAdapterSpec / AdapterStatusRow / gradient_adapter_status_matrix,
# rl_engine/validation/operators/gradient_adapters.py:44-307, 1221-1354).
from pathlib import Path  # noqa: E402
from typing import Any, Sequence  # noqa: E402

from rl_kernel_b200.config.workload import profile_required_nodes  # noqa: E402
from rl_kernel_b200.validation.operators.operator_specs import _load_object  # noqa: E402

# chain node of the manifest -> operator of the harness that judges it
CHAIN_NODE_OPERATORS: dict[str, str] = {
    "embedding": "embedding", "input_layernorm": "rms_norm", "qkv_proj": "det_gemm", "qk_norm": "qk_norm", "rope": "rope",
    "attention": "attention", "o_proj": "det_gemm", "post_attention_layernorm": "rms_norm", "gate_up_proj": "det_gemm", "swiglu": "swiglu",
    "down_proj": "det_gemm", "final_layernorm": "rms_norm", "lm_head": "lm_head", "logprob": "linear_logp"}
# operators outside the chain: fused or layout-only forms that a profile may or may not ask for
OPTIONAL_FUSED = ("batch_invariant_logp", "logp", "kv_cache_attention", "prefix_shared_attention", "matmul", "silu", "grpo_loss")
LAYOUT_SUPPORTED = ("pack",)
PROFILE_CANDIDATE = {"b200": "b200", "reference": "pytorch", "pytorch": "pytorch"}
REPO_ROOT = Path(__file__).resolve().parents[3]


@dataclass(frozen=True)
class GradientAdapterSpec:
    op_name: str
    chain_nodes: tuple[str, ...]
    op_class: str
    adapter: str
    token_inputs: tuple[str, ...]
    parameter_inputs: tuple[str, ...]
    requirement: str                      # required | optional_fused | layout_supported | forward_only
    source_files: tuple[str, ...]
    shape_dependent_bwd_accum: str = "forbidden"
    atomic_add: str = "forbidden"

    @property
    def grad_tensor_names(self) -> tuple[str, ...]:
        return self.token_inputs + self.parameter_inputs


def _source_files(spec) -> tuple[str, ...]:
    out = []
    for path in (spec.gold_path, *spec.candidate_paths.values()):
        mod = path.rsplit(".", 1)[0].replace("rl_engine.", "rl_kernel_b200.", 1).replace(".", "/")
        for cand in (f"{mod}.py", f"{mod}/__init__.py"):
            if (REPO_ROOT / cand).exists() and cand not in out:
                out.append(cand)
    return tuple(out)


def _adapter_spec(name: str) -> GradientAdapterSpec:
    spec = OP_SPECS[name]
    nodes = tuple(n for n, op in CHAIN_NODE_OPERATORS.items() if op == name)
    req = ("layout_supported" if name in LAYOUT_SUPPORTED else "required" if nodes else "optional_fused")
    if not spec.grad_input_names and req != "layout_supported":
        req = "forward_only" if not nodes else req
    return GradientAdapterSpec(name, nodes, spec.op_class, spec.adapter, tuple(n for n in spec.grad_input_names if n in TOKEN_INPUTS),
                               tuple(n for n in spec.grad_input_names if n in PARAMETER_INPUTS), req, _source_files(spec))


ADAPTER_SPECS: dict[str, GradientAdapterSpec] = {name: _adapter_spec(name) for name in OP_SPECS}


def adapter_names() -> tuple[str, ...]:
    return tuple(ADAPTER_SPECS)


def get_adapter(op_name: str) -> GradientAdapterSpec:
    try:
        return ADAPTER_SPECS[op_name]
    except KeyError as exc:
        raise KeyError(f"unknown gradient adapter {op_name!r}") from exc


def required_gradient_adapters() -> tuple[GradientAdapterSpec, ...]:
    return tuple(a for a in ADAPTER_SPECS.values() if a.requirement in ("required", "layout_supported") and a.grad_tensor_names)


def required_forward_adapters() -> tuple[GradientAdapterSpec, ...]:
    """The forward judgments enumerate the same registry (there is no second list to fall out of step)."""
    return tuple(a for a in ADAPTER_SPECS.values() if a.requirement in ("required", "layout_supported"))


@dataclass(frozen=True)
class AdapterStatusRow:
    op_name: str
    chain_node: str
    backend_profile: str
    requirement: str
    candidate_status: str                 # declared | optional | absent_not_required | untracked_missing_node | missing_candidate
    adapter_registered: bool
    expected_backend_id: str | None
    candidate_path: str | None
    tracked_red: bool                     # the profile asks for it and says it is missing
    untracked_red: bool                   # the profile asks for it and nothing here can judge it
    grad_tensor_names: tuple[str, ...]

    def to_dict(self) -> dict[str, Any]:
        return dict(self.__dict__)


def resolve_profile_candidate(adapter: GradientAdapterSpec, profile: str, manifest=None, node: str | None = None) -> dict[str, Any]:
    m = manifest or load_manifest()
    family = m.backend_profiles[profile]["backend_family"]
    cand = PROFILE_CANDIDATE.get(family, family)
    spec = OP_SPECS[adapter.op_name]
    if adapter.requirement == "layout_supported":
        return {"status": "declared", "expected_backend_id": cand if cand in spec.candidate_paths else "pytorch",
                "candidate_path": spec.candidate_paths.get(cand, spec.candidate_paths.get("pytorch"))}
    asked = set(profile_required_nodes(m, profile))
    nodes = [node] if node else list(adapter.chain_nodes)
    if not nodes:
        return {"status": "optional" if adapter.requirement == "optional_fused" else "absent_not_required", "expected_backend_id": None,
                "candidate_path": spec.candidate_paths.get(cand)}
    if not any(n in asked for n in nodes):
        return {"status": "untracked_missing_node", "expected_backend_id": None, "candidate_path": None}
    path = spec.candidate_paths.get(cand)
    return {"status": "declared" if path else "missing_candidate", "expected_backend_id": cand, "candidate_path": path}


def gradient_adapter_status_matrix(manifest=None, profiles: Sequence[str] | None = None) -> tuple[AdapterStatusRow, ...]:
    """One row per (backend profile, chain node) plus one per operator outside the chain.  ``untracked_red`` rows are the
    ones a green matrix must not have: a node the profile runs with no adapter or no candidate to judge it."""
    m = manifest or load_manifest()
    rows: list[AdapterStatusRow] = []
    for profile in (profiles or tuple(m.backend_profiles)):
        for node in profile_required_nodes(m, profile):
            op = CHAIN_NODE_OPERATORS.get(node)
            if op is None or op not in ADAPTER_SPECS:
                rows.append(AdapterStatusRow(op or "?", node, profile, "required", "untracked_missing_node", False, None, None, False, True, ()))
                continue
            a = ADAPTER_SPECS[op]
            r = resolve_profile_candidate(a, profile, m, node)
            rows.append(AdapterStatusRow(op, node, profile, a.requirement, r["status"], True, r["expected_backend_id"], r["candidate_path"],
                                         False, r["status"] in ("missing_candidate", "untracked_missing_node"), a.grad_tensor_names))
        for a in ADAPTER_SPECS.values():
            if a.chain_nodes:
                continue
            r = resolve_profile_candidate(a, profile, m)
            rows.append(AdapterStatusRow(a.op_name, "-", profile, a.requirement, r["status"], True, r["expected_backend_id"], r["candidate_path"],
                                         False, False, a.grad_tensor_names))
    return tuple(rows)


def load_adapter_operator(op_name: str, candidate: str) -> Any:
    spec = OP_SPECS[get_adapter(op_name).op_name]
    if candidate not in spec.candidate_paths:
        raise RuntimeError(f"operator {op_name!r} has no candidate {candidate!r}; it has {sorted(spec.candidate_paths)}")
    return _load_object(spec.candidate_paths[candidate])()


def load_adapter_gold(op_name: str) -> Any:
    """The fp32 definition an operator is judged against: the harness's own formula where it has one (plain PyTorch on
    the logical values), else the method of the reference operator the spec names."""
    from rl_kernel_b200.validation.operators.operator_specs import GOLD

    spec = OP_SPECS[get_adapter(op_name).op_name]
    if spec.name in GOLD:
        return GOLD[spec.name]
    obj = _load_object(spec.gold_path)()
    for method in (spec.gold_method, "forward_fp32", "forward", "__call__"):
        if hasattr(obj, method):
            return getattr(obj, method)
    raise RuntimeError(f"gold of {op_name!r} ({spec.gold_path}) exposes none of the expected methods")


def listed_source_paths(adapter: GradientAdapterSpec) -> list[Path]:
    return [REPO_ROOT / rel for rel in adapter.source_files]


__all__ = ["ADAPTER_SPECS", "AdapterStatusRow", "CHAIN_NODE_OPERATORS", "GRADIENT_ADAPTERS", "GradientAdapterInfo", "GradientAdapterSpec",
           "PARAMETER_INPUTS", "TOKEN_INPUTS", "adapter_names", "get_adapter", "gradient_adapter_info", "gradient_adapter_status_matrix",
           "listed_source_paths", "load_adapter_gold", "load_adapter_operator", "required_forward_adapters", "required_gradient_adapters",
           "resolve_profile_candidate", "run_gradient_case"]
