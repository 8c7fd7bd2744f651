"""Tolerance resolution (parity: rl_engine/contracts/numerical.py:191-660, profile ws1.json).

Two kinds of judgment exist and must not be mixed: ACCURACY (candidate vs fp32 gold, within a
per-operator tolerance) and INVARIANCE (candidate vs itself under another batch / chunk / padding /
parallel layout: raw-bit equality, never a tolerance)."""
from __future__ import annotations

import json
from dataclasses import dataclass
from functools import lru_cache
from pathlib import Path

import torch

_PROFILE_DIR = Path(__file__).resolve().parent / "profiles" / "precision"


@dataclass(frozen=True)
class ToleranceSpec:
    atol: float
    rtol: float
    scale: str = "elementwise"   # or "row_abs_max": rtol applies to the largest |gold| of the row

    def check(self, candidate: torch.Tensor, gold: torch.Tensor) -> tuple[bool, float]:
        c, g = candidate.float(), gold.float()
        err = (c - g).abs()
        if self.scale == "row_abs_max":
            bound = self.atol + self.rtol * g.abs().amax(dim=-1, keepdim=True).expand_as(g)
        else:
            bound = self.atol + self.rtol * g.abs()
        worst = float((err - bound).max()) if err.numel() else 0.0
        return worst <= 0.0, float(err.max()) if err.numel() else 0.0


@lru_cache(maxsize=8)
def load_precision_profile(name: str = "ws1") -> dict:
    path = _PROFILE_DIR / f"{name}.json"
    data = json.loads(path.read_text())
    for key in ("profile_id", "defaults", "operators", "chain"):
        if key not in data:
            raise ValueError(f"precision profile {path} lacks {key!r}")
    return data


def resolve_tolerance(op_name: str, dtype: torch.dtype | str, profile: str = "ws1") -> ToleranceSpec:
    data = load_precision_profile(profile)
    key = str(dtype).removeprefix("torch.")
    entry = data["operators"].get(op_name, {}).get(key) or data["defaults"].get(key)
    if entry is None:
        raise KeyError(f"no tolerance for operator {op_name!r} dtype {key!r} in profile {profile!r}")
    return ToleranceSpec(float(entry["atol"]), float(entry["rtol"]), entry.get("scale", "elementwise"))


def load_contract(profile: str = "ws1") -> dict:
    """The whole precision profile (the tolerance contract) as a plain dict."""
    return load_precision_profile(profile)


def tolerance_contract_fingerprint(profile: str = "ws1") -> str:
    """sha256 of the canonical JSON of the profile: artifacts judged under different contracts never compare."""
    import hashlib

    return hashlib.sha256(json.dumps(load_precision_profile(profile), sort_keys=True, separators=(",", ":")).encode()).hexdigest()


def cross_config_threshold(dtype_a: str, dtype_b: str | None = None, profile: str = "ws1") -> float:
    """Fixed |dlogp| bound between a rollout and a training score computed in the given dtypes."""
    table = load_precision_profile(profile)["cross_config"]["fixed_threshold"]
    names = {"bf16": "bfloat16", "fp16": "float16", "fp32": "float32", "half": "float16", "float": "float32"}
    keys = [names.get(str(d).removeprefix("torch."), str(d).removeprefix("torch.")) for d in (dtype_a, dtype_b or dtype_a)]
    for k in keys:
        if k not in table:
            raise KeyError(f"no cross-config threshold for dtype {k!r}")
    return max(float(table[k]) for k in keys)


def chain_thresholds(profile: str = "ws1") -> dict:
    return dict(load_precision_profile(profile)["chain"])


# ================================================================================================ the full contract surface
# (parity: DtypePolicy / BackendProvenance / ToleranceSupport / ComparisonRoles / LogprobAggregates and their resolvers,
#  rl_engine/contracts/numerical.py:26-1062)
import math as _math
from dataclasses import asdict as _asdict
from typing import Any as _Any, Mapping as _Mapping

JUDGMENTS = ("forward_accuracy", "forward_invariance", "gradient_accuracy", "gradient_invariance")
OP_CLASSES = ("elementwise", "reduction", "logprob", "attention", "gather", "loss")
MANDATORY_DTYPES = ("float32", "bfloat16")
OPTIONAL_DTYPES = ("float16",)
OUT_OF_SCOPE_DTYPES = ("float8",)
ALL_DTYPES = MANDATORY_DTYPES + OPTIONAL_DTYPES + OUT_OF_SCOPE_DTYPES
CHAIN_AGGREGATE_METRICS = ("max_abs_dlogp", "approx_kl0", "clipfrac0")
INVARIANCE_JUDGMENTS = ("forward_invariance", "gradient_invariance")
REPORT_KINDS = ("forward_accuracy", "forward_invariance", "train_infer_logprob_parity", "gradient_accuracy", "gradient_invariance")


class ContractError(ValueError):
    pass


class ContractSchemaError(ContractError):
    pass


class ContractResolveError(ContractError):
    pass


@dataclass(frozen=True)
class DtypePolicy:
    execution_dtype: str
    accumulation_dtype: str
    reference_dtype: str
    output_dtype_default: str
    logprob_aggregates_dtype: str
    fp8: str
    fp16_status: str
    tf32_reference: str
    tf32_candidate_execution: str
    backend_profiles: tuple
    backend_private_tolerance_relaxation: bool

    def to_dict(self) -> dict:
        return _asdict(self)


@dataclass(frozen=True)
class BackendProvenance:
    """The backend and dtype facts a report persists; validated against the policy before a report counts."""
    backend_profile: str
    requested_backend: str
    actual_backend: str
    execution_dtype: str
    accumulation_dtype: str
    output_dtype: str
    reference_dtype: str
    candidate_tf32_enabled: bool
    reference_tf32_enabled: bool

    def to_dict(self) -> dict:
        return _asdict(self)


@dataclass(frozen=True)
class ToleranceSupport:
    judgment: str
    op_class: str
    dtype_name: str
    status: str              # applicable | optional | out_of_scope
    reason: str | None = None

    def to_dict(self) -> dict:
        return _asdict(self)


@dataclass(frozen=True)
class ComparisonRoles:
    report_kind: str
    comparison_lhs_role: str
    comparison_rhs_role: str

    def to_dict(self) -> dict:
        return _asdict(self)


@dataclass(frozen=True)
class JudgmentTolerance:
    """Resolved cell of (judgment, op class, dtype): ``mode`` is ``tolerance`` or ``bitwise``."""
    judgment: str
    op_class: str
    dtype_name: str
    status: str
    mode: str
    atol: float
    rtol: float
    comparison_lhs_role: str
    comparison_rhs_role: str
    backend_profile: str | None = None
    arch_key: str | None = None

    def to_dict(self) -> dict:
        return _asdict(self)

    def check(self, candidate: torch.Tensor, reference: torch.Tensor) -> tuple[bool, float]:
        if self.mode == "bitwise":
            same = candidate.dtype == reference.dtype and candidate.shape == reference.shape and bool(
                torch.equal(candidate.contiguous().view(torch.uint8), reference.contiguous().view(torch.uint8)))
            return same, 0.0 if same else float((candidate.double() - reference.double()).abs().max())
        return ToleranceSpec(self.atol, self.rtol).check(candidate, reference)


@dataclass(frozen=True)
class LogprobAggregates:
    max_abs_dlogp: float
    approx_kl0: float
    clipfrac0: float
    active_token_count: int
    clip_interval: tuple
    report_kind: str
    comparison_lhs_role: str
    comparison_rhs_role: str

    def to_dict(self) -> dict:
        d = _asdict(self)
        d["clip_interval"] = list(self.clip_interval)
        return d


@dataclass(frozen=True)
class AggregateMetricVerdict:
    metric: str
    value: float
    threshold: float
    passed: bool


@dataclass(frozen=True)
class LogprobAggregateVerdict:
    aggregates: LogprobAggregates
    metrics: tuple
    passed: bool
    report_kind: str
    comparison_lhs_role: str
    comparison_rhs_role: str

    def to_dict(self) -> dict:
        return {"aggregates": self.aggregates.to_dict(), "metrics": [_asdict(m) for m in self.metrics], "passed": self.passed,
                "report_kind": self.report_kind, "comparison_lhs_role": self.comparison_lhs_role, "comparison_rhs_role": self.comparison_rhs_role}


_DTYPE_ALIASES = {"bf16": "bfloat16", "bfloat16": "bfloat16", "fp16": "float16", "half": "float16", "float16": "float16", "fp32": "float32",
                  "float": "float32", "float32": "float32", "fp8": "float8", "float8": "float8", "float8_e4m3fn": "float8", "float8_e5m2": "float8"}


def normalize_dtype_name(dtype) -> str:
    name = str(dtype).removeprefix("torch.").strip().lower()
    if name not in _DTYPE_ALIASES:
        raise ContractResolveError(f"unknown dtype {dtype!r}")
    return _DTYPE_ALIASES[name]


def validate_contract_schema(contract: _Mapping[str, _Any]) -> None:
    for key in ("version", "policy", "comparison_roles", "judgments", "chain_logprob_aggregates", "batch_invariance"):
        if key not in contract:
            raise ContractSchemaError(f"the contract lacks {key!r}")
    pol = contract["policy"]
    for key in ("execution_dtype", "accumulation_dtype", "reference_dtype", "tf32", "backend_profiles", "backend_private_tolerance_relaxation"):
        if key not in pol:
            raise ContractSchemaError(f"policy lacks {key!r}")
    if pol["backend_private_tolerance_relaxation"] is not False:
        raise ContractSchemaError("a backend may not relax tolerances privately")
    if pol["tf32"].get("reference") != "disabled" or pol["tf32"].get("candidate_execution") != "disabled":
        raise ContractSchemaError("TF32 is disabled on both sides of every comparison")
    roles = contract["comparison_roles"]
    if set(roles["by_report_kind"]) != set(REPORT_KINDS):
        raise ContractSchemaError(f"comparison roles must cover exactly {REPORT_KINDS}")
    for kind, r in roles["by_report_kind"].items():
        for side in ("comparison_lhs_role", "comparison_rhs_role"):
            if r[side] in roles["forbidden"] or r[side] not in roles["allowed"]:
                raise ContractSchemaError(f"{kind}: role {r[side]!r} is not an allowed comparison role")
    if set(contract["judgments"]) != set(JUDGMENTS):
        raise ContractSchemaError(f"judgments must be exactly {JUDGMENTS}")
    for name, j in contract["judgments"].items():
        want = "bitwise" if name in INVARIANCE_JUDGMENTS else "tolerance"
        if j["default_mode"] != want:
            raise ContractSchemaError(f"{name} is judged by {want}")
        for oc, cells in j["by_op_class"].items():
            if oc not in OP_CLASSES:
                raise ContractSchemaError(f"{name}: unknown op class {oc!r}")
            for dt in MANDATORY_DTYPES:
                c = cells.get(dt)
                if c is None or c["status"] != "applicable" or c["mode"] != want:
                    raise ContractSchemaError(f"{name}/{oc}/{dt}: a mandatory dtype needs an applicable {want} cell")
                if want == "bitwise" and (c["atol"] != 0.0 or c["rtol"] != 0.0):
                    raise ContractSchemaError(f"{name}/{oc}/{dt}: invariance has no tolerance")
    agg = contract["chain_logprob_aggregates"]
    if set(agg["metrics"]) != set(CHAIN_AGGREGATE_METRICS) or agg.get("require_all") is not True:
        raise ContractSchemaError(f"the chain is judged by all of {CHAIN_AGGREGATE_METRICS}")
    if contract["batch_invariance"] != {"atol": 0.0, "rtol": 0.0}:
        raise ContractSchemaError("batch invariance is exact")


def resolve_dtype_policy(contract: _Mapping[str, _Any] | None = None) -> DtypePolicy:
    p = (contract or load_contract())["policy"]
    return DtypePolicy(p["execution_dtype"], p["accumulation_dtype"], p["reference_dtype"], p["output_dtype"]["default"],
                       p["output_dtype"]["logprob_aggregates"], p["fp8"], p["fp16"]["status"], p["tf32"]["reference"],
                       p["tf32"]["candidate_execution"], tuple(p["backend_profiles"]), bool(p["backend_private_tolerance_relaxation"]))


def validate_backend_provenance(prov: BackendProvenance, contract: _Mapping[str, _Any] | None = None, *, allow_fallback: bool = False) -> None:
    """A report counts only if it ran the profile it names, in the policy's dtypes, with TF32 off, on the backend it asked for."""
    c = contract or load_contract()
    pol = resolve_dtype_policy(c)
    if prov.backend_profile not in pol.backend_profiles:
        raise ContractResolveError(f"unknown backend profile {prov.backend_profile!r}; known: {list(pol.backend_profiles)}")
    want_exec = c["policy"]["backend_profile_contracts"][prov.backend_profile].get("execution_dtype", pol.execution_dtype)
    if normalize_dtype_name(prov.execution_dtype) != want_exec:
        raise ContractResolveError(f"profile {prov.backend_profile} executes in {want_exec}, the report says {prov.execution_dtype}")
    if normalize_dtype_name(prov.accumulation_dtype) != pol.accumulation_dtype:
        raise ContractResolveError(f"accumulation must be {pol.accumulation_dtype}, the report says {prov.accumulation_dtype}")
    if normalize_dtype_name(prov.reference_dtype) != pol.reference_dtype:
        raise ContractResolveError(f"the reference is {pol.reference_dtype}, the report says {prov.reference_dtype}")
    if prov.candidate_tf32_enabled or prov.reference_tf32_enabled:
        raise ContractResolveError("TF32 was enabled during the run")
    if prov.actual_backend != prov.requested_backend and not allow_fallback:
        raise ContractResolveError(f"requested backend {prov.requested_backend!r} but {prov.actual_backend!r} ran")


def resolve_comparison_roles(report_kind: str, contract: _Mapping[str, _Any] | None = None) -> ComparisonRoles:
    roles = (contract or load_contract())["comparison_roles"]["by_report_kind"]
    if report_kind not in roles:
        raise ContractResolveError(f"unknown report kind {report_kind!r}; known: {sorted(roles)}")
    return ComparisonRoles(report_kind, roles[report_kind]["comparison_lhs_role"], roles[report_kind]["comparison_rhs_role"])


def assert_comparison_roles(report_kind: str, lhs_role: str, rhs_role: str, contract: _Mapping[str, _Any] | None = None) -> None:
    want = resolve_comparison_roles(report_kind, contract)
    if (lhs_role, rhs_role) != (want.comparison_lhs_role, want.comparison_rhs_role):
        raise ContractResolveError(f"{report_kind} compares {want.comparison_lhs_role} with {want.comparison_rhs_role}, not {lhs_role} with {rhs_role}")


def resolve_tolerance_support(judgment: str, op_class: str, dtype, contract: _Mapping[str, _Any] | None = None) -> ToleranceSupport:
    c = contract or load_contract()
    if judgment not in JUDGMENTS:
        raise ContractResolveError(f"unknown judgment {judgment!r}")
    if op_class not in OP_CLASSES:
        raise ContractResolveError(f"unknown op class {op_class!r}")
    dt = normalize_dtype_name(dtype)
    cell = c["judgments"][judgment]["by_op_class"].get(op_class, {}).get(dt)
    if cell is None:
        return ToleranceSupport(judgment, op_class, dt, "out_of_scope", "the contract has no cell for this dtype")
    return ToleranceSupport(judgment, op_class, dt, cell["status"], None if cell["status"] == "applicable" else f"dtype is {cell['status']}")


def resolve_judgment_tolerance(judgment: str, op_class: str, dtype, *, backend_profile: str | None = None, arch_key: str | None = None,
                               contract: _Mapping[str, _Any] | None = None) -> JudgmentTolerance:
    """The cell of (judgment, op class, dtype), with an architecture override applied when the contract has one."""
    c = contract or load_contract()
    sup = resolve_tolerance_support(judgment, op_class, dtype, c)
    if sup.status == "out_of_scope":
        raise ContractResolveError(f"{judgment}/{op_class}/{sup.dtype_name} is out of scope: {sup.reason}")
    j = c["judgments"][judgment]
    cell = dict(j["by_op_class"][op_class][sup.dtype_name])
    if arch_key:
        cell.update(j.get("arch_overrides", {}).get(arch_key, {}).get(op_class, {}).get(sup.dtype_name, {}))
    roles = resolve_comparison_roles(judgment, c)
    return JudgmentTolerance(judgment, op_class, sup.dtype_name, cell["status"], cell["mode"], float(cell["atol"]), float(cell["rtol"]),
                             roles.comparison_lhs_role, roles.comparison_rhs_role, backend_profile, arch_key)


def resolve_chain_aggregate_thresholds(execution_dtype, contract: _Mapping[str, _Any] | None = None) -> dict:
    m = (contract or load_contract())["chain_logprob_aggregates"]["metrics"]
    dt = normalize_dtype_name(execution_dtype)
    try:
        return {k: float(m[k]["by_execution_dtype"][dt]["threshold"]) for k in CHAIN_AGGREGATE_METRICS}
    except KeyError:
        raise ContractResolveError(f"no chain thresholds for execution dtype {dt}") from None


def default_clip_interval(contract: _Mapping[str, _Any] | None = None) -> tuple:
    lo, hi = (contract or load_contract())["chain_logprob_aggregates"]["default_clip_interval"]
    return float(lo), float(hi)


def compute_logprob_aggregates(lhs_logp: torch.Tensor, rhs_logp: torch.Tensor, active_mask: torch.Tensor | None = None, *,
                               report_kind: str = "train_infer_logprob_parity", clip_interval: tuple | None = None,
                               contract: _Mapping[str, _Any] | None = None) -> LogprobAggregates:
    """The three chain-level aggregates over the active selected tokens, in fp32, dlogp = lhs - rhs.  NaN / Inf on an
    active token and an empty active set are hard failures, not zeros."""
    if lhs_logp.shape != rhs_logp.shape:
        raise ContractResolveError("the two log-prob tensors must have one shape")
    roles = resolve_comparison_roles(report_kind, contract)
    lo, hi = clip_interval or default_clip_interval(contract)
    mask = torch.ones_like(lhs_logp, dtype=torch.bool) if active_mask is None else active_mask.bool().to(lhs_logp.device)
    a, b = lhs_logp.float()[mask], rhs_logp.float().to(lhs_logp.device)[mask]
    if a.numel() == 0:
        raise ContractResolveError("empty active token set")
    if not (bool(torch.isfinite(a).all()) and bool(torch.isfinite(b).all())):
        raise ContractResolveError("NaN or Inf log-prob on an active token")
    d = a - b
    ratio = torch.exp(d)
    return LogprobAggregates(float(d.abs().max()), float((ratio - 1 - d).mean()), float(((ratio < lo) | (ratio > hi)).float().mean()),
                             int(a.numel()), (lo, hi), report_kind, roles.comparison_lhs_role, roles.comparison_rhs_role)


def judge_logprob_aggregates(aggregates: LogprobAggregates, execution_dtype, contract: _Mapping[str, _Any] | None = None) -> LogprobAggregateVerdict:
    th = resolve_chain_aggregate_thresholds(execution_dtype, contract)
    metrics = tuple(AggregateMetricVerdict(k, getattr(aggregates, k), th[k], _math.isfinite(getattr(aggregates, k)) and getattr(aggregates, k) <= th[k])
                    for k in CHAIN_AGGREGATE_METRICS)
    return LogprobAggregateVerdict(aggregates, metrics, all(m.passed for m in metrics), aggregates.report_kind, aggregates.comparison_lhs_role,
                                   aggregates.comparison_rhs_role)


def resolve_logprob_threshold(dtype) -> float:
    """Absolute |dlogp| bound of a selected log-prob computed in ``dtype`` against the fp32 reference."""
    return resolve_judgment_tolerance("forward_accuracy", "logprob", dtype).atol


validate_contract_schema(load_contract())
