"""Forward invariance of an operator across batch configurations (parity: rl_engine/validation/
operators/forward_invariance.py:195-294).

A ``ConfigSpec`` names one physical presentation of the SAME logical batch: packed in canonical
order (the baseline), samples permuted, every sample alone, chunked, padded on the left or right.
``run_forward_invariance`` runs a candidate under every configuration through the operator's
layout adapter and compares the outputs per logical token ``(sample_id, position)`` with the
baseline, bit for bit; it also reports the error of the baseline against the fp32 gold.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from rl_kernel_b200.config.workload import (LogicalBatch, apply_chunking, apply_packing, apply_padding,
                                            batch_permutation_from_manifest, build_logical_batch, load_manifest, permute_batch)
from rl_kernel_b200.contracts.numerical import resolve_tolerance
from rl_kernel_b200.validation.operators.operator_specs import OP_SPECS, make_candidate, make_operator_case


@dataclass(frozen=True)
class ConfigSpec:
    config_id: str
    layout_kind: str                      # packed | permuted | singleton | chunked | padded_left | padded_right
    chunk_size: int | None = None
    permutation: tuple[int, ...] | None = None
    is_baseline: bool = False


def build_config_matrix(manifest=None, *, include: tuple[str, ...] | None = None) -> tuple[ConfigSpec, ...]:
    """The configurations of the primary matrix; chunk size and permutation come from the workload manifest."""
    m = manifest or load_manifest()
    chunk = int(m.primary_matrix["chunking"]["chunk_size"]) if "chunking" in m.primary_matrix else 7
    perm = batch_permutation_from_manifest(m)
    cfgs = (ConfigSpec("BN/full", "packed", is_baseline=True), ConfigSpec("BN/permuted", "permuted", permutation=perm),
            ConfigSpec("B1/singletons", "singleton"), ConfigSpec("BN/chunked", "chunked", chunk_size=chunk),
            ConfigSpec("BN/padded_left", "padded_left"), ConfigSpec("BN/padded_right", "padded_right"))
    return tuple(c for c in cfgs if include is None or c.config_id in include)


def layouts_for(config: ConfigSpec, batch: LogicalBatch, manifest=None) -> list:
    """Physical layouts whose union covers every logical token of ``batch`` exactly once."""
    if config.layout_kind == "packed":
        return [apply_packing(batch)]
    if config.layout_kind == "permuted":
        return [apply_packing(permute_batch(batch, config.permutation))]
    if config.layout_kind == "singleton":
        return [apply_packing(LogicalBatch(batch.workload_id, batch.seed, (s,))) for s in batch.samples]
    if config.layout_kind == "chunked":
        return [apply_chunking(batch, chunk_size=config.chunk_size)]
    if config.layout_kind in ("padded_left", "padded_right"):
        return [apply_padding(batch, pad_side=config.layout_kind.split("_")[1], manifest=manifest)]
    raise ValueError(f"unknown layout kind {config.layout_kind!r}")


@dataclass
class TokenComparison:
    tokens: int = 0
    mismatched: int = 0
    max_abs: float = 0.0
    first: tuple | None = None

    @property
    def ok(self) -> bool:
        return self.tokens > 0 and self.mismatched == 0


def compare_tokens(base: dict, other: dict) -> TokenComparison:
    """Bitwise comparison per logical token; a token missing on either side counts as a mismatch."""
    c = TokenComparison()
    for k in sorted(set(base) | set(other)):
        c.tokens += 1
        a, b = base.get(k), other.get(k)
        if a is None or b is None or a.shape != b.shape or a.dtype != b.dtype:
            c.mismatched += 1
            c.first = c.first or k
            continue
        if a.dtype.is_floating_point:
            av, bv = a.contiguous().view(torch.int16 if a.element_size() == 2 else torch.int32 if a.element_size() == 4 else torch.int64), None
            bv = b.contiguous().view(av.dtype)
            same = bool(torch.equal(av, bv))
        else:
            same = bool(torch.equal(a, b))
        if not same:
            c.mismatched += 1
            c.first = c.first or k
            c.max_abs = max(c.max_abs, float((a.double() - b.double()).abs().max()))
    return c


def accuracy(out: dict, gold: dict, op_name: str, dtype: torch.dtype, tol_key: str | None = None) -> tuple[bool, float]:
    """Candidate vs fp32 gold inside the precision profile's tolerance for the candidate's output dtype."""
    if not gold:
        return True, 0.0
    keys = sorted(gold)
    c = torch.stack([out[k].float().reshape(-1) for k in keys])
    g = torch.stack([gold[k].float().reshape(-1) for k in keys])
    first = out[keys[0]]
    key = str(first.dtype if first.dtype.is_floating_point else dtype).removeprefix("torch.")
    try:
        tol = resolve_tolerance(tol_key or op_name, key)
    except KeyError:
        tol = resolve_tolerance("default", key)
    ok, err = tol.check(c, g)
    return bool(ok), float(err)


@dataclass
class InvarianceReport:
    op_name: str
    candidate: str
    device: str
    dtype: str
    accuracy_ok: bool = True
    accuracy_err: float = 0.0
    configs: dict[str, TokenComparison] = field(default_factory=dict)
    grad_accuracy_ok: bool = True
    grad_accuracy_err: float = 0.0
    grad_configs: dict[str, dict[str, TokenComparison]] = field(default_factory=dict)
    param_grad_rel: dict[str, float] = field(default_factory=dict)

    @property
    def forward_invariant(self) -> bool:
        return all(c.ok for c in self.configs.values())

    @property
    def gradient_invariant(self) -> bool:
        return all(c.ok for per in self.grad_configs.values() for c in per.values())

    def failing(self) -> list[str]:
        bad = [k for k, c in self.configs.items() if not c.ok]
        bad += [f"{k}:d{n}" for k, per in self.grad_configs.items() for n, c in per.items() if not c.ok]
        return bad


def _run_config(spec, adapter, cand, st, config, batch, manifest, want_grads: bool):
    out, grads = {}, {}
    for layout in layouts_for(config, batch, manifest):
        g = {} if want_grads else None
        out.update(adapter.run(spec, cand.op, st, layout, g))
        if g:
            for name, val in g.items():
                if isinstance(val, dict):
                    grads.setdefault(name, {}).update(val)
                else:                                           # a parameter gradient: layouts (singletons) add up
                    grads[name] = val.float() if name not in grads else grads[name] + val.float()
    return out, grads


def run_forward_invariance(op_name: str, *, candidate: str = "auto", device: str = "cpu", dtype: torch.dtype | None = None,
                           seed: int = 0, manifest=None, batch: LogicalBatch | None = None, gradients: bool = False,
                           configs: tuple[ConfigSpec, ...] | None = None) -> InvarianceReport:
    """Forward (and with ``gradients`` the backward) of ``op_name`` under every configuration."""
    m = manifest or load_manifest()
    batch = batch or build_logical_batch(m)
    cand = make_candidate(op_name=op_name, candidate=candidate, device=device, dtype=dtype)
    spec, adapter, st = make_operator_case(op_name, batch=batch, device=cand.device, dtype=cand.dtype, seed=seed)
    rep = InvarianceReport(op_name, cand.candidate, cand.device, str(cand.dtype).removeprefix("torch."))
    want = gradients and bool(spec.grad_input_names)
    cfgs = configs or build_config_matrix(m)
    base_cfg = next(c for c in cfgs if c.is_baseline)
    with torch.enable_grad() if want else torch.no_grad():
        base, base_g = _run_config(spec, adapter, cand, st, base_cfg, batch, m, want)
        rep.accuracy_ok, rep.accuracy_err = accuracy(base, adapter.gold(spec, st, batch), op_name, cand.dtype, spec.tolerance_key)
        for cfg in cfgs:
            out, g = _run_config(spec, adapter, cand, st, cfg, batch, m, want)
            rep.configs[cfg.config_id] = compare_tokens(base, out)
            if want:
                per = {}
                for name, val in base_g.items():
                    if isinstance(val, dict):
                        per[name] = compare_tokens(val, g.get(name, {}))
                    else:
                        # a parameter's gradient sums over tokens in physical order: its bits follow the order, so
                        # it is held to a relative bound here and to bit equality only where the order is the same
                        rel = float((val - g[name]).abs().max() / val.abs().max().clamp_min(1e-30))
                        rep.param_grad_rel[f"{cfg.config_id}:{name}"] = rel
                        if cfg.is_baseline:
                            per[name] = TokenComparison(tokens=1, mismatched=int(rel != 0.0), max_abs=rel)
                rep.grad_configs[cfg.config_id] = per
    return rep


__all__ = ["ConfigSpec", "InvarianceReport", "OP_SPECS", "TokenComparison", "accuracy", "build_config_matrix", "compare_tokens",
           "layouts_for", "run_forward_invariance"]
