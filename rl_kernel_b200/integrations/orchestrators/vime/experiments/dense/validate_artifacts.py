"""Checks on the artifacts a strict run leaves behind (parity: validate_artifacts.py of the reference's dense experiment):

* the framework read-backs (one JSON per process, written by ``FrameworkOperatorIntegration``): both engines present,
  every module hooked and actually called, no fallback, only this package's backends, the strict log-prob entry point;
* the training dumps (``*.pt`` mappings with ``log_probs`` and ``rollout_log_probs`` per sample, optionally
  ``loss_masks``): the two log-probs of every active token compared bit for bit.

``python -m ...validate_artifacts READBACK_DIR TRAIN_DUMP_DIR`` prints the report and exits non-zero when a check fails."""
from __future__ import annotations

import argparse
import json
import sys
from collections.abc import Mapping
from pathlib import Path
from typing import Any

import torch

FRAMEWORKS = (("vllm", "rollout"), ("megatron", "training"))
MODULES = ("attention", "ffn", "logp")
BACKEND_PREFIXES = ("rl_kernel_b200.", "b200", "rlkernel.")
STRICT_LOGP_BACKEND = "rl_kernel_b200.linear_logp.bitwise.v1"
FOREIGN_MARKERS = ("triton", "torch.compile", "inductor")


def load_readbacks(directory: str | Path) -> list[dict[str, Any]]:
    out = []
    for p in sorted(Path(directory).glob("*.json")):
        v = json.loads(p.read_text())
        if not isinstance(v, dict):
            raise ValueError(f"readback must contain an object: {p}")
        v["_path"] = str(p)
        out.append(v)
    if not out:
        raise ValueError(f"no framework readbacks found in {directory}")
    return out


def _mentions_foreign_compiler(record: Any) -> bool:
    text = json.dumps(record, default=str).lower()
    return any(m in text for m in FOREIGN_MARKERS)


def validate_readbacks(readbacks: list[dict[str, Any]], *, frameworks=FRAMEWORKS, modules=MODULES) -> dict[str, Any]:
    errors: list[str] = []
    summary: dict[str, Any] = {}
    for framework, target in frameworks:
        label = f"{framework}/{target}"
        mine = [r for r in readbacks if r.get("framework") == framework and r.get("target") == target]
        if not mine:
            errors.append(f"missing {label} readback")
            continue
        errors += [f"{label} recorded fallback: {r['fallbacks']}" for r in mine if r.get("fallbacks")]
        per_module = {}
        for m in modules:
            hooks = sum(m in (r.get("installed_hooks") or {}) for r in mine)
            records = [r["operators"][m] for r in mine if isinstance(r.get("operators"), Mapping) and m in r["operators"]]
            calls = sum(int(rec.get("call_count", 0)) for rec in records)
            if hooks == 0:
                errors.append(f"{label} {m} hook was not installed")
            if calls == 0:
                errors.append(f"{label} {m} had zero calls")
            for rec in records:
                backend = str(rec.get("backend_id", ""))
                if m == "logp" and backend != STRICT_LOGP_BACKEND:
                    errors.append(f"{label} logp used {backend!r}, expected {STRICT_LOGP_BACKEND!r}")
                elif m != "logp" and not backend.startswith(BACKEND_PREFIXES):
                    errors.append(f"{label} {m} used unexpected backend {backend!r}")
                if _mentions_foreign_compiler(rec):
                    errors.append(f"{label} {m} went through a tracing compiler")
                platform = (rec.get("provenance") or {}).get("runtime_platform")
                if platform not in (None, "cuda"):
                    errors.append(f"{label} {m} did not report CUDA execution (got {platform!r})")
            per_module[m] = {"installed_processes": hooks, "call_count": calls, "backend_ids": sorted({str(r.get("backend_id", "")) for r in records})}
        summary[label] = {"readback_count": len(mine), "modules": per_module}
    return {"passed": not errors, "errors": errors, "frameworks": summary}


def _as_list(v: Any) -> list[torch.Tensor]:
    if isinstance(v, torch.Tensor):
        return [v]
    return [torch.as_tensor(x) for x in v]


def compare_train_rollout_logps(paths: list[str | Path]) -> dict[str, Any]:
    """Bit comparison of ``log_probs`` (training) against ``rollout_log_probs`` over every dump; inactive positions
    (``loss_masks`` zero) are left out."""
    samples = elements = mismatching = 0
    max_abs = 0.0
    worst: dict[str, Any] | None = None
    errors: list[str] = []
    for p in paths:
        d = torch.load(p, map_location="cpu", weights_only=False)
        if not isinstance(d, Mapping):
            raise ValueError(f"train dump must contain a mapping: {p}")
        if "log_probs" not in d or "rollout_log_probs" not in d:
            errors.append(f"{p}: needs log_probs and rollout_log_probs")
            continue
        train, roll = _as_list(d["log_probs"]), _as_list(d["rollout_log_probs"])
        masks = _as_list(d["loss_masks"]) if d.get("loss_masks") is not None else [None] * len(train)
        if not (len(train) == len(roll) == len(masks)):
            errors.append(f"{p}: {len(train)} training, {len(roll)} rollout samples and {len(masks)} masks")
            continue
        for i, (a, b, m) in enumerate(zip(train, roll, masks)):
            a, b = a.reshape(-1).float(), b.reshape(-1).float()
            if a.shape != b.shape:
                errors.append(f"{p} sample {i}: training has {a.numel()} tokens, rollout {b.numel()}")
                continue
            keep = torch.ones_like(a, dtype=torch.bool) if m is None else m.reshape(-1).bool()
            a, b = a[keep], b[keep]
            diff = a.view(torch.int32) != b.view(torch.int32)
            samples += 1
            elements += a.numel()
            mismatching += int(diff.sum())
            if a.numel():
                gap = float((a - b).abs().max())
                if gap > max_abs:
                    j = int((a - b).abs().argmax())
                    max_abs, worst = gap, {"file": str(p), "sample": i, "token": j, "training": float(a[j]), "rollout": float(b[j])}
    return {"passed": not errors and mismatching == 0 and samples > 0, "errors": errors, "samples": samples, "tokens": elements,
            "mismatching_tokens": mismatching, "max_abs_difference": max_abs, "worst": worst}


def validate_artifacts(readback_dir: str | Path, train_data_dir: str | Path) -> dict[str, Any]:
    rb = validate_readbacks(load_readbacks(readback_dir))
    dumps = sorted(Path(train_data_dir).glob("*.pt"))
    lp = compare_train_rollout_logps(dumps) if dumps else {"passed": False, "errors": [f"no training dumps in {train_data_dir}"]}
    return {"passed": rb["passed"] and lp["passed"], "readbacks": rb, "train_rollout_logps": lp}


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("readback_dir")
    ap.add_argument("train_data_dir")
    a = ap.parse_args(argv)
    rep = validate_artifacts(a.readback_dir, a.train_data_dir)
    print(json.dumps(rep, indent=1))
    return 0 if rep["passed"] else 2


if __name__ == "__main__":
    sys.exit(main())
