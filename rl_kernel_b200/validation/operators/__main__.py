"""Operator checks from the command line (parity: tools/validation/operators/{check_operator, check_forward_invariance,
check_gradient_invariance, check_decode_prefill, check_stateful_kv, sweep_ws1_four_judgments}.py of the reference).

    python -m rl_kernel_b200.validation.operators list
    python -m rl_kernel_b200.validation.operators operator rms_norm --device cuda
    python -m rl_kernel_b200.validation.operators forward-invariance attention --device cuda
    python -m rl_kernel_b200.validation.operators gradient-invariance linear_logp
    python -m rl_kernel_b200.validation.operators decode-prefill --device cuda
    python -m rl_kernel_b200.validation.operators stateful-kv
    python -m rl_kernel_b200.validation.operators sweep --device cuda --output evidence.json

Every command prints one JSON document and exits 0 only if the check is green.  ``--device cuda`` judges the sm_100a
candidates in bf16 and refuses to run without a GPU; the default judges the PyTorch references on the CPU in fp32."""
from __future__ import annotations

import argparse
import json
import sys

import torch


def _dev(a):
    from rl_kernel_b200.validation.operators import accelerator as acc

    dev = acc.resolve_device(a.device, required=True)
    acc.disable_tf32(dev.type)
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    return dev, dtype, acc.describe(dev).to_dict()


def cmd_grid(args) -> int:
    import json as _json

    import torch as _torch

    from rl_kernel_b200.validation.operators import four_judgment_matrix as fj

    profiles = (args.profile,) if args.profile else None
    executed = None
    if args.execute:
        prof = args.profile or ("b200_bf16" if args.device.startswith("cuda") else "reference_fp32")
        profiles = (prof,)
        cuda = args.device.startswith("cuda")
        executed = fj.executed_results(prof, device=args.device, dtype=_torch.bfloat16 if cuda else _torch.float32,
                                       candidate="b200" if cuda else "pytorch")
    rep = fj.build_classified_matrix(profiles=profiles, executed=executed)
    if args.json:
        print(_json.dumps(rep.to_dict(), indent=1))
    else:
        for c in rep.cells:
            if c.judgment == "forward_accuracy":
                row = [x for x in rep.cells if (x.profile, x.op_name, x.tier) == (c.profile, c.op_name, c.tier)]
                print(f"{c.profile:<15} {c.op_name:<12} {c.tier:<8} " + " ".join(f"{x.status:<18}" for x in row) + f" {c.case_id or '-'}")
        print(rep.counts)
    bad = [c for c in rep.cells if c.status == "red"]
    return 2 if bad or (args.execute and not rep.green) else 0


def cmd_adapters(args) -> int:
    import json as _json

    from rl_kernel_b200.validation.operators.gradient_adapters import gradient_adapter_status_matrix

    rows = gradient_adapter_status_matrix()
    if args.json:
        print(_json.dumps([r.to_dict() for r in rows], indent=1))
    else:
        for r in rows:
            flag = "RED " if (r.untracked_red or r.tracked_red) else "    "
            print(f"{flag}{r.backend_profile:<15} {r.chain_node:<26} {r.op_name:<24} {r.candidate_status:<22} {r.candidate_path or '-'}")
    return 2 if any(r.untracked_red or r.tracked_red for r in rows) else 0


def cmd_list(a) -> int:
    from rl_kernel_b200.validation.operators.operator_specs import OP_SPECS

    print(json.dumps({n: {"class": s.op_class, "adapter": s.adapter, "grad_inputs": list(s.grad_input_names), "candidates": s.candidate_paths}
                      for n, s in OP_SPECS.items()}, indent=1))
    return 0


def cmd_operator(a) -> int:
    from rl_kernel_b200.validation.operators.four_judgment_matrix import judge_operator

    dev, dtype, info = _dev(a)
    res = judge_operator(a.op, str(dev), dtype, seed=a.seed)
    print(json.dumps({"op": a.op, "accelerator": info, "judgments": {k: {"status": s, "detail": d} for k, (s, d) in res.items()}}, indent=1))
    return 0 if all(s == "pass" for s, _ in res.values()) else 1


def _invariance(a, gradients: bool) -> int:
    from rl_kernel_b200.validation.operators.forward_invariance import run_forward_invariance
    from rl_kernel_b200.validation.operators.gradient_invariance import run_gradient_invariance

    dev, dtype, info = _dev(a)
    rep = (run_gradient_invariance if gradients else run_forward_invariance)(a.op, device=str(dev), dtype=dtype, seed=a.seed)
    cells = {k: {"tokens": c.tokens, "mismatched": c.mismatched, "max_abs": c.max_abs} for k, c in rep.configs.items()}
    out = {"op": a.op, "candidate": rep.candidate, "accelerator": info, "forward": cells, "accuracy_ok": rep.accuracy_ok, "accuracy_err": rep.accuracy_err}
    ok = rep.forward_invariant and rep.accuracy_ok
    if gradients:
        out["gradients"] = {k: {n: {"tokens": c.tokens, "mismatched": c.mismatched, "max_abs": c.max_abs} for n, c in per.items()}
                            for k, per in rep.grad_configs.items()}
        out["parameter_gradient_relative_difference"] = rep.param_grad_rel
        out["gradient_accuracy_err"] = rep.grad_accuracy_err
        ok = ok and rep.gradient_invariant and rep.grad_accuracy_ok
    print(json.dumps(out, indent=1))
    return 0 if ok else 1


def cmd_decode_prefill(a) -> int:
    from rl_kernel_b200.validation.operators.kv_consistency import assert_decode_prefill_consistent

    dev, _, info = _dev(a)
    try:
        rep = assert_decode_prefill_consistent(device=str(dev))
    except AssertionError as exc:
        print(json.dumps({"check": "decode_prefill", "accelerator": info, "passed": False, "reason": str(exc)}))
        return 1
    print(json.dumps({"check": "decode_prefill", "accelerator": info, "candidate": rep.candidate, "cells": len(rep.cells), "bitwise": rep.bitwise,
                      "max_abs_dlogp": rep.max_abs_dlogp, "passed": True}))
    return 0


def cmd_stateful_kv(a) -> int:
    from rl_kernel_b200.validation.operators.kv_consistency import assert_stateful_kv_consistent

    dev, _, info = _dev(a)
    try:
        rep = assert_stateful_kv_consistent(device=str(dev))
    except AssertionError as exc:
        print(json.dumps({"check": "stateful_kv", "accelerator": info, "passed": False, "reason": str(exc)}))
        return 1
    print(json.dumps({"check": "stateful_kv", "accelerator": info, "candidate": rep.candidate, "generated_positions": rep.generated_positions,
                      "mismatched_positions": rep.mismatched_positions, "cache_identity": rep.cache_identity, "passed": True}))
    return 0


def cmd_sweep(a) -> int:
    from rl_kernel_b200.validation.operators.elementwise_inventory import unexecuted_cells, unresolved_needs_fix
    from rl_kernel_b200.validation.operators.four_judgment_matrix import four_judgment_matrix

    dev, dtype, info = _dev(a)
    m = four_judgment_matrix(device=str(dev), dtype=dtype)
    doc = {"accelerator": info, "dtype": str(dtype).removeprefix("torch."), "green": m.green,
           "cells": {f"{r}/{c}": {"status": cell.status, "detail": cell.detail} for (r, c), cell in m.cells.items()},
           "inventory": {"unexecuted": [i.name for i in unexecuted_cells()], "needs_fix": [i.name for i in unresolved_needs_fix()]}}
    text = json.dumps(doc, indent=1)
    if a.output:
        open(a.output, "w").write(text + "\n")
    print(m.render() if not a.json else text)
    return 0 if m.green else 1


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m rl_kernel_b200.validation.operators", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)

    def common(p, op=False):
        if op:
            p.add_argument("op")
        p.add_argument("--device", default="cpu")
        p.add_argument("--seed", type=int, default=0)

    sub.add_parser("list").set_defaults(fn=cmd_list)
    p = sub.add_parser("grid", help="coverage grid of the four judgments; --execute runs them on this host for one profile")
    p.add_argument("--profile", default=None)
    p.add_argument("--execute", action="store_true")
    p.add_argument("--device", default="cpu")
    p.add_argument("--json", action="store_true")
    p.set_defaults(fn=cmd_grid)
    p = sub.add_parser("adapters", help="status matrix: backend profile x chain node -> adapter, candidate, coverage")
    p.add_argument("--json", action="store_true")
    p.set_defaults(fn=cmd_adapters)
    p = sub.add_parser("operator"); common(p, True); p.set_defaults(fn=cmd_operator)
    p = sub.add_parser("forward-invariance"); common(p, True); p.set_defaults(fn=lambda a: _invariance(a, False))
    p = sub.add_parser("gradient-invariance"); common(p, True); p.set_defaults(fn=lambda a: _invariance(a, True))
    p = sub.add_parser("decode-prefill"); common(p); p.set_defaults(fn=cmd_decode_prefill)
    p = sub.add_parser("stateful-kv"); common(p); p.set_defaults(fn=cmd_stateful_kv)
    p = sub.add_parser("sweep"); common(p); p.add_argument("--output", default=None); p.add_argument("--json", action="store_true")
    p.set_defaults(fn=cmd_sweep)
    a = ap.parse_args(argv)
    return int(a.fn(a))


if __name__ == "__main__":
    sys.exit(main())
