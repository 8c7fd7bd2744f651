"""Performance analysis, SVG plots and artifact validation of the dense experiment tools on synthetic run directories."""
import json
import math

import torch

from rl_kernel_b200.integrations.orchestrators.vime.experiments.dense import analyze_performance as ap
from rl_kernel_b200.integrations.orchestrators.vime.experiments.dense import plot_results as pr
from rl_kernel_b200.integrations.orchestrators.vime.experiments.dense import validate_artifacts as va


def _run(tmp_path, name, base, n=30, tokens=65536):
    d = tmp_path / name
    d.mkdir()
    with open(d / "rounds.jsonl", "w") as f:
        for i in range(n):
            sec = base * (2.0 if i == 0 else 1.0) + 0.01 * math.sin(i)
            f.write(json.dumps({"step": i, "step_seconds": sec, "tokens_compared": tokens, "mismatch_count": 0, "reward_mean": 0.5, "kl": 0.01 * i,
                                "grad_norm": 4.8, "loss": 1e-5, "max_abs_dlogp": 0.0,
                                "phase_ms": {"rollout": sec * 480, "ref_score": sec * 100, "train_fwd_bwd": sec * 400, "optimizer": 4.0}}) + "\n")
    return d


def test_statistics_helpers():
    d = ap.describe([1, 2, 3, 4, float("nan"), None])
    assert d["count"] == 4 and d["median"] == 2.5 and d["min"] == 1 and d["max"] == 4 and abs(d["p95"] - 3.85) < 1e-9
    assert ap.describe([]) == {"count": 0}
    assert ap.moving_average([1, 2, 3, 4], 2) == [1, 1.5, 2.5, 3.5]
    r = ap.regression([1, 2, 3, 4], [3, 5, 7, 9], at=10)
    assert abs(r["slope"] - 2) < 1e-12 and abs(r["intercept"] - 1) < 1e-12 and abs(r["r2"] - 1) < 1e-12 and abs(r["value"] - 21) < 1e-9
    assert ap.regression([1], [1]) == {"n": 1} and ap.regression([2, 2], [1, 3])["slope"] == 0.0
    b1 = ap.bootstrap_mean_difference([10.0, 10.2, 9.9, 10.1] * 5, [12.0, 12.1, 11.9] * 5)
    assert b1 == ap.bootstrap_mean_difference([10.0, 10.2, 9.9, 10.1] * 5, [12.0, 12.1, 11.9] * 5)          # seeded
    assert b1["ci_low"] <= b1["difference"] <= b1["ci_high"] < 0


def test_analyze_two_groups_writes_summary_rows_and_plots(tmp_path, capsys):
    a, b = _run(tmp_path, "strict", 13.0), _run(tmp_path, "library", 11.0)
    out = tmp_path / "perf"
    assert ap.main([f"strict={a}", str(b), "--out", str(out), "--tokens-per-step", "98304"]) == 0
    printed = json.loads(capsys.readouterr().out)
    assert set(printed) == {"strict", "library"} and abs(printed["strict"]["median_step_seconds"] - 13.0) < 0.02
    s = json.loads((out / "performance.json").read_text())
    g = s["groups"]["strict"]
    assert g["steps"] == 29 and abs(g["tokens_per_second"]["median"] - 98304 / 13.0) < 20             # the warm-up step is left out
    assert abs(g["phase_share"]["rollout"] - 0.48) < 0.01 and abs(sum(g["phase_share"].values()) - 1) < 1e-9
    (c,) = s["comparisons"]
    assert {c["a"], c["b"]} == {"library", "strict"} and abs(abs(c["mean_step_seconds_difference"]["difference"]) - 2.0) < 0.01
    rows = pr.load_rows(out / "performance_rows.csv")
    assert len(rows) == 60 and rows[0]["warmup"] is True and rows[1]["warmup"] is False
    for name in ("performance_step_seconds.svg", "performance_tokens_per_second.svg", "performance_phases.svg"):
        text = (out / name).read_text()
        assert text.startswith("<svg") and text.rstrip().endswith("</svg>") and "strict" in text
    figs = pr.write_figures([{**r, "seed": 1} for r in rows], tmp_path / "plots")
    assert {f.name for f in figs} == {"consistency_mismatch_count.svg", "performance_step_seconds.svg", "performance_tokens_per_second.svg"}
    assert pr.main([str(out / "performance_rows.csv"), "--out", str(tmp_path / "p2")]) == 0


def test_svg_charts_handle_degenerate_input():
    assert "<polyline" not in pr.line_chart({"a": [(0, 1.0)]}, title="one point") and "circle" in pr.line_chart({"a": [(0, 1.0)]}, title="t")
    assert pr.line_chart({}, title="empty").startswith("<svg")
    assert "polyline" in pr.line_chart({"m": [(0, 0), (1, 1000), (2, 0)]}, title="counts", symlog=True)
    svg = pr.bar_chart({"x": {"a": 1.0, "b": 2.0}, "y": {"a": 0.5, "b": None}}, title="bars <&>")
    assert svg.count("<rect") >= 5 and "&lt;&amp;&gt;" in svg


def _readback(framework, target, **over):
    ops = {m: {"backend_id": "rl_kernel_b200.linear_logp.bitwise.v1" if m == "logp" else f"rl_kernel_b200.{m}", "call_count": 12,
               "provenance": {"runtime_platform": "cuda"}} for m in va.MODULES}
    rb = {"framework": framework, "target": target, "installed_hooks": {m: True for m in va.MODULES}, "operators": ops, "fallbacks": []}
    rb.update(over)
    return rb


def test_artifact_validation(tmp_path):
    rbd, dumps = tmp_path / "rb", tmp_path / "dumps"
    rbd.mkdir()
    dumps.mkdir()
    (rbd / "vllm.json").write_text(json.dumps(_readback("vllm", "rollout")))
    (rbd / "megatron.json").write_text(json.dumps(_readback("megatron", "training")))
    lp = [torch.randn(7), torch.randn(5)]
    torch.save({"log_probs": lp, "rollout_log_probs": [t.clone() for t in lp], "loss_masks": [torch.ones(7), torch.tensor([1, 1, 1, 0, 0])]}, dumps / "a.pt")
    rep = va.validate_artifacts(rbd, dumps)
    assert rep["passed"] and rep["train_rollout_logps"]["tokens"] == 10 and rep["readbacks"]["frameworks"]["vllm/rollout"]["modules"]["ffn"]["call_count"] == 12
    assert va.main([str(rbd), str(dumps)]) == 0
    # one differing active token, one differing masked token
    other = [t.clone() for t in lp]
    other[0][2] += 1e-3
    other[1][4] += 1.0
    torch.save({"log_probs": lp, "rollout_log_probs": other, "loss_masks": [torch.ones(7), torch.tensor([1, 1, 1, 0, 0])]}, dumps / "b.pt")
    bad = va.compare_train_rollout_logps(sorted(dumps.glob("*.pt")))
    assert not bad["passed"] and bad["mismatching_tokens"] == 1 and bad["worst"]["sample"] == 0 and bad["worst"]["token"] == 2
    # read-back problems
    broken = _readback("megatron", "training", fallbacks=["ffn"])
    broken["operators"]["logp"]["backend_id"] = "something.else"
    broken["operators"]["attention"]["call_count"] = 0
    broken["operators"]["ffn"]["provenance"] = {"runtime_platform": "cuda", "note": "compiled with Triton"}
    del broken["installed_hooks"]["attention"]
    rep = va.validate_readbacks([_readback("vllm", "rollout"), broken])
    text = " | ".join(rep["errors"])
    for needle in ("recorded fallback", "logp used 'something.else'", "attention had zero calls", "attention hook was not installed",
                   "tracing compiler"):
        assert needle in text, (needle, text)
    assert "missing vllm/rollout readback" in va.validate_readbacks([_readback("megatron", "training")])["errors"]
    assert va.main([str(rbd), str(tmp_path / "rb")]) == 2                        # no dumps there


def test_integration_evidence_feeds_artifact_validation(tmp_path, monkeypatch):
    """Read-backs written by the framework adapter are what the artifact validation reads."""
    import pytest

    from rl_kernel_b200.integrations.common.runtime import FrameworkOperatorIntegration
    from rl_kernel_b200.runtime.plan import IntegrationPlan

    monkeypatch.setenv("RL_KERNEL_READBACK_DIR", str(tmp_path / "rb"))

    class Op:
        def __init__(self, backend_id, provenance=None):
            self.backend_id, self.provenance, self.calls = backend_id, provenance or {"runtime_platform": "cuda"}, 0

        def __call__(self, x):
            self.calls += 1
            return x + 1

    def native(x):
        return x - 1

    for framework, side in (("vllm", "rollout"), ("megatron", "training")):
        ops = {"attention": Op("rl_kernel_b200.attention"), "ffn": Op("rl_kernel_b200.ffn"), "logp": Op("rl_kernel_b200.linear_logp.bitwise.v1")}
        integ = FrameworkOperatorIntegration(framework, side, IntegrationPlan.uniform("R/R"), rl_kernel_operators=ops)
        with pytest.raises(RuntimeError, match="missing hooks"):
            integ.assert_strict_evidence()
        for m in ops:
            integ.record_installed_hook(m, f"{framework}.{m}.forward")
            assert integ.route(m, native, 1) == 2                                   # the plan selects the installed operator
        integ.record_profile_call("attention")
        integ.assert_strict_evidence()
        rb = integ.readback()
        assert rb["operators"]["logp"]["call_count"] == 1 and rb["profile_calls"] == {"attention": 1} and rb["target"] in ("rollout", "training")
        with pytest.raises(RuntimeError, match="did not use the installed"):
            integ.record_execution("ffn", native)
        with pytest.raises(ValueError):
            integ.record_execution("ffn", ops["ffn"], execution_mode="interpreted")
        integ.record_execution("ffn", ops["ffn"], execution_mode="compiled_cuda_graph")
        assert integ.readback()["operators"]["ffn"]["execution_mode"] == "compiled_cuda_graph"
    rep = va.validate_readbacks(va.load_readbacks(tmp_path / "rb"))
    assert rep["passed"], rep["errors"]
    # a plan that leaves a module to the framework routes to the native callable and records it as production
    mixed = FrameworkOperatorIntegration("vllm", "rollout", IntegrationPlan.uniform("P/R"))
    assert mixed.route("ffn", native, 1) == 0 and mixed.readback()["operators"]["ffn"]["implementation"] == "production"
    assert mixed.readback()["operators"]["ffn"]["backend_id"] == "vllm.production.ffn"
    # a strict operator whose own provenance admits a fallback is refused and remembered
    strict = FrameworkOperatorIntegration("megatron", "train", IntegrationPlan.uniform("R/R"),
                                          rl_kernel_operators={"logp": Op("rl_kernel_b200.linear_logp.bitwise.v1",
                                                                          {"runtime_platform": "cuda", "fallback": True, "actual_backend": "torch"})})
    with pytest.raises(RuntimeError, match="reported fallback"):
        strict.route("logp", native, 1)
    assert strict.readback()["fallbacks"][0]["module"] == "logp"
    with pytest.raises(RuntimeError, match="no operator was installed"):
        strict.route("attention", native, 1)
    with pytest.raises(ValueError, match="unknown integration module"):
        strict.record_installed_hook("sampler", "x")
