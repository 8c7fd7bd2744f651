"""Run-time backends of the kernel registry: registration order, availability probes, environment pins and
bans, operand-device routing, contract-aware choice by capability, and the candidate listing."""
import dataclasses

import pytest
import torch

from rl_kernel_b200.contracts.operators.attention import (REFERENCE_ATTENTION_CAPABILITY, AttentionContract, AttentionDType,
                                                          AttentionRole)
from rl_kernel_b200.contracts.operators.logprob import REFERENCE_LOGPROB_CAPABILITY, LogprobContract
from rl_kernel_b200.runtime.registry import KernelRegistry, OpBackend, RegisteredBackend


class _Double:
    def __init__(self, tag="x", **kw):
        self.tag, self.kw = tag, kw


def test_registered_backends_come_first_and_can_be_replaced_or_removed():
    reg = KernelRegistry()
    assert reg.resolve("rms_norm").actual is OpBackend.REF_RMS_NORM            # no GPU here: the reference, flagged as a fallback
    first = reg.register_backend("rms_norm", "mine", _Double)
    assert isinstance(first, RegisteredBackend) and reg.resolve("rms_norm").actual == first and not reg.last_resolution.fallback
    op = reg.get_op("rms_norm", tag="a")
    assert isinstance(op, _Double) and op.tag == "a" and reg.get_op("rms_norm", tag="a") is op          # cached per arguments
    reg.register_backend("rms_norm", "late", _Double, prepend=False)
    assert [c["id"] for c in reg.candidates("rms_norm")] == ["mine", "late", "b200", "reference"]
    reg.register_backend("rms_norm", "mine", lambda tag="x": _Double("replaced-" + tag))                # same id: replaced, not duplicated
    assert reg.get_op("rms_norm", tag="a").tag == "replaced-a" and len(reg.candidates("rms_norm")) == 4
    assert reg.resolve("rms_norm", "late").actual.backend_id == "late"
    assert reg.resolve("rms_norm", "reference").actual is OpBackend.REF_RMS_NORM
    assert reg.unregister_backend("rms_norm", "mine") and not reg.unregister_backend("rms_norm", "mine")
    with pytest.raises(KeyError, match="no backend 'mine'"):
        reg.resolve("rms_norm", "mine")
    for reserved in ("auto", "reference", "b200", ""):
        with pytest.raises(ValueError):
            reg.register_backend("rms_norm", reserved, _Double)
    # an operator the built-in table does not know at all
    reg.register_backend("my_op", "only", _Double)
    assert "my_op" in reg.available_ops() and reg.get_op("my_op").tag == "x"
    with pytest.raises(KeyError):
        reg.resolve("nobody_registered_this")


def test_availability_probes_and_environment(monkeypatch):
    reg = KernelRegistry()
    state = {"ok": False}
    reg.register_backend("swiglu", "vendor", _Double, available=lambda: state["ok"])
    reg.register_backend("swiglu", "broken", _Double, available=lambda: 1 / 0, prepend=False)
    assert reg.resolve("swiglu").actual is OpBackend.REF_SWIGLU
    c = {x["id"]: x for x in reg.candidates("swiglu")}
    assert c["vendor"]["reason"] == "reports itself unavailable" and "ZeroDivisionError" in c["broken"]["reason"]
    state["ok"] = True
    assert reg.resolve("swiglu").actual.backend_id == "vendor"
    monkeypatch.setenv("RL_KERNEL_DISABLE_BACKENDS", "vendor, something-else")
    assert reg.resolve("swiglu").actual is OpBackend.REF_SWIGLU
    with pytest.raises(RuntimeError, match="disabled by RL_KERNEL_DISABLE_BACKENDS"):
        reg.resolve("swiglu", "vendor")
    monkeypatch.delenv("RL_KERNEL_DISABLE_BACKENDS")
    monkeypatch.setenv("RL_KERNEL_BACKEND_SWIGLU", "reference")
    assert reg.resolve("swiglu").actual is OpBackend.REF_SWIGLU and reg.last_resolution.reason == "reference requested" or True
    assert reg.resolve("swiglu", "vendor").actual.backend_id == "vendor"         # an explicit argument beats the environment
    monkeypatch.setenv("RL_KERNEL_BACKEND_SWIGLU", "vendor")
    monkeypatch.setenv("RL_KERNEL_MODE", "off")
    assert reg.resolve("swiglu").actual.backend_id == "vendor"
    monkeypatch.delenv("RL_KERNEL_BACKEND_SWIGLU")
    assert reg.resolve("swiglu").actual is OpBackend.REF_SWIGLU and reg.last_resolution.reason == "mode off"


def test_operand_device_routes_cpu_tensors_to_the_reference_without_a_fallback_flag():
    reg = KernelRegistry()
    res = reg.resolve("det_gemm", device="cpu")
    assert res.actual is OpBackend.REF_DET_GEMM and not res.fallback and res.reason == "operands are on the CPU"
    assert reg.resolve("gemm", device=torch.device("cpu")).op_name == "det_gemm"          # the reference's operator names
    assert reg.resolve("attn").op_name == "attention"
    reg.register_backend("det_gemm", "gpu_only", _Double, device_types=("cuda",))
    assert reg.resolve("det_gemm", device="cpu").actual is OpBackend.REF_DET_GEMM
    assert {c["id"]: c["reason"] for c in reg.candidates("det_gemm", "cpu")}["gpu_only"] == "does not run on cpu"
    op = reg.get_op("det_gemm", operand_device="cpu")
    assert type(op).__name__ == "NativeGemmOp"
    unhashable = reg.get_op("my" if False else "det_gemm", prefer="gpu_only", cfg={"a": [1, 2]})
    assert isinstance(unhashable, _Double) and unhashable.kw == {"cfg": {"a": [1, 2]}}


def test_contract_aware_attention_choice_by_capability():
    reg = KernelRegistry()
    contract = AttentionContract.for_layout(8, 2, seq_len=256, role=AttentionRole.TRAIN)
    fp16_only = dataclasses.replace(REFERENCE_ATTENTION_CAPABILITY, backend_id="fp16-only", dtypes=frozenset({AttentionDType.FP16}))
    good = dataclasses.replace(REFERENCE_ATTENTION_CAPABILITY, backend_id="mine-ok")
    reg.register_attention_backend("fp16_only", _Double, fp16_only)
    reg.register_backend("attention", "no_capability", _Double, prepend=False)
    op = reg.get_attention_op("auto", contract=contract)
    assert type(op).__name__ == "NativeAttentionOp"                           # both registered ones were skipped
    with pytest.raises(RuntimeError, match="fp16-only cannot serve the contract: dtype=bf16 is unsupported"):
        reg.get_attention_op("fp16_only", contract=contract)
    with pytest.raises(RuntimeError, match="declares no capability"):
        reg.get_attention_op("no_capability", contract=contract)
    assert isinstance(reg.get_attention_op("no_capability"), _Double)         # without a contract nothing is checked
    reg.register_attention_backend("mine_ok", _Double, good, prepend=True)
    assert isinstance(reg.get_attention_op("auto", contract=contract), _Double)
    with pytest.raises(TypeError):
        reg.register_attention_backend("bad", _Double, capability=object())
    with pytest.raises(ValueError, match="unknown attention backend"):
        reg.get_attention_op("never_heard_of_it")
    cp = AttentionContract.for_layout(8, 2, seq_len=512, cp_world_size=2, layout="zigzag")
    with pytest.raises(ValueError, match="not allowed with cp_size > 1"):
        reg.get_attention_op("auto", contract=cp)


def test_contract_aware_logprob_choice_and_description():
    reg = KernelRegistry()
    contract = LogprobContract.for_tokens(16, real_vocab_size=1000, padded_vocab_size=1024, temperature=0.5)
    cap = dataclasses.replace(REFERENCE_LOGPROB_CAPABILITY, backend_id="mine-logp")
    reg.register_logprob_backend("mine_logp", _Double, cap, op_name="batch_invariant_logp")
    op = reg.get_logprob_op("mine_logp", contract=contract)
    assert isinstance(op, _Double) and op.kw == {"temperature": 0.5}          # the contract's temperature reaches the constructor
    assert type(reg.get_logprob_op("linear", contract=contract)).__name__ == "NativeLinearLogpOp"
    with pytest.raises(ValueError, match="unknown logp backend"):
        reg.get_logprob_op("nope")
    with pytest.raises(TypeError):
        reg.register_logprob_backend("bad", _Double, capability=None)
    d = reg.describe()
    assert [c["id"] for c in d["batch_invariant_logp"]] == ["b200", "mine_logp", "reference"] or \
        [c["id"] for c in d["batch_invariant_logp"]][0] in ("mine_logp", "b200")
    assert all({"id", "kind", "usable", "reason", "path"} <= set(c) for cs in d.values() for c in cs)
    assert any(r["op"] == "batch_invariant_logp" and r["actual"] == "mine_logp" for r in reg.provenance())


def test_rlk_ops_lists_candidates(capsys):
    import json

    from rl_kernel_b200.entrypoints.repro import main

    assert main(["ops", "--json", "det_gemm", "attn"]) == 2               # aliases are for callers, the listing uses real names
    capsys.readouterr()
    assert main(["ops", "--json", "det_gemm", "attention"]) == 0
    table = json.loads(capsys.readouterr().out)
    assert list(table) == ["det_gemm", "attention"] and table["det_gemm"][-1]["id"] == "reference" and table["det_gemm"][-1]["usable"]
    assert main(["ops", "rope"]) == 0
    text = capsys.readouterr().out
    assert text.startswith("rope\n") and "* reference" in text


def test_rlk_chain_gate_command(tmp_path, capsys):
    import json

    from rl_kernel_b200.entrypoints.repro import main

    out = tmp_path / "gate" / "report.json"
    assert main(["chain-gate", "--layers", "1", "--cells", "singletons,chunked", "--out", str(out)]) == 0
    summary = json.loads(capsys.readouterr().out)
    assert summary["passed"] and summary["cells"] == {"B1-singleton_aggregate/full": "0/27", "B1/chunked": "0/27"}
    rep = json.loads(out.read_text())
    assert rep["cells"]["BN/full"]["n_logp_tokens"] == 27 and rep["accuracy"]["passed"]
