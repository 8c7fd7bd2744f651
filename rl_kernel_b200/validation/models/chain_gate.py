"""Model chain gate (parity: run_chain_gate, rl_engine/validation/models/chain_gate.py:288-1874):
the whole decoder chain is run in packed / padded / singleton / chunked(decode) cells; the cells must
agree bit for bit with each other (invariance) and with the fp32 gold within the chain thresholds
max|dlogp| <= 0.06, approx_kl0 <= 0.05, clipfrac0 = 0 (train-infer parity aggregates); the first
node whose output drifts is located from captured node outputs."""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from rl_kernel_b200.contracts.numerical import chain_thresholds
from rl_kernel_b200.utils.bits import bit_equal


@dataclass
class ChainGateResult:
    cells: dict[str, bool] = field(default_factory=dict)
    aggregates: dict[str, float] = field(default_factory=dict)
    first_drift: str | None = None
    passed: bool = False


def parity_aggregates(candidate_logp: torch.Tensor, gold_logp: torch.Tensor, clip_eps: float = 0.2) -> dict[str, float]:
    d = gold_logp.double() - candidate_logp.double()
    ratio = torch.exp(candidate_logp.double() - gold_logp.double())
    return {"max_abs_dlogp": float(d.abs().max()), "approx_kl0": float((torch.exp(d) - d - 1).mean()),
            "clipfrac0": float(((ratio < 1 - clip_eps) | (ratio > 1 + clip_eps)).double().mean())}


def locate_first_drift(candidate_nodes: dict[str, torch.Tensor], gold_nodes: dict[str, torch.Tensor], order,
                       rtol: float = 5e-2) -> str | None:
    for name in order:
        if name in candidate_nodes and name in gold_nodes:
            c, g = candidate_nodes[name].float(), gold_nodes[name].float()
            if c.shape == g.shape and float((c - g).abs().max()) > rtol * float(g.abs().max().clamp_min(1e-6)):
                return name
    return None


def run_chain_gate(model, gold_model, input_ids: torch.Tensor, *, decode_from: int | None = None) -> ChainGateResult:
    """``model`` / ``gold_model``: Qwen3DenseBIModel-like (forward, decode_step, allocate_cache,
    selected_logprobs, captured_node_outputs)."""
    res = ChainGateResult()
    B, S = input_ids.shape
    full = model(input_ids, target_ids=input_ids, capture_nodes=True, return_logits=False)
    nodes = model.captured_node_outputs()
    lp = full["selected_logp"]
    res.cells["packed/full"] = True
    singles = torch.cat([model(input_ids[i:i + 1], target_ids=input_ids[i:i + 1], return_logits=False)["selected_logp"]
                         for i in range(B)])
    res.cells["singletons"] = bit_equal(singles, lp)
    perm = torch.arange(B - 1, -1, -1)
    res.cells["permuted"] = bit_equal(model(input_ids[perm], target_ids=input_ids[perm], return_logits=False)["selected_logp"], lp[perm])
    pad = torch.cat([input_ids, input_ids[:1]])
    res.cells["padded_batch"] = bit_equal(model(pad, target_ids=pad, return_logits=False)["selected_logp"][:B], lp)
    if decode_from is not None and 0 < decode_from < S - 1:
        cache = model.allocate_cache(B, S + 1)
        model(input_ids[:, :decode_from], kv_cache=cache, return_logits=False)
        cols = []
        for t in range(decode_from, S - 1):
            out = model.decode_step(input_ids[:, t], torch.full((B,), t), cache, return_logits=False)
            cols.append(model.selected_logprobs(out["hidden"].reshape(B, -1), input_ids[:, t + 1]))
        res.cells["chunked/decode"] = bit_equal(torch.stack(cols, 1), lp[:, decode_from:S - 1])
    gold = gold_model(input_ids, target_ids=input_ids, capture_nodes=True, return_logits=False)
    res.aggregates = parity_aggregates(lp, gold["selected_logp"])
    th = chain_thresholds()
    ok_acc = (res.aggregates["max_abs_dlogp"] <= th["max_abs_dlogp"] and res.aggregates["approx_kl0"] <= th["approx_kl0"]
              and res.aggregates["clipfrac0"] <= th["clipfrac0"])
    if not ok_acc:
        res.first_drift = locate_first_drift(nodes, gold_model.captured_node_outputs(), model.node_names())
    res.passed = ok_acc and all(res.cells.values())
    return res
