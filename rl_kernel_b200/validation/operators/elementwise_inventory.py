"""Inventory of the elementwise / RoPE work on the Qwen3 training and rollout chain (parity: rl_engine/validation/
operators/elementwise_inventory.py:20-215).

Every item says where on the chain it sits, which entry point of this framework computes it, whether it reduces
(and over what), and its verdict.  Items with an operator spec are *executed* by ``run_inventory`` through the
four-judgment harness; items fused into another kernel name the kernel that carries them and are judged with it."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Literal

Verdict = Literal["pass", "blocker", "blocked_hardware", "tracked_red", "absent_not_required"]


@dataclass(frozen=True)
class InventoryItem:
    name: str
    category: str                 # elementwise | rope | norm | residual | gather | cast
    on_chain: bool
    differentiable: bool
    entry_point: str
    reduction: str                # none | row (over the hidden / head dim) | token (over tokens, in a gradient)
    spec: str | None = None       # operator-spec name that executes it, if it has one of its own
    carried_by: str | None = None  # kernel that contains it when it has no launch of its own
    verdict: Verdict = "pass"
    note: str = ""


_I = InventoryItem
_ITEMS: tuple[InventoryItem, ...] = (
    _I("embedding_lookup", "gather", True, True, "rl_kernel_b200.ops.embedding.canonical_embedding.embedding", "token", spec="embedding",
       note="forward is a row copy; the weight gradient sums duplicate ids in ascending token order"),
    _I("input_rmsnorm", "norm", True, True, "rl_kernel_b200.ops.norm.rms_norm", "row", spec="rms_norm"),
    _I("residual_add", "residual", True, True, "csrc/norm/rmsnorm.cu: rmsnorm_fwd(res=, res_out=)", "none", carried_by="rms_norm",
       note="fused into the following RMSNorm: one read of x and the residual, one write of each"),
    _I("q_norm", "norm", True, True, "rl_kernel_b200.ops.norm.rms_norm over [T, H, D]", "row", spec="qk_norm"),
    _I("k_norm", "norm", True, True, "rl_kernel_b200.ops.norm.rms_norm over [T, Hkv, D]", "row", spec="qk_norm"),
    _I("rope_q", "rope", True, True, "rl_kernel_b200.ops.rope.rope", "none", spec="rope",
       note="in the engine the rotation is fused with q/k norm (csrc/norm/qk_norm_rope.cu); the stand-alone kernel is bit-equal"),
    _I("rope_k", "rope", True, True, "rl_kernel_b200.ops.rope.rope", "none", spec="rope"),
    _I("attention_scale", "elementwise", True, True, "csrc/attention/attn_fwd_sm100.cu (softmax prologue)", "none", carried_by="attention",
       note="applied to the fp32 scores inside exp2: never to bf16 q"),
    _I("swiglu", "elementwise", True, True, "rl_kernel_b200.ops.activation.swiglu", "none", spec="swiglu",
       note="in the engine it runs in the gate/up GEMM epilogue on the fp32 accumulators and rounds once"),
    _I("silu", "elementwise", False, True, "rl_kernel_b200.backends.cuda.activation.swiglu.SiLUCudaOp", "none", spec="silu"),
    _I("post_attention_rmsnorm", "norm", True, True, "rl_kernel_b200.ops.norm.rms_norm", "row", spec="rms_norm"),
    _I("final_rmsnorm", "norm", True, True, "rl_kernel_b200.ops.norm.rms_norm", "row", spec="rms_norm"),
    _I("logit_temperature", "elementwise", True, True, "csrc/gemm/det_gemm_sm100.cu (LM-head epilogue)", "none", carried_by="linear_logp",
       note="multiplies the fp32 accumulator by 1/T before the tile statistics"),
    _I("support_threshold_mask", "elementwise", True, True, "csrc/logprob/logp.cu, LM-head epilogue", "none", carried_by="linear_logp",
       note="top-k / top-p replay: scaled logits below the token's threshold count as -inf"),
    _I("policy_ratio_kl", "elementwise", True, True, "rl_kernel_b200.ops.loss.grpo_loss", "token", spec="grpo_loss"),
    _I("bf16_casts", "cast", True, False, "every kernel's epilogue", "none", carried_by="det_gemm",
       note="one rounding per kernel output; no intermediate bf16 round trips inside a kernel"),
    _I("dropout", "elementwise", False, False, "-", "none", verdict="absent_not_required", note="Qwen3 trains without dropout"),
    _I("attention_bias", "elementwise", False, False, "-", "none", verdict="absent_not_required", note="Qwen3 projections have no bias"),
)


def inventory_items() -> tuple[InventoryItem, ...]:
    return _ITEMS


def inventory_names() -> tuple[str, ...]:
    return tuple(i.name for i in _ITEMS)


def unresolved_needs_fix() -> tuple[InventoryItem, ...]:
    return tuple(i for i in _ITEMS if i.verdict in ("blocker", "tracked_red"))


def unexecuted_cells() -> tuple[InventoryItem, ...]:
    """On-chain items that neither have a spec of their own nor name a carrying kernel."""
    return tuple(i for i in _ITEMS if i.on_chain and i.spec is None and i.carried_by is None)


def run_inventory(device: str = "cpu", dtype=None) -> dict[str, dict]:
    """Execute every item: its own spec, or the spec of the kernel that carries it.  -> {item: {judgment: status}}."""
    import torch

    from rl_kernel_b200.validation.operators.four_judgment_matrix import judge_operator

    dtype = dtype or (torch.bfloat16 if device.startswith("cuda") else torch.float32)
    cache: dict[str, dict] = {}
    out = {}
    for item in _ITEMS:
        spec = item.spec or item.carried_by
        if spec is None or item.verdict == "absent_not_required":
            out[item.name] = {"status": item.verdict}
            continue
        if spec not in cache:
            cache[spec] = {j: s for j, (s, _) in judge_operator(spec, device, dtype).items()}
        out[item.name] = {"executed_as": spec, **cache[spec]}
    return out


__all__ = ["InventoryItem", "Verdict", "inventory_items", "inventory_names", "run_inventory", "unexecuted_cells", "unresolved_needs_fix"]
