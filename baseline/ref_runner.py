"""Child process of the reference arm: a GRPO step built ONLY from the reference's public API.

    rollout : Qwen3DenseBIModel.forward (prefill) + .decode_step with its StatefulKVCache,
              support restriction by rl_engine.ops.sampling.policy.sampling_keep_mask
    scoring : Qwen3DenseBIModel.forward(target_ids=...) -> selected_logp   (reference policy + train pass)
    loss    : compute_policy_ratio / compute_reference_kl / masked_mean (rl_engine.validation.common)
    update  : torch autograd through the reference's operator profile inside its
              canonical_backward_session (rl_engine/ops/autograd/canonical_backward.py:131), one
              session per micro-batch as rl_engine/validation/models/chain_gate.py:1228 does per cell,
              + torch.optim.AdamW
Same synthetic data shape as the main arm: 8 prompts x group 8, prompt 512 + response 1024.
Prints one JSON line; any failure is reported as {"impl": "reference", "unavailable": ...}.

Row limit of one ``forward`` call.  The reference's Triton operator profile computes the LM head
with ``_det_gemm_fp32_kernel`` (rl_engine/backends/shared/triton/gemm/det_gemm.py:679-723), whose
output pointers are ``c_ptr + offs_m * stride_cm + offs_n * stride_cn`` in 32-bit integers.  With
the full vocabulary (stride_cm = 151936) the product passes 2^31 from row 14135 on and the store
lands outside the tensor.  An earlier version of this runner prefilled all 64 sequences x 512
prompt tokens in one ``forward`` (32768 rows) and met exactly that: "illegal memory access" in the
first forward.  The reference's own workloads never do this (its trainer scores a few sequences
per call), so the runner now prefills the 8 distinct prompts once (4096 rows), expands the cache
to the 64 samples, and checks ``MAX_FORWARD_ROWS`` before every call.

Why the training pass runs inside a canonical backward session.  Outside one, ``_linear``
(rl_engine/models/qwen3/reference.py:996-1031) multiplies through ``TritonDetGemmOp.forward_accum_fp32``;
the FFN down projection receives the FP32 SwiGLU product, and the backward of that autograd function
(backends/shared/triton/gemm/det_gemm.py:1050-1060) hands the saved FP32 operand to
``_triton_tree_gemm``, which raises "Triton tree GEMM requires BF16 inputs".  The reference's own
training cells never take that branch: with a session active and ``logical_keys`` given, every
projection, norm gain, embedding and the LM head go through the ``canonical_*`` functions, whose
parameter gradients are one GEMM over the rows sorted by (sample, position).
"""
from __future__ import annotations

import argparse
import json
import signal
import sys
import time

PROMPTS, GROUP, PROMPT_LEN = 8, 8, 512
VOCAB = 151936
MAX_FORWARD_ROWS = (2 ** 31 - 1) // VOCAB - 128      # rows of one forward call: 32-bit output offsets (see above)


PROGRESS: dict = {}


def _partial_report(budget: float) -> str:
    """What was measured before the time budget ran out (the reference's step is not interruptible, so an
    over-long run is reported with the rates seen so far instead of a number)."""
    pr, ph = PROGRESS.get("progress"), PROGRESS.get("phase")
    if not pr:
        return f"the reference did not finish its set-up within {budget:.0f} s"
    now = PROGRESS["clock"]()
    spent = now - pr["t_phase"]
    if pr["phase"] == "rollout":
        return (f"one reference step does not fit the arm's {budget:.0f} s budget: step {pr['step']} was still in its rollout "
                f"after {spent:.0f} s with {pr['decode_tokens_done']} decode tokens done")
    done, total = pr["microbatches_done"], pr["microbatches"]
    per = spent / max(done, 1)
    est = ph["rollout_s"] + per * total
    return (f"one reference step does not fit the arm's {budget:.0f} s budget: step {pr['step']} took {ph['rollout_s']:.0f} s "
            f"for its rollout and {spent:.0f} s for {done} of {total} scoring+training micro-batches "
            f"(about {per:.1f} s each), i.e. about {est:.0f} s per step")


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=1)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--response-len", type=int, default=1024)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--micro-batch", type=int, default=2)
    ap.add_argument("--time-budget", type=float, default=1500.0,
                    help="seconds for warm-up + timed steps together; fewer steps are run (and reported) when "
                         "the requested ones do not fit")
    a = ap.parse_args()
    try:
        out = run(a)
    except BaseException as exc:  # noqa: BLE001 - reported to the parent
        out = {"impl": "reference", "unavailable": f"{type(exc).__name__}: {str(exc)[:600]}"}
    print(json.dumps(out), flush=True)
    return 0


def run(a) -> dict:
    import torch

    import rl_engine  # noqa: F401  (must be the reference: the parent set PYTHONPATH)
    from rl_engine.models.qwen3.reference import Qwen3DenseBIModel, Qwen3DenseWeights, load_profile_ops
    from rl_engine.models.qwen3.spec import Qwen3DenseSpec
    from rl_engine.ops.autograd.canonical_backward import canonical_backward_session
    from rl_engine.ops.sampling.policy import sampling_keep_mask
    from rl_engine.validation.common import compute_policy_ratio, compute_reference_kl, masked_mean

    if "baseline/_ref" not in rl_engine.__file__.replace("\\", "/"):
        raise RuntimeError(f"imported {rl_engine.__file__}, not the reference install")
    dev = torch.device("cuda:0")
    spec = Qwen3DenseSpec.from_manifest()
    if a.layers:
        import dataclasses

        spec = dataclasses.replace(spec, num_hidden_layers=a.layers)
    ops = load_profile_ops("triton_cuda_bf16")
    weights = Qwen3DenseWeights.synthetic(spec, device=dev, dtype=torch.bfloat16, seed=1234)
    for k, t in weights.tensors.items():
        if t.dim() == 2:
            t.mul_(0.02)
    ref_weights = Qwen3DenseWeights({k: v.clone() for k, v in weights.tensors.items()}, "synthetic", "synthetic")
    params = [t.requires_grad_(True) for t in weights.tensors.values()]
    model = Qwen3DenseBIModel(spec, weights, ops)
    ref_model = Qwen3DenseBIModel(spec, ref_weights, ops)
    opt = torch.optim.AdamW(params, lr=1e-6, betas=(0.9, 0.95), weight_decay=0.01)
    B, P, R = PROMPTS * GROUP, PROMPT_LEN, a.response_len
    S = P + R
    total = a.warmup + a.steps
    host_prompts = torch.randint(0, spec.vocab_size, (total, PROMPTS, P),
                                 generator=torch.Generator().manual_seed(99)).pin_memory()
    host_loss = torch.empty(1).pin_memory()

    def check_rows(rows: int) -> None:
        if rows > MAX_FORWARD_ROWS:
            raise ValueError(f"{rows} rows in one forward call exceed the reference's 32-bit LM-head offsets "
                             f"({MAX_FORWARD_ROWS} rows at vocabulary {VOCAB})")

    def alarm(_sig, _frm):
        raise TimeoutError(_partial_report(a.time_budget))

    signal.signal(signal.SIGALRM, alarm)
    signal.alarm(int(a.time_budget))                      # one budget for everything: warm-up and timed steps

    phase = {"rollout_s": 0.0, "score_train_s": 0.0, "optimizer_s": 0.0}
    progress = {"step": -1, "phase": "start", "microbatches_done": 0, "microbatches": B // a.micro_batch,
                "decode_tokens_done": 0, "t_phase": 0.0}
    PROGRESS.update(progress=progress, phase=phase, clock=time.perf_counter)

    def lap(name: str, t0: float) -> float:
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        phase[name] = t1 - t0                      # the last step's split (the sync is part of every step anyway)
        return t1

    def one_step(i: int) -> None:
        t_phase = time.perf_counter()
        progress.update(step=i, phase="rollout", microbatches_done=0, decode_tokens_done=0, t_phase=t_phase)
        uniq = host_prompts[i].to(dev, non_blocking=True)
        prompts = uniq.repeat_interleave(GROUP, 0)
        # ---- rollout: every distinct prompt is prefilled once, its K/V then serve the whole group
        with torch.no_grad():
            check_rows(PROMPTS * P)
            pcache = model.allocate_cache(PROMPTS, S, dev)
            out = model.forward(uniq, kv_cache=pcache)
            logits = out["logits"][:, -1].float().repeat_interleave(GROUP, 0)
            cache = model.allocate_cache(B, S, dev)
            cache.k.copy_(pcache.k.repeat_interleave(GROUP, 1))
            cache.v.copy_(pcache.v.repeat_interleave(GROUP, 1))
            cache.lengths.copy_(pcache.lengths.repeat_interleave(GROUP, 1))
            cache.valid.copy_(pcache.valid.repeat_interleave(GROUP, 1))
            del pcache, out
            toks, lps = [], []
            pos = torch.full((B, 1), P, device=dev, dtype=torch.long)
            for t in range(R):
                keep = sampling_keep_mask(logits, temperature=1.0, top_k=-1, top_p=1.0)
                z = logits.masked_fill(~keep, float("-inf")) if keep is not None else logits
                probs = torch.softmax(z, -1)
                tok = torch.multinomial(probs, 1)
                toks.append(tok)
                lps.append(torch.log_softmax(z, -1).gather(1, tok))
                progress["decode_tokens_done"] = t + 1
                if t + 1 < R:
                    if t % 32 == 0:
                        torch.cuda.synchronize()          # lets the time budget interrupt a long rollout
                    out = model.decode_step(tok, cache, position_ids=pos)
                    logits = out["logits"][:, -1].float()
                    pos = pos + 1
            resp = torch.cat(toks, 1)
            old_logp = torch.cat(lps, 1)
            tokens = torch.cat([prompts, resp], 1)
            del cache
        t_phase = lap("rollout_s", t_phase)
        progress.update(phase="score_train", t_phase=t_phase)
        rewards = torch.bernoulli(torch.full((B,), 0.5, device=dev))
        g = rewards.view(PROMPTS, GROUP)
        adv = ((g - g.mean(1, keepdim=True)) / g.std(1, unbiased=False, keepdim=True).clamp_min(1e-6)).reshape(B)
        mask = torch.ones(B, R, dtype=torch.bool, device=dev)
        opt.zero_grad(set_to_none=True)
        loss_total = torch.zeros((), device=dev)
        check_rows(a.micro_batch * S)
        for b0 in range(0, B, a.micro_batch):
            tk = tokens[b0:b0 + a.micro_batch]
            with torch.no_grad():
                ref_lp = ref_model.forward(tk, target_ids=tk)["selected_logp"][:, P - 1:]
            keys = torch.stack([torch.arange(b0, b0 + tk.shape[0], device=dev)[:, None].expand(-1, S),
                                torch.arange(S, device=dev)[None, :].expand(tk.shape[0], -1)], -1)
            with canonical_backward_session() as session:
                lp = model.forward(tk, target_ids=tk, logical_keys=keys)["selected_logp"][:, P - 1:]
                m = mask[b0:b0 + a.micro_batch]
                ratio = compute_policy_ratio(lp, old_logp[b0:b0 + a.micro_batch], m)
                av = adv[b0:b0 + a.micro_batch, None].expand_as(lp)
                pol = -torch.minimum(ratio * av, torch.clamp(ratio, 0.8, 1.2) * av)
                kl = compute_reference_kl(lp, ref_lp, m)
                loss = (masked_mean(pol, m) + 0.001 * masked_mean(kl, m)) * (tk.shape[0] / B)
                loss.backward()
                session.validate_complete()
            loss_total += loss.detach()
            torch.cuda.synchronize()                      # a micro-batch is seconds long: the sync costs nothing
            progress["microbatches_done"] += 1
        t_phase = lap("score_train_s", t_phase)
        torch.nn.utils.clip_grad_norm_(params, 1.0)
        opt.step()
        host_loss.copy_(loss_total.reshape(1), non_blocking=True)
        torch.cuda.current_stream().synchronize()
        lap("optimizer_s", t_phase)
        progress["phase"] = "done"

    # warm-up and timed steps share one time budget: the reference's step is minutes long at full
    # size, and a run that is cut off from outside reports nothing at all
    t_begin = time.perf_counter()
    warm_done, step_s = 0, 0.0
    for i in range(a.warmup):
        ts = time.perf_counter()
        one_step(i)
        torch.cuda.synchronize()
        step_s = time.perf_counter() - ts
        warm_done += 1
        left = a.time_budget - (time.perf_counter() - t_begin)
        if left < step_s * (a.warmup - warm_done + 1) and warm_done >= 1:
            break                       # keep room for at least one timed step
    left = a.time_budget - (time.perf_counter() - t_begin)
    steps = max(1, min(a.steps, int(left // max(step_s, 1e-3)))) if warm_done else a.steps
    if warm_done and left < step_s:
        raise TimeoutError(f"one reference step takes {step_s:.0f} s (rollout {phase['rollout_s']:.0f} s, scoring+training "
                           f"{phase['score_train_s']:.0f} s); a warm-up step and a timed step do not both fit the arm's "
                           f"{a.time_budget:.0f} s budget")
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for i in range(a.warmup, a.warmup + steps):
        one_step(i)
    e1.record()
    torch.cuda.synchronize()
    signal.alarm(0)
    wall = time.perf_counter() - t0
    ms = e0.elapsed_time(e1) / steps
    tokens_per_step = B * S
    return {"metric": "qwen3_8b_grpo_step_tokens_per_s", "value": tokens_per_step / (ms / 1e3), "unit": "tokens/s",
            "n_gpus": 1, "steps": steps, "warmup": warm_done, "steps_requested": a.steps,
            "warmup_requested": a.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "impl": "reference",
            "data": "synthetic (uniform-random prompt ids, Bernoulli rewards, random-init weights)",
            "config": {"model": "Qwen3-8B" if not a.layers else f"Qwen3-8B-shape-{a.layers}L", "global_batch": B,
                       "seq_len": S, "parallelism": "single GPU", "operator_profile": "triton_cuda_bf16",
                       "micro_batch_seqs": a.micro_batch, "response_len": R,
                       "tokens_counted": "prompt + response tokens of every sequence"},
            "phase_s_last_step": {k: round(v, 3) for k, v in phase.items()},
            "e2e": {"value": tokens_per_step * steps / wall, "unit": "tokens/s",
                    "h2d_bytes_per_step": PROMPTS * P * 8, "d2h_bytes_per_step": 4}}


if __name__ == "__main__":
    sys.exit(main())
