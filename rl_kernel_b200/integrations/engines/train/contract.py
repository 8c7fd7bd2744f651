"""Contract between the orchestrator and training / scoring workers (parity:
rl_engine/integrations/engines/train/contract.py:22-1026)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Protocol

import torch

from rl_kernel_b200.ops.loss import group_advantages


@dataclass
class RolloutStageResult:
    tokens: torch.Tensor            # [B, S] prompt + response
    response_mask: torch.Tensor     # [B, R]
    rollout_logp: torch.Tensor      # [B, R] fp32, recorded by the sampler with the strict operator
    rewards: torch.Tensor           # [B]
    prompt_len: int
    samples_per_prompt: int
    weight_version: int = 0
    metadata: dict = field(default_factory=dict)

    def validate(self) -> None:
        B, R = self.rollout_logp.shape
        if self.tokens.shape[0] != B or self.response_mask.shape != (B, R) or self.rewards.shape[0] != B:
            raise ValueError("rollout result tensors disagree on the batch / response size")
        if self.tokens.shape[1] != self.prompt_len + R:
            raise ValueError("tokens must be prompt_len + response_len wide")
        if B % self.samples_per_prompt:
            raise ValueError("batch must be a multiple of samples_per_prompt")


@dataclass
class TrainingStageResult:
    loss: float
    policy_loss: float
    kl: float
    grad_norm: float
    train_logp: torch.Tensor
    mismatch_count: int
    tokens_compared: int
    weight_version: int
    metrics: dict = field(default_factory=dict)


class TrainingWorker(Protocol):
    def train(self, rollout: RolloutStageResult) -> TrainingStageResult: ...
    def publish_weights(self, weight_version: int): ...


class RolloutBatchMixin:
    @staticmethod
    def advantages(rollout: RolloutStageResult, eps: float = 1e-6) -> torch.Tensor:
        return group_advantages(rollout.rewards, rollout.samples_per_prompt, eps)

    @staticmethod
    def mismatches(train_logp: torch.Tensor, rollout: RolloutStageResult) -> int:
        m = rollout.response_mask.bool()
        return int(((train_logp.view(torch.int32) != rollout.rollout_logp.view(torch.int32)) & m).sum())


class StatelessScoringWorker:
    """Reference / reward scoring worker: no KV cache, no state between calls."""

    def __init__(self, executor):
        self.executor = executor

    def score(self, rollout: RolloutStageResult) -> torch.Tensor:
        lp = self.executor.score(rollout.tokens)
        return lp[:, -rollout.rollout_logp.shape[1]:]


# ================================================================================================ rollout payloads
# (parity: the payload side of rl_engine/integrations/engines/train/contract.py:58-1026: serving engines hand back grouped
#  candidates in several shapes; workers read them through these functions and attach scores in place)
import math
from typing import Any, Optional, Sequence


@dataclass(frozen=True)
class TorchRLTrainingConfig:
    learning_rate: float = 1e-6
    clip_eps: float = 0.2
    kl_coef: float = 0.0
    max_grad_norm: float = 1.0
    micro_batch_size: int = 8
    temperature: float = 1.0
    advantage_eps: float = 1e-6
    pad_token_id: int = 0
    use_rollout_logprobs: bool = False          # take the sampler's log-probs as old log-probs instead of recomputing them
    seed: int = 1234

    def __post_init__(self) -> None:
        if self.learning_rate <= 0 or self.micro_batch_size <= 0 or self.temperature <= 0:
            raise ValueError("learning_rate, micro_batch_size and temperature must be positive")
        if not 0 <= self.clip_eps < 1 or self.kl_coef < 0:
            raise ValueError("clip_eps must lie in [0, 1) and kl_coef must not be negative")


def _get(obj: Any, *names: str, default=None):
    for n in names:
        if isinstance(obj, dict):
            if n in obj:
                return obj[n]
        elif hasattr(obj, n):
            return getattr(obj, n)
    return default


def _ints(v: Any) -> list[int]:
    if isinstance(v, torch.Tensor):
        v = v.tolist()
    out = [int(x) for x in v]
    if any(isinstance(x, bool) for x in v):
        raise TypeError("token ids must be integers")
    return out


def _floats(v: Any) -> list[float]:
    if isinstance(v, torch.Tensor):
        v = v.tolist()
    return [float(x) for x in v]


def _groups(payload: Any) -> list[Any]:
    """The prompt groups of a payload: a list of groups, or an object / dict with ``grouped_outputs`` / ``groups`` / ``outputs``."""
    inner = _get(payload, "grouped_outputs", "groups", default=None)
    if inner is None:
        inner = payload
    if not isinstance(inner, (list, tuple)):
        raise TypeError("a rollout payload is a sequence of prompt groups (or carries one as grouped_outputs / groups)")
    return list(inner)


def _candidates(group: Any) -> tuple[list[int], list[Any]]:
    """(prompt ids, candidates) of one group.  A group is a serving engine's request output (``prompt_token_ids`` plus
    ``outputs``), a dict of that shape, or a plain list of candidates."""
    outs = _get(group, "outputs", "candidates", "samples", default=None)
    prompt = _get(group, "prompt_token_ids", "prompt_ids", default=None)
    if outs is None:
        if not isinstance(group, (list, tuple)):
            raise TypeError("a prompt group needs outputs / candidates")
        outs = group
    return ([] if prompt is None else _ints(prompt)), list(outs)


def candidate_token_ids(candidate: Any) -> list[int]:
    ids = _get(candidate, "token_ids", "completion_token_ids", "response_token_ids", "tokens", default=None)
    if ids is None:
        if isinstance(candidate, (list, tuple, torch.Tensor)):
            return _ints(candidate)
        raise TypeError("a candidate needs token_ids")
    return _ints(ids)


def candidate_prompt_token_ids(candidate: Any, group_prompt: Sequence[int] = ()) -> list[int]:
    own = _get(candidate, "prompt_token_ids", "prompt_ids", default=None)
    return _ints(own) if own is not None else list(group_prompt)


def candidate_reward(candidate: Any) -> Optional[float]:
    r = _get(candidate, "reward", "score", default=None)
    if r is None:
        md = _get(candidate, "metadata", "extra", default=None)
        r = _get(md, "reward", default=None) if md is not None else None
    if r is None:
        return None
    r = float(r)
    if not math.isfinite(r):
        raise ValueError("a candidate's reward must be finite")
    return r


def candidate_reference_logps(candidate: Any) -> Optional[list[float]]:
    v = _get(candidate, "reference_logprobs", "ref_logprobs", "reference_logps", default=None)
    return None if v is None else _floats(v)


def candidate_rollout_logps(candidate: Any) -> Optional[list[float]]:
    v = _get(candidate, "rollout_logprobs", "token_logprobs", "logprobs", default=None)
    if v is None:
        return None
    if v and isinstance(v[0], dict):                      # a serving engine's per-token {id: Logprob} maps
        ids = candidate_token_ids(candidate)
        return [float(_get(d[t], "logprob", default=d[t])) for d, t in zip(v, ids)]
    return _floats(v)


def extract_rollout_candidate_groups(payload: Any) -> list[list[list[int]]]:
    return [[candidate_token_ids(c) for c in _candidates(g)[1]] for g in _groups(payload)]


def extract_rollout_token_groups(payload: Any) -> list[list[int]]:
    """Prompt ids of every group."""
    return [_candidates(g)[0] for g in _groups(payload)]


def extract_rollout_reward_groups(payload: Any) -> list[list[float]]:
    out = []
    for g in _groups(payload):
        rs = [candidate_reward(c) for c in _candidates(g)[1]]
        if any(r is None for r in rs):
            raise ValueError("every candidate needs a reward before the batch is built")
        out.append(rs)
    return out


def extract_rollout_reference_logp_groups(payload: Any) -> list[list[list[float]]]:
    out = []
    for g in _groups(payload):
        ls = [candidate_reference_logps(c) for c in _candidates(g)[1]]
        if any(x is None for x in ls):
            raise ValueError("every candidate needs reference log-probs")
        out.append(ls)
    return out


def _set(candidate: Any, name: str, value: Any) -> None:
    if isinstance(candidate, dict):
        candidate[name] = value
    else:
        try:
            setattr(candidate, name, value)
        except AttributeError as exc:
            raise TypeError(f"cannot attach {name} to a {type(candidate).__name__}; use objects or dicts as candidates") from exc


def attach_stateless_scores_to_payload(payload: Any, *, rewards: Optional[torch.Tensor] = None,
                                       reference_logps: Optional[torch.Tensor] = None, completion_mask: Optional[torch.Tensor] = None) -> Any:
    """Write a scoring worker's results back onto the candidates, in payload order: ``rewards`` [B]; ``reference_logps``
    [B, L] with ``completion_mask`` [B, L] marking each candidate's own tokens (right-padded)."""
    flat = [c for g in _groups(payload) for c in _candidates(g)[1]]
    if rewards is not None:
        if rewards.shape[0] != len(flat):
            raise ValueError(f"{rewards.shape[0]} rewards for {len(flat)} candidates")
        for c, r in zip(flat, rewards.tolist()):
            _set(c, "reward", float(r))
    if reference_logps is not None:
        if reference_logps.shape[0] != len(flat):
            raise ValueError(f"{reference_logps.shape[0]} log-prob rows for {len(flat)} candidates")
        for i, c in enumerate(flat):
            n = len(candidate_token_ids(c))
            row = reference_logps[i][completion_mask[i].bool()] if completion_mask is not None else reference_logps[i, :n]
            if row.numel() != n:
                raise ValueError(f"candidate {i}: {row.numel()} log-probs for {n} tokens")
            _set(c, "reference_logprobs", row.tolist())
    return payload


def build_stateless_inputs_from_rollout_payload(payload: Any, *, pad_token_id: int = 0):
    """Right-padded [B, S] ids with attention and completion masks: what a stateless scoring worker needs."""
    from rl_kernel_b200.runtime.executor import StatelessForwardInputs

    rows, comp = [], []
    for g in _groups(payload):
        prompt, cands = _candidates(g)
        for c in cands:
            p = candidate_prompt_token_ids(c, prompt)
            t = candidate_token_ids(c)
            if not p or not t:
                raise ValueError("every candidate needs a non-empty prompt and completion")
            rows.append(p + t)
            comp.append((len(p), len(t)))
    S = max(len(r) for r in rows)
    ids = torch.full((len(rows), S), pad_token_id, dtype=torch.long)
    attn = torch.zeros(len(rows), S, dtype=torch.bool)
    cm = torch.zeros(len(rows), S, dtype=torch.bool)
    for i, (r, (np_, nt)) in enumerate(zip(rows, comp)):
        ids[i, : len(r)] = torch.tensor(r)
        attn[i, : len(r)] = True
        cm[i, np_: np_ + nt] = True
    return StatelessForwardInputs(ids, attn, cm)


def compute_group_relative_advantages(reward_groups: Sequence[Sequence[float]], eps: float = 1e-6) -> list[list[float]]:
    """(r - mean) / std per prompt group, two-pass variance; a group whose rewards are all equal gets zeros."""
    out = []
    for g in reward_groups:
        r = torch.tensor(list(g), dtype=torch.float32)
        d = r - r.mean()
        var = (d * d).mean()
        out.append((d / var.clamp_min(eps ** 2).sqrt()).tolist())
    return out


def broadcast_sequence_advantages(advantages: torch.Tensor, completion_mask: torch.Tensor) -> torch.Tensor:
    """[B] -> [B, L]: the sequence's advantage on its own tokens, zero elsewhere."""
    return advantages.float().view(-1, 1) * completion_mask.float()


def objective_reference_logps(reference_logps: Optional[torch.Tensor], policy_logps: torch.Tensor, kl_coef: float) -> Optional[torch.Tensor]:
    """What the loss takes as reference: nothing without a KL term, the scored reference otherwise (it must exist)."""
    if kl_coef == 0:
        return None
    if reference_logps is None:
        raise ValueError("a KL term needs reference log-probs")
    if reference_logps.shape != policy_logps.shape:
        raise ValueError("reference and policy log-probs must have one shape")
    return reference_logps


def make_rollout_result(payload: Any, *, samples_per_prompt: Optional[int] = None, pad_token_id: int = 0, weight_version: int = 0
                        ) -> RolloutStageResult:
    """A ``RolloutStageResult`` from a grouped payload whose candidates carry token ids, rollout log-probs and rewards.
    Prompts must have one length and completions are right-padded to the longest."""
    prompts = extract_rollout_token_groups(payload)
    cands = extract_rollout_candidate_groups(payload)
    rewards = extract_rollout_reward_groups(payload)
    g = samples_per_prompt or len(cands[0])
    if any(len(c) != g for c in cands):
        raise ValueError("every prompt group must hold samples_per_prompt candidates")
    P = len(prompts[0])
    if P == 0 or any(len(p) != P for p in prompts):
        raise ValueError("prompts must be non-empty and of one length")
    flat = [c for grp in _groups(payload) for c in _candidates(grp)[1]]
    R = max(len(t) for grp in cands for t in grp)
    B = len(flat)
    tokens = torch.full((B, P + R), pad_token_id, dtype=torch.long)
    mask = torch.zeros(B, R, dtype=torch.bool)
    lp = torch.zeros(B, R, dtype=torch.float32)
    i = 0
    for prompt, grp in zip(prompts, cands):
        for t in grp:
            tokens[i, :P] = torch.tensor(prompt)
            tokens[i, P: P + len(t)] = torch.tensor(t)
            mask[i, : len(t)] = True
            rl = candidate_rollout_logps(flat[i])
            if rl is None or len(rl) != len(t):
                raise ValueError(f"candidate {i} needs one rollout log-prob per token")
            lp[i, : len(t)] = torch.tensor(rl)
            i += 1
    res = RolloutStageResult(tokens, mask, lp, torch.tensor([r for grp in rewards for r in grp], dtype=torch.float32), P, g, weight_version)
    res.validate()
    return res


# ================================================================================================ training batches
# (parity: RolloutBatchMixin._batch_from_rollout_or_synthetic / _batch_from_candidate_groups,
#  rl_engine/integrations/engines/train/contract.py:84-305)
def batch_from_candidate_groups(candidate_groups: Sequence[Sequence[Sequence[int]]], prompt_groups: Sequence[Sequence[int]] | None = None, *,
                                reward_groups: Sequence[Sequence[float]] | None = None,
                                reference_logp_groups: Sequence[Sequence[Sequence[float]]] | None = None,
                                rollout_logp_groups: Sequence[Sequence[Sequence[float]]] | None = None, completion_len: int | None = None,
                                pad_token_id: int = 0, advantage_eps: float = 1e-6, dtype: torch.dtype = torch.float32,
                                device: torch.device | str = "cpu"):
    """A ``SyntheticRLKernelBatch``-shaped training batch from grouped completions.  Prompts (one per group, one length)
    are left-aligned, completions right-padded (or cut) to ``completion_len``; advantages are group-relative from the
    rewards (a reward a payload does not carry is replaced by a token-id proxy, named as such in the metadata);
    reference / old log-probs default to zero with the source recorded."""
    from rl_kernel_b200.validation.common.rl_batch import SyntheticRLKernelBatch

    groups = [[list(map(int, c)) for c in grp] for grp in candidate_groups]
    if not groups or any(not grp for grp in groups):
        raise ValueError("every prompt group needs at least one completion")
    prompts = [list(map(int, p)) for p in (prompt_groups or [[] for _ in groups])]
    if len(prompts) != len(groups):
        raise ValueError("one prompt per group")
    P = len(prompts[0])
    if any(len(p) != P for p in prompts):
        raise ValueError("prompts must have one length")
    L = completion_len or max(len(c) for grp in groups for c in grp)
    if L < 1:
        raise ValueError("completions are empty")
    B = sum(len(grp) for grp in groups)
    ids = torch.full((B, P + L), pad_token_id, dtype=torch.long)
    cmask = torch.zeros(B, L, dtype=torch.bool)
    old, ref = torch.zeros(B, L), torch.zeros(B, L)
    rewards = torch.zeros(B)
    adv_rows: list[float] = []
    sizes = []
    i = 0
    have_r = reward_groups is not None and [len(g) for g in reward_groups] == [len(g) for g in groups]
    for gi, grp in enumerate(groups):
        rs = [float(x) for x in reward_groups[gi]] if have_r else [float(sum(c) % 97) / 97.0 for c in grp]
        adv_rows += compute_group_relative_advantages([rs], advantage_eps)[0]
        sizes.append(len(grp))
        for ci, c in enumerate(grp):
            n = min(len(c), L)
            ids[i, :P] = torch.tensor(prompts[gi], dtype=torch.long) if P else ids[i, :P]
            ids[i, P:P + n] = torch.tensor(c[:n], dtype=torch.long)
            cmask[i, :n] = True
            rewards[i] = rs[ci]
            for src, dst in ((reference_logp_groups, ref), (rollout_logp_groups, old)):
                if src is not None and len(src) > gi and len(src[gi]) > ci and len(src[gi][ci]) >= n:
                    dst[i, :n] = torch.tensor([float(x) for x in src[gi][ci][:n]])
            i += 1
    adv = broadcast_sequence_advantages(torch.tensor(adv_rows), cmask)
    attn = torch.cat([torch.ones(B, P, dtype=torch.bool), cmask], 1)
    pmask = torch.cat([torch.ones(B, P, dtype=torch.bool), torch.zeros(B, L, dtype=torch.bool)], 1)
    dev = torch.device(device)
    md = {"num_prompts": len(groups), "samples_per_prompt": sizes[0] if len(set(sizes)) == 1 else None, "group_sizes": sizes, "batch_size": B,
          "prompt_len": P, "completion_len": L, "total_seq_len": P + L, "valid_tokens": int(cmask.sum()), "dtype": dtype, "device": str(dev),
          "reward_source": "payload_rewards" if have_r else "token_id_proxy",
          "reference_logp_source": "payload_reference_logps" if reference_logp_groups is not None else "zeros",
          "old_logp_source": "payload_rollout_logps" if rollout_logp_groups is not None else "zeros"}
    return SyntheticRLKernelBatch(ids.to(dev), attn.to(dev), pmask.to(dev), cmask.to(dev), ids[:, P:].contiguous().to(dev), rewards.to(dtype).to(dev),
                                  adv.to(dtype).to(dev), old.to(dtype).to(dev), ref.to(dtype).to(dev),
                                  cmask.reshape(-1).nonzero().squeeze(-1).to(dev), md)


def batch_from_rollout_or_synthetic(payload: Any, *, iteration: int = 0, num_prompts: int = 1, samples_per_prompt: int = 2, prompt_len: int = 4,
                                    completion_len: int = 8, vocab_size: int = 64, valid_density: float = 0.75, seed: int = 0,
                                    pad_token_id: int = 0, advantage_eps: float = 1e-6, dtype: torch.dtype = torch.float32,
                                    device: torch.device | str = "cpu"):
    """(batch, provenance).  A payload with grouped candidates becomes the batch (with whatever rewards, reference and
    rollout log-probs it carries); anything else -- a smoke run without a serving engine -- gets the synthetic batch of
    ``seed + iteration``, and the provenance says so."""
    try:
        cands = extract_rollout_candidate_groups(payload) if payload else []
    except TypeError:                            # not a grouped payload at all (e.g. an engine's status object)
        cands = []
    if cands:
        prompts = extract_rollout_token_groups(payload)

        def optional(reader):                    # the strict readers raise when a candidate lacks the field
            try:
                return reader(payload)
            except ValueError:
                return []

        rewards, refs = optional(extract_rollout_reward_groups), optional(extract_rollout_reference_logp_groups)
        flat = [c for grp in _groups(payload) for c in _candidates(grp)[1]]
        rl, k = [], 0
        for grp in cands:
            rl.append([candidate_rollout_logps(flat[k + j]) or [] for j in range(len(grp))])
            k += len(grp)
        have_rl = all(len(r) >= min(len(c), completion_len) and r for rg, cg in zip(rl, cands) for r, c in zip(rg, cg))
        have_ref = bool(refs) and [len(g) for g in refs] == [len(g) for g in cands] and \
            all(len(r) >= min(len(c), completion_len) for rg, cg in zip(refs, cands) for r, c in zip(rg, cg))
        same_prompt_len = bool(prompts) and len({len(p) for p in prompts}) == 1
        batch = batch_from_candidate_groups(cands, prompts if same_prompt_len else None, reward_groups=rewards or None,
                                            reference_logp_groups=refs if have_ref else None, rollout_logp_groups=rl if have_rl else None,
                                            completion_len=completion_len, pad_token_id=pad_token_id, advantage_eps=advantage_eps, dtype=dtype,
                                            device=device)
        toks = [c for grp in cands for c in grp]
        return batch, {"training_data_source": "rollout_payload", "reward_source": batch.metadata["reward_source"],
                       "reference_logp_source": batch.metadata["reference_logp_source"], "old_logp_source": batch.metadata["old_logp_source"],
                       "rollout_prompt_groups": len(cands), "rollout_sequences": len(toks), "rollout_tokens": sum(len(t) for t in toks)}
    from rl_kernel_b200.validation.common.rl_batch import make_synthetic_rl_kernel_batch

    batch = make_synthetic_rl_kernel_batch(num_prompts=num_prompts, samples_per_prompt=samples_per_prompt, prompt_len=prompt_len,
                                           completion_len=completion_len, vocab_size=vocab_size, valid_density=valid_density, dtype=dtype,
                                           device=device, seed=seed + int(iteration))
    return batch, {"training_data_source": "synthetic_fallback", "rollout_sequences": 0, "rollout_tokens": 0,
                   "reward_source": "synthetic_rewards", "reference_logp_source": "synthetic", "old_logp_source": "synthetic"}
