"""Weight audit between the trainer's parameters and the rollout engine's copy (parity: weight_audit.py of the reference's
dense experiment): after a publish, every tensor of the rollout copy must hold the trainer's bits."""
from __future__ import annotations

import hashlib

import torch


def tensor_digest(t: torch.Tensor) -> str:
    return hashlib.sha256(t.detach().contiguous().cpu().view(torch.uint8).numpy().tobytes()).hexdigest()


def audit_weights(policy: dict[str, torch.Tensor], rollout: dict[str, torch.Tensor]) -> dict:
    missing = sorted(set(policy) - set(rollout))
    extra = sorted(set(rollout) - set(policy))
    differing = [k for k in sorted(set(policy) & set(rollout))
                 if policy[k].shape != rollout[k].shape or policy[k].dtype != rollout[k].dtype or not torch.equal(policy[k], rollout[k])]
    return {"tensors": len(policy), "missing_in_rollout": missing, "unexpected_in_rollout": extra, "differing": differing,
            "in_sync": not (missing or extra or differing)}


def audit_trainer(trainer) -> dict:
    """Publish, then compare the two engines' parameter tables of a ``GRPOTrainer``."""
    trainer.publish_weights()
    torch.cuda.synchronize()
    return audit_weights(dict(trainer.engine.p.w), dict(trainer.rollout_engine.p.w))
