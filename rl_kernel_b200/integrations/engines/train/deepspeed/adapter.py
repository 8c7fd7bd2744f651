"""DeepSpeed-style training worker: wraps an engine object exposing ``backward`` / ``step`` and a
module, trains on a rollout with the strict log-prob + GRPO operators, and publishes a full
(ZeRO-gathered) state through the weight bridge (parity: DeepSpeedTrainingWorker,
rl_engine/integrations/engines/train/deepspeed/adapter.py:74-316)."""
from __future__ import annotations

import torch

from rl_kernel_b200.integrations.common.weights import WeightPublisher
from rl_kernel_b200.integrations.engines.train.contract import (RolloutBatchMixin, RolloutStageResult,
                                                                 TrainingStageResult)
from rl_kernel_b200.ops.loss import grpo_loss
from rl_kernel_b200.ops.logprob import linear_logp


def gather_zero3_parameter(param, group=None) -> torch.Tensor:
    """Assemble a ZeRO-3 partitioned parameter: every rank of ``group`` holds ``param.ds_tensor`` (a flat slice, the last
    one zero-padded); the whole is their concatenation in rank order cut to ``ds_numel`` and shaped ``ds_shape``.
    Without an initialised process group the local partition must already be the whole parameter."""
    import torch.distributed as dist

    part = param.ds_tensor.detach().reshape(-1)
    numel = int(getattr(param, "ds_numel", part.numel()))
    shape = tuple(getattr(param, "ds_shape", param.shape))
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        parts = [torch.empty_like(part) for _ in range(dist.get_world_size(group))]
        dist.all_gather(parts, part.contiguous(), group=group)
        flat = torch.cat(parts)
    else:
        flat = part
    if flat.numel() < numel:
        raise ValueError(f"partitions hold {flat.numel()} elements, the parameter has {numel}")
    return flat[:numel].reshape(shape).clone()


class DeepSpeedTrainingWorker(RolloutBatchMixin):
    def __init__(self, engine, publisher: WeightPublisher, *, hidden_fn=None, lm_head_name: str = "lm_head.weight",
                 clip_eps: float = 0.2, kl_coef: float = 0.0, temperature: float = 1.0, ref_scorer=None,
                 gather_context=None):
        self.engine, self.publisher = engine, publisher
        self.hidden_fn = hidden_fn or (lambda module, ids: module(ids))
        self.lm_head_name, self.clip_eps, self.kl_coef, self.temperature = lm_head_name, clip_eps, kl_coef, temperature
        self.ref_scorer, self.gather_context = ref_scorer, gather_context
        self.weight_version = 0

    def _lm_head(self):
        return dict(self.engine.module.named_parameters())[self.lm_head_name]

    def train(self, rollout: RolloutStageResult) -> TrainingStageResult:
        rollout.validate()
        P, R = rollout.prompt_len, rollout.rollout_logp.shape[1]
        hidden = self.hidden_fn(self.engine.module, rollout.tokens)            # [B, S, H]
        rows = hidden[:, P - 1:P - 1 + R]
        logp = linear_logp(rows, self._lm_head(), rollout.tokens[:, P:], self.temperature)
        ref = self.ref_scorer.score(rollout) if self.ref_scorer is not None and self.kl_coef > 0 else None
        adv = self.advantages(rollout)
        loss, pol, kl = grpo_loss(logp, rollout.rollout_logp, ref, adv, rollout.response_mask, clip_eps=self.clip_eps,
                                  beta=self.kl_coef)
        self.engine.backward(loss)
        self.engine.step()
        gn = getattr(self.engine, "get_global_grad_norm", lambda: 0.0)() or 0.0
        return TrainingStageResult(float(loss.detach()), float(pol.detach()), float(kl.detach()), float(gn), logp.detach(),
                                   self.mismatches(logp.detach(), rollout), int(rollout.response_mask.sum()),
                                   self.weight_version)

    def _full_state(self) -> dict[str, torch.Tensor]:
        """The whole model on every rank.  ZeRO-3 keeps only a 1 / dp flat partition of every parameter on a rank
        (``param.ds_tensor``; ``ds_shape`` / ``ds_numel`` describe the whole).  Order of preference: an injected
        ``gather_context`` (``deepspeed.zero.GatheredParameters``), else this worker's own rank-ordered all-gather of the
        partitions, else the state dict as it is (ZeRO stage 0-2: parameters are whole)."""
        module = self.engine.module
        params = dict(module.named_parameters())
        partitioned = {k: p for k, p in params.items() if hasattr(p, "ds_tensor")}
        if self.gather_context is not None:
            with self.gather_context(module.parameters()):
                return {k: v.detach().clone() for k, v in module.state_dict().items()}
        state = {k: v.detach().clone() for k, v in module.state_dict().items() if k not in partitioned}
        for name, p in partitioned.items():
            state[name] = gather_zero3_parameter(p, getattr(self.engine, "dp_process_group", None) or getattr(p, "ds_process_group", None))
        return state

    def publish_weights(self, weight_version: int):
        if weight_version <= self.weight_version and self.weight_version != 0:
            raise ValueError("weight_version must increase")
        self.weight_version = weight_version
        return self.publisher.publish(self._full_state(), weight_version, {"layout": {"kind": "full-state"}, "source": "deepspeed"})


# ------------------------------------------------------------------------------------------------ building the engine
# DeepSpeed is optional: nothing above imports it.  The helpers below load it on demand, resolve its config from a small
# set of arguments plus the caller's overrides, and read hidden states / logits out of whatever a wrapped model returns
# (parity: DeepSpeedTrainingConfig, _load_deepspeed, _resolved_deepspeed_config, _extract_hidden_states,
#  rl_engine/integrations/engines/train/deepspeed/adapter.py:37-127, 305-560).
import importlib  # noqa: E402
import os  # noqa: E402
import sysconfig  # noqa: E402
from collections.abc import Mapping  # noqa: E402
from dataclasses import dataclass, field  # noqa: E402
from pathlib import Path  # noqa: E402
from typing import Any  # noqa: E402


class DeepSpeedUnavailableError(RuntimeError):
    """The optional DeepSpeed runtime cannot be imported here."""


@dataclass(frozen=True)
class DeepSpeedTrainingConfig:
    micro_batch_size: int = 8
    gradient_accumulation_steps: int = 1
    zero_stage: int = 0
    dtype: torch.dtype = torch.bfloat16
    lr: float = 1e-6
    max_grad_norm: float = 1.0
    clip_eps: float = 0.2
    kl_coef: float = 0.0
    temperature: float = 1.0
    seed: int = 1234
    deepspeed_config: Mapping[str, Any] = field(default_factory=dict)        # merged over the resolved defaults
    initialize_kwargs: Mapping[str, Any] = field(default_factory=dict)

    def __post_init__(self) -> None:
        if self.zero_stage not in (0, 1, 2, 3):
            raise ValueError("zero_stage must be 0, 1, 2 or 3")
        if self.micro_batch_size < 1 or self.gradient_accumulation_steps < 1 or self.lr <= 0 or self.temperature <= 0:
            raise ValueError("micro_batch_size, gradient_accumulation_steps, lr and temperature must be positive")


def deep_merge(base: dict[str, Any], override: Mapping[str, Any]) -> dict[str, Any]:
    out = dict(base)
    for k, v in override.items():
        out[k] = deep_merge(dict(out[k]), v) if isinstance(v, Mapping) and isinstance(out.get(k), Mapping) else v
    return out


def resolved_deepspeed_config(cfg: DeepSpeedTrainingConfig) -> dict[str, Any]:
    """The JSON DeepSpeed gets.  Reduction of gradients in fp32 and no overlap of communication with the backward pass:
    a reduce that races with compute changes the order partial sums meet in."""
    base = {"train_micro_batch_size_per_gpu": cfg.micro_batch_size, "gradient_accumulation_steps": cfg.gradient_accumulation_steps,
            "gradient_clipping": cfg.max_grad_norm, "zero_optimization": {"stage": cfg.zero_stage, "overlap_comm": False,
                                                                          "contiguous_gradients": True, "reduce_scatter": True},
            "fp16": {"enabled": cfg.dtype == torch.float16}, "bf16": {"enabled": cfg.dtype == torch.bfloat16},
            "communication_data_type": "fp32", "optimizer": {"type": "AdamW", "params": {"lr": cfg.lr, "weight_decay": 0.0}}}
    return deep_merge(base, dict(cfg.deepspeed_config))


def resolved_zero_stage(config: Mapping[str, Any], *, fallback: int = 0) -> int:
    z = config.get("zero_optimization")
    if isinstance(z, Mapping):
        return int(z.get("stage", fallback))
    return 0 if z is False else int(fallback)


def cuda_home_candidates() -> list[Path]:
    """Toolkit roots DeepSpeed's op builder could use: NVIDIA wheels under site-packages (newest first), then torch's."""
    out: list[Path] = []
    for key in ("purelib", "platlib"):
        root = sysconfig.get_paths().get(key)
        if root and (Path(root) / "nvidia").is_dir():
            out += sorted((Path(root) / "nvidia").glob("cu*"), reverse=True)
    try:
        from torch.utils.cpp_extension import CUDA_HOME
    except Exception:  # noqa: BLE001
        CUDA_HOME = None
    if CUDA_HOME:
        out.append(Path(str(CUDA_HOME)))
    return list(dict.fromkeys(out))


def looks_like_cuda_home(path: Path) -> bool:
    return (path / "bin" / "nvcc").is_file() and (path / "include" / "cuda.h").is_file()


def configure_cuda_home(env: dict | None = None) -> str | None:
    """Point CUDA_HOME (and PATH / LD_LIBRARY_PATH) at a toolkit root when none is set; returns the root in use."""
    env = os.environ if env is None else env
    if env.get("CUDA_HOME"):
        return env["CUDA_HOME"]
    for c in cuda_home_candidates():
        if looks_like_cuda_home(c):
            env["CUDA_HOME"] = str(c)
            for key, sub in (("PATH", "bin"), ("LD_LIBRARY_PATH", "lib64"), ("LD_LIBRARY_PATH", "lib")):
                d = c / sub
                if d.is_dir() and str(d) not in env.get(key, "").split(os.pathsep):
                    env[key] = os.pathsep.join([str(d)] + ([env[key]] if env.get(key) else []))
            return str(c)
    return None


def load_deepspeed():
    configure_cuda_home()
    try:
        return importlib.import_module("deepspeed")
    except ImportError as exc:
        raise DeepSpeedUnavailableError("DeepSpeed is not installed; install a build that matches this Python / PyTorch / CUDA "
                                        "before constructing a DeepSpeed engine") from exc
    except Exception as exc:  # noqa: BLE001 - a broken install raises all sorts of things at import
        raise DeepSpeedUnavailableError("DeepSpeed is installed but failed to import here; if CUDA comes from Python wheels, CUDA_HOME "
                                        "must point at a root with bin/nvcc and include/cuda.h") from exc


def first_initialize_result(init_result: Any) -> Any:
    if isinstance(init_result, tuple):
        if not init_result:
            raise RuntimeError("deepspeed.initialize returned an empty tuple")
        return init_result[0]
    return init_result


def extract_logits(model_output: Any) -> torch.Tensor:
    if isinstance(model_output, torch.Tensor):
        return model_output
    if isinstance(model_output, Mapping) and "logits" in model_output:
        return model_output["logits"]
    if getattr(model_output, "logits", None) is not None:
        return model_output.logits
    if isinstance(model_output, (tuple, list)) and model_output:
        return extract_logits(model_output[0])
    raise TypeError(f"model output does not expose logits: {type(model_output)!r}")


def extract_hidden_states(model_output: Any, *, expected_hidden_dim: int | None = None) -> torch.Tensor:
    """The final hidden states [B, S, H] of a wrapped model's output: a tensor, ``last_hidden_state``, the last entry of
    ``hidden_states``, or the first fitting tensor of a tuple.  ``expected_hidden_dim`` rejects logits taken by mistake."""
    def fits(t: Any) -> bool:
        return isinstance(t, torch.Tensor) and t.dim() >= 2 and (expected_hidden_dim is None or t.shape[-1] == expected_hidden_dim)

    def get(o: Any, name: str) -> Any:
        return o.get(name) if isinstance(o, Mapping) else getattr(o, name, None)

    if fits(model_output):
        return model_output
    for name in ("last_hidden_state", "hidden", "final_hidden_states"):
        if fits(get(model_output, name)):
            return get(model_output, name)
    hs = get(model_output, "hidden_states")
    if isinstance(hs, (tuple, list)) and hs and fits(hs[-1]):
        return hs[-1]
    if isinstance(model_output, (tuple, list)):
        for item in model_output:
            if fits(item):
                return item
    raise TypeError(f"model output does not expose a hidden-state tensor"
                    f"{'' if expected_hidden_dim is None else f' of width {expected_hidden_dim}'}: {type(model_output)!r}")


def build_deepspeed_worker(model: torch.nn.Module, publisher: WeightPublisher, cfg: DeepSpeedTrainingConfig | None = None, *,
                           lm_head_name: str = "lm_head.weight", hidden_fn=None, ref_scorer=None, deepspeed_module=None
                           ) -> "DeepSpeedTrainingWorker":
    """``deepspeed.initialize`` around ``model`` with the resolved config, wrapped in the training worker.  With ZeRO-3
    the worker gathers partitioned parameters through ``deepspeed.zero.GatheredParameters``."""
    cfg = cfg or DeepSpeedTrainingConfig()
    ds = deepspeed_module or load_deepspeed()
    torch.manual_seed(cfg.seed)
    config = resolved_deepspeed_config(cfg)
    engine = first_initialize_result(ds.initialize(model=model, model_parameters=[p for p in model.parameters() if p.requires_grad],
                                                   config=config, **dict(cfg.initialize_kwargs)))
    gather = None
    if resolved_zero_stage(config, fallback=cfg.zero_stage) == 3 and hasattr(getattr(ds, "zero", None), "GatheredParameters"):
        gather = lambda params: ds.zero.GatheredParameters(list(params), modifier_rank=None)          # noqa: E731
    width = getattr(getattr(model, "config", None), "hidden_size", None)
    worker = DeepSpeedTrainingWorker(engine, publisher, hidden_fn=hidden_fn or (lambda m, ids: extract_hidden_states(m(ids), expected_hidden_dim=width)),
                                     lm_head_name=lm_head_name, clip_eps=cfg.clip_eps, kl_coef=cfg.kl_coef, temperature=cfg.temperature,
                                     ref_scorer=ref_scorer, gather_context=gather)
    worker.deepspeed_config = config
    return worker
